"""Host side of einsum: the equation parser and the wire format of the reference
(`ParsedEinsum::parse`, crates/hodu_core/src/einsum.rs:15-111; `einsum_metadata`,
crates/hodu_core/src/op_metadatas.rs:1502-1567).  Only parsing and shape algebra happen here;
the contraction itself runs in libhodu_b200.so (`hodu_b200_einsum`)."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Sequence

from .layout import Layout


@dataclass
class ParsedEinsum:
    input_subscripts: List[List[str]]
    output_subscripts: List[str]
    contraction_indices: List[str]
    all_indices: List[str]          # sorted; an index id is a position in this list
    index_sizes: Dict[str, int]

    @staticmethod
    def parse(equation: str, input_shapes: Sequence[Sequence[int]]) -> "ParsedEinsum":
        eq = equation.replace(" ", "")
        if "->" in eq:
            parts = eq.split("->")
            if len(parts) != 2:
                raise ValueError("einsum equation must have exactly one '->'")
            inputs_str, output_str = parts[0], parts[1]
        else:
            inputs_str, output_str = eq, None
        subs = [list(s) for s in inputs_str.split(",")]
        if len(subs) != len(input_shapes):
            raise ValueError(f"einsum equation has {len(subs)} operands but {len(input_shapes)} tensors provided")
        for i, (sub, shape) in enumerate(zip(subs, input_shapes)):
            if len(sub) != len(shape):
                raise ValueError(f"einsum operand {i} has {len(sub)} subscripts but tensor has {len(shape)} dimensions")
        sizes: Dict[str, int] = {}
        counts: Dict[str, int] = {}
        for sub, shape in zip(subs, input_shapes):
            for c, n in zip(sub, shape):
                if c in sizes and sizes[c] != n:
                    raise ValueError(f"einsum index '{c}' has inconsistent sizes: {sizes[c]} vs {n}")
                sizes.setdefault(c, int(n))
                counts[c] = counts.get(c, 0) + 1
        all_indices = sorted(sizes)
        if output_str is not None:
            out = list(output_str)
        else:  # implicit output: the indices that occur once, in sorted order
            out = [c for c in all_indices if counts[c] == 1]
        for c in out:
            if c not in sizes:
                raise ValueError(f"einsum output index '{c}' not found in any input")
        contraction = [c for c in all_indices if c not in set(out)]
        return ParsedEinsum(subs, out, contraction, all_indices, sizes)

    def compute_output_shape(self) -> List[int]:
        return [self.index_sizes[c] for c in self.output_subscripts]


def einsum_metadata(parsed: ParsedEinsum, input_layouts: Sequence[Layout], output_layout: Layout) -> List[int]:
    """[num_output_els, num_inputs, num_total_indices, num_contraction_indices, output_ndim,
    output_shape.., per input (ndim, shape.., strides.., offset, dim_to_index_id..),
    contraction_index_ids.., index_sizes.., output_index_ids..]"""
    ids = {c: i for i, c in enumerate(parsed.all_indices)}
    md = [max(output_layout.size(), 1), len(input_layouts), len(parsed.all_indices),
          len(parsed.contraction_indices), output_layout.ndim, *output_layout.shape]
    for sub, layout in zip(parsed.input_subscripts, input_layouts):
        md += [layout.ndim, *layout.shape, *layout.strides, layout.offset, *[ids[c] for c in sub]]
    md += [ids[c] for c in parsed.contraction_indices]
    md += [parsed.index_sizes[c] for c in parsed.all_indices]
    md += [ids[c] for c in parsed.output_subscripts]
    return [int(x) for x in md]
