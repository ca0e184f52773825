"""Generates tests/golden/reference_einsum_linear.npz by running the REFERENCE's own C kernels
(oracle/_ref, compiled from its sources by oracle/build.py) on small seeded inputs:
`hodu_cpu_einsum_{f32,i32}` for the contraction forms that are matrix products, and
`hodu_cpu_dot_f32_fallback` followed by `hodu_cpu_add_f32` for a Linear layer with bias.
Needs the reference tree; the committed .npz is what the tests read.

    python tests/golden/make_golden_einsum_linear.py
"""
import ctypes
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
from hodu_b200.einsum import ParsedEinsum, einsum_metadata  # noqa: E402
from hodu_b200.layout import Layout  # noqa: E402
from hodu_b200.op_metadatas import dot_metadata  # noqa: E402
from oracle import oracle as O  # noqa: E402

HERE = os.path.dirname(os.path.abspath(__file__))

# (name, equation, layouts as (shape, strides or None, offset))
EINSUM_CASES = [
    ("mm", "ij,jk->ik", [((13, 21), None, 0), ((21, 9), None, 0)]),
    ("bmm", "bij,bjk->bik", [((3, 5, 8), None, 0), ((3, 8, 6), None, 0)]),
    ("nt", "ik,jk->ij", [((7, 12), None, 0), ((10, 12), None, 0)]),
    ("attn_scores", "bhqd,bhkd->bhqk", [((2, 3, 5, 8), None, 0), ((2, 3, 6, 8), None, 0)]),
    ("inner", "i,i->", [((33,), None, 0), ((33,), None, 0)]),
    ("outer", "i,j->ij", [((6,), None, 0), ((11,), None, 0)]),
    ("mm_out_t", "ij,jk->ki", [((13, 21), None, 0), ((21, 9), None, 0)]),
    ("merged_k", "bij,ijk->bk", [((4, 3, 5), None, 0), ((3, 5, 7), None, 0)]),
    ("merged_m", "abk,kn->abn", [((2, 6, 10), None, 0), ((10, 4), None, 0)]),
    ("strided", "ij,jk->ik", [((6, 10), (23, 2), 3), ((10, 4), (1, 12), 5)]),
    ("implicit", "ij,jk", [((4, 5), None, 0), ((5, 3), None, 0)]),
]


def layouts_of(spec):
    out = []
    for shape, strides, off in spec:
        out.append(Layout.from_shape(shape) if strides is None else Layout(tuple(shape), tuple(strides), off))
    return out


def storage_len(l: Layout) -> int:
    return l.offset + sum((n - 1) * s for n, s in zip(l.shape, l.strides)) + 1


def main():
    ref = O.ref()
    if ref is None or not hasattr(ref.base, "hodu_cpu_einsum_f32"):
        raise SystemExit("oracle/_ref (with ops_einsum.c) is missing and the reference tree is not mounted")
    rng = np.random.Generator(np.random.Philox(key=4321))
    cases = {}
    for name, eq, spec in EINSUM_CASES:
        ls = layouts_of(spec)
        parsed = ParsedEinsum.parse(eq, [l.shape for l in ls])
        out_l = Layout.from_shape(tuple(parsed.compute_output_shape()))
        md = einsum_metadata(parsed, ls, out_l)
        for dt_name, np_dt in (("f32", np.float32), ("i32", np.int32)):
            if np_dt == np.float32:
                ins = [rng.standard_normal(storage_len(l), dtype=np.float32) for l in ls]
            else:
                ins = [rng.integers(-127, 128, size=storage_len(l), dtype=np.int32) for l in ls]
            out = np.zeros(max(out_l.size(), 1), dtype=np_dt)
            ref.einsum(f"hodu_cpu_einsum_{dt_name}", ins, out, md)
            key = f"einsum_{name}_{dt_name}"
            cases[key + "__eq"] = np.array(eq)
            cases[key + "__md"] = np.array(md, dtype=np.int64)
            cases[key + "__in0"], cases[key + "__in1"] = ins
            cases[key + "__out"] = out

    # Linear with bias: x[M,K] . (w[N,K] seen as [K,N]) by the k-ordered f32 kernel, then the
    # broadcast add (binary wire format: [num_els, ndim, lhs_shape, rhs_shape, lhs_strides,
    # rhs_strides, lhs_off, rhs_off]).
    m, k, n = 17, 40, 11
    x = rng.standard_normal((m, k), dtype=np.float32)
    w = rng.standard_normal((n, k), dtype=np.float32)
    bias = rng.standard_normal((n,), dtype=np.float32)
    md = dot_metadata(Layout.from_shape((m, k)), Layout.from_shape((n, k)).transpose(0, 1))
    prod = np.zeros(m * n, dtype=np.float32)
    ref.call("hodu_cpu_dot_f32_fallback", x, w, prod, md)
    out = np.zeros(m * n, dtype=np.float32)
    bmd = [m * n, 2, m, n, m, n, n, 1, 0, 1, 0, 0]
    fn = getattr(ref.base, "hodu_cpu_add_f32")
    fn.restype = None
    fn(prod.ctypes.data_as(ctypes.c_void_p), bias.ctypes.data_as(ctypes.c_void_p),
       out.ctypes.data_as(ctypes.c_void_p), (ctypes.c_size_t * len(bmd))(*bmd))
    cases["linear_f32__x"], cases["linear_f32__w"], cases["linear_f32__bias"] = x, w, bias
    cases["linear_f32__out"] = out

    np.savez_compressed(os.path.join(HERE, "reference_einsum_linear.npz"), **cases)
    print("wrote", len(cases), "arrays")


if __name__ == "__main__":
    main()
