"""Mirror of the launch wrappers of the reference's `hodu_cuda_kernels` crate
(src/kernels/ops_matrix.rs:415-429,611-625; src/kernels/ops_cast.rs:27-64): same
names, same argument meaning, same error variants -- but every call goes to
libhodu_b200.so through its C ABI.

Operands are raw device pointers (ints).  `metadata` is the host list built by
`hodu_b200.op_metadatas`.  Calls only enqueue on `stream` (a CUstream handle as
int; 0 = the default stream).
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass
from typing import Optional, Sequence

from . import _lib
from ._lib import CudaKernelError, check, metadata_array
from .dtype import DType

_SUFFIX = {str(d): d for d in DType}


@dataclass(frozen=True)
class Kernel:
    """`Kernel(pub &'static str)`: "hodu_cuda_matmul_bf16", "hodu_cuda_cast_f32_to_bf16", ..."""
    name: str


class _Family:
    def __init__(self, op: str):
        self._op = op

    def __getattr__(self, dtype_upper: str) -> Kernel:  # matmul.BF16, dot.F32, cast.F32_BF16
        parts = dtype_upper.lower().split("_")
        if self._op == "cast":
            if len(parts) != 2:
                raise AttributeError(dtype_upper)
            return Kernel(f"hodu_cuda_cast_{parts[0]}_to_{parts[1]}")
        return Kernel(f"hodu_cuda_{self._op}_{dtype_upper.lower()}")


contiguous = _Family("contiguous")
matmul = _Family("matmul")
dot = _Family("dot")
cast = _Family("cast")
einsum = _Family("einsum")
conv2d = _Family("conv2d")


def _parse(kernel: Kernel, op: str):
    prefix = f"hodu_cuda_{op}_"
    if not kernel.name.startswith(prefix):
        raise CudaKernelError(-1, "invalid kernel", f"{kernel.name} is not a {op} kernel")
    rest = kernel.name[len(prefix):]
    try:
        if op == "cast":
            s, d = rest.split("_to_")
            return _SUFFIX[s], _SUFFIX[d]
        return _SUFFIX[rest]
    except (KeyError, ValueError):
        raise CudaKernelError(-1, "invalid kernel", f"unknown kernel {kernel.name}") from None


def call_ops_matmul(kernel: Kernel, device: int, lhs: int, rhs: int, output: int,
                    metadata: Sequence[int], stream: int = 0) -> None:
    dt = _parse(kernel, "matmul")
    md = metadata_array(metadata)
    check(_lib.lib().hodu_b200_matmul(device, stream, int(dt), lhs, rhs, output, md, len(metadata)))


def call_ops_dot(kernel: Kernel, device: int, lhs: int, rhs: int, output: int,
                 metadata: Sequence[int], stream: int = 0) -> None:
    dt = _parse(kernel, "dot")
    md = metadata_array(metadata)
    check(_lib.lib().hodu_b200_dot(device, stream, int(dt), lhs, rhs, output, md, len(metadata)))


def call_ops_cast(kernel: Kernel, device: int, input: int, output: int,
                  metadata: Sequence[int], stream: int = 0) -> None:
    src, dst = _parse(kernel, "cast")
    md = metadata_array(metadata)
    check(_lib.lib().hodu_b200_cast(device, stream, int(src), int(dst), input, output, md, len(metadata)))


def call_ops_contiguous(kernel: Kernel, device: int, input: int, output: int,
                        metadata: Sequence[int], stream: int = 0) -> None:
    """`call_ops_contiguous` (hodu_cuda_contiguous_{dtype}): strided -> contiguous copy."""
    dt = _parse(kernel, "contiguous")
    md = metadata_array(metadata)
    check(_lib.lib().hodu_b200_contiguous(device, stream, int(dt), input, output, md, len(metadata)))


# ---- extensions with no counterpart in the reference crate -------------------------------

def call_ops_matmul_ex(in_dtype: DType, out_dtype: DType, device: int, lhs: int, rhs: int, output: int,
                       metadata: Sequence[int], scale_lhs: float = 1.0, scale_rhs: float = 1.0,
                       stream: int = 0, is_dot: bool = False) -> None:
    md = metadata_array(metadata)
    fn = _lib.lib().hodu_b200_dot_ex if is_dot else _lib.lib().hodu_b200_matmul_ex
    check(fn(device, stream, int(in_dtype), int(out_dtype), lhs, rhs, output, md, len(metadata),
             scale_lhs, scale_rhs, 0))


def call_ops_swiglu(dtype: DType, device: int, x: int, w_gate: int, w_up: int, output: int,
                    metadata: Sequence[int], flags: int = _lib.SWIGLU_ROUND_EACH_OP, stream: int = 0) -> None:
    md = metadata_array(metadata)
    check(_lib.lib().hodu_b200_swiglu(device, stream, int(dtype), x, w_gate, w_up, output, md,
                                      len(metadata), flags))


def call_ops_linear(dtype: DType, device: int, x: int, w: int, bias: Optional[int], output: int,
                    metadata: Sequence[int], flags: int = _lib.LINEAR_ROUND_EACH_OP, stream: int = 0) -> None:
    """x . w + bias in one launch; `metadata` = matmul wire format + [bias_stride, bias_offset]."""
    md = metadata_array(metadata)
    check(_lib.lib().hodu_b200_linear(device, stream, int(dtype), x, w, bias, output, md, len(metadata), flags))


def call_ops_einsum(kernel: Kernel, device: int, inputs: Sequence[int], output: int,
                    metadata: Sequence[int], stream: int = 0) -> None:
    """`call_ops_einsum` (crates/hodu_cuda_kernels/src/kernels/ops_einsum.rs:24-70) for the
    two-operand contractions that are matrix products; other forms raise `invalid kernel`."""
    dt = _parse(kernel, "einsum")
    md = metadata_array(metadata)
    ptrs = (C.c_void_p * len(inputs))(*[int(p) for p in inputs])
    check(_lib.lib().hodu_b200_einsum(device, stream, int(dt), ptrs, len(inputs), output, md, len(metadata)))


def call_ops_conv(kernel: Kernel, device: int, input: int, weight: int, output: int,
                  metadata: Sequence[int], stream: int = 0) -> None:
    """`call_ops_conv` (crates/hodu_cuda_kernels/src/kernels/ops_conv.rs) for conv2d."""
    dt = _parse(kernel, "conv2d")
    md = metadata_array(metadata)
    check(_lib.lib().hodu_b200_conv2d(device, stream, int(dt), input, weight, output, md, len(metadata)))


def call_ops_matmul_host(in_dtype: DType, out_dtype: DType, device: int, lhs_host: int, rhs_host: int,
                         out_host: int, metadata: Sequence[int], scale_lhs: float = 1.0,
                         scale_rhs: float = 1.0, is_dot: bool = False) -> None:
    md = metadata_array(metadata)
    fn = _lib.lib().hodu_b200_dot_host if is_dot else _lib.lib().hodu_b200_matmul_host
    check(fn(device, int(in_dtype), int(out_dtype), lhs_host, rhs_host, out_host, md, len(metadata),
             scale_lhs, scale_rhs))


def call_ops_swiglu_mlp_host(dtype: DType, device: int, x_host: int, w_gate: int, w_up: int, w_down: int,
                             y_host: int, metadata: Sequence[int], flags: int = _lib.SWIGLU_ROUND_EACH_OP) -> None:
    """Host activations in, host result out, device-resident weights (`hodu_b200_swiglu_mlp_host`)."""
    md = metadata_array(metadata)
    check(_lib.lib().hodu_b200_swiglu_mlp_host(device, int(dtype), x_host, w_gate, w_up, w_down, y_host, md,
                                               len(metadata), flags))


def last_status(device: int) -> int:
    """Synchronises `device`, returns (and clears) its status word; raises if non-zero."""
    w = C.c_uint32(0)
    check(_lib.lib().hodu_b200_last_status(device, C.byref(w)))
    return w.value


def force_path(path: int) -> int:
    return _lib.lib().hodu_b200_force_path(path)


def last_path() -> int:
    return _lib.lib().hodu_b200_last_path()


def launch_count() -> int:
    return int(_lib.lib().hodu_b200_launch_count())
