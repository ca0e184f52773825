"""ctypes binding of libhodu_b200.so (the C ABI declared in include/hodu_b200.h).

There is no fallback: if the library is missing or a call fails, an exception is
raised.  Nothing here computes on the CPU.
"""
from __future__ import annotations

import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
# HODU_B200_LIB points the binding at another build of the same library (A/B comparisons).
LIB_PATH = os.environ.get("HODU_B200_LIB") or os.path.join(_HERE, "lib", "libhodu_b200.so")

# Every symbol include/hodu_b200.h declares: name -> (restype, argtypes)
_vp, _sz, _u8, _u32, _i, _f = C.c_void_p, C.c_size_t, C.c_uint8, C.c_uint32, C.c_int, C.c_float
_szp = C.POINTER(C.c_size_t)
SIGNATURES = {
    "hodu_b200_init": (_i, [_i]),
    "hodu_b200_shutdown": (None, [_i]),
    "hodu_b200_matmul": (_i, [_i, _vp, _u8, _vp, _vp, _vp, _szp, _sz]),
    "hodu_b200_dot": (_i, [_i, _vp, _u8, _vp, _vp, _vp, _szp, _sz]),
    "hodu_b200_matmul_ex": (_i, [_i, _vp, _u8, _u8, _vp, _vp, _vp, _szp, _sz, _f, _f, _u32]),
    "hodu_b200_dot_ex": (_i, [_i, _vp, _u8, _u8, _vp, _vp, _vp, _szp, _sz, _f, _f, _u32]),
    "hodu_b200_cast": (_i, [_i, _vp, _u8, _u8, _vp, _vp, _szp, _sz]),
    "hodu_b200_contiguous": (_i, [_i, _vp, _u8, _vp, _vp, _szp, _sz]),
    "hodu_b200_swiglu": (_i, [_i, _vp, _u8, _vp, _vp, _vp, _vp, _szp, _sz, _u32]),
    "hodu_b200_linear": (_i, [_i, _vp, _u8, _vp, _vp, _vp, _vp, _szp, _sz, _u32]),
    "hodu_b200_einsum": (_i, [_i, _vp, _u8, C.POINTER(C.c_void_p), _sz, _vp, _szp, _sz]),
    "hodu_b200_conv2d": (_i, [_i, _vp, _u8, _vp, _vp, _vp, _szp, _sz]),
    "hodu_b200_matmul_host": (_i, [_i, _u8, _u8, _vp, _vp, _vp, _szp, _sz, _f, _f]),
    "hodu_b200_dot_host": (_i, [_i, _u8, _u8, _vp, _vp, _vp, _szp, _sz, _f, _f]),
    "hodu_b200_swiglu_mlp_host": (_i, [_i, _u8, _vp, _vp, _vp, _vp, _vp, _szp, _sz, _u32]),
    "hodu_b200_dot_f32_static": (_i, [_i, _vp, _vp, _vp, _vp, _szp, _sz]),
    "hodu_b200_dot_f32_static_status": (_i, [_i, C.POINTER(C.c_uint32)]),
    "hodu_b200_strerror": (C.c_char_p, [_i]),
    "hodu_b200_last_error_message": (C.c_char_p, []),
    "hodu_b200_last_status": (_i, [_i, C.POINTER(C.c_uint32)]),
    "hodu_b200_debug_wait_timeout": (_i, [_i, _vp, _u32]),
    "hodu_b200_force_path": (_i, [_i]),
    "hodu_b200_last_path": (_i, []),
    "hodu_b200_launch_count": (C.c_uint64, []),
    "hodu_b200_version": (_i, []),
}

PATH_AUTO, PATH_SIMT, PATH_TENSOR, PATH_TENSOR_1CTA, PATH_TENSOR_2CTA, PATH_TENSOR_2CTA_512 = 0, 1, 2, 3, 4, 5
SWIGLU_ROUND_EACH_OP, SWIGLU_ROUND_ONCE = 0, 1
LINEAR_ROUND_EACH_OP, LINEAR_ROUND_ONCE = 0, 1


class CudaKernelError(RuntimeError):
    """Mirror of `CudaKernelError` (crates/hodu_cuda_kernels/src/error.rs:7-18)."""

    def __init__(self, code: int, kind: str, message: str):
        super().__init__(f"{kind}: {message}" if message else kind)
        self.code = code
        self.kind = kind


_lib = None


def lib() -> C.CDLL:
    """Loads the library once; raises if it has not been built."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise ImportError(
                f"{LIB_PATH} is missing: build it with `python -m hodu_b200.build` "
                "(there is no CPU or PyTorch fallback)")
        handle = C.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(handle, name)  # AttributeError if the symbol is not exported
            fn.restype = res
            fn.argtypes = args
        _lib = handle
    return _lib


def check(code: int) -> None:
    if code != 0:
        l = lib()
        kind = l.hodu_b200_strerror(code).decode()
        msg = l.hodu_b200_last_error_message().decode()
        raise CudaKernelError(code, kind, msg)


def metadata_array(md) -> "C.Array":
    return (C.c_size_t * len(md))(*[int(x) for x in md])
