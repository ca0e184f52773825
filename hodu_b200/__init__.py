"""hodu_b200: the matmul / dot / cast path of Hodu on B200 (sm_100a).

The product is libhodu_b200.so (C ABI: include/hodu_b200.h).  This package is the
host-side mirror of the reference interfaces around it, used by the tests and
the benchmark:

  kernels        the `hodu_cuda_kernels` launch wrappers (call_ops_matmul / dot / cast)
  op_metadatas   the metadata wire formats
  einsum         the einsum equation parser and its wire format
  layout, dtype  `Layout`, `DType`
  tensor         `Tensor::matmul` / `dot` / `transpose` / `to_dtype` (needs torch + CUDA)
  nn             `Linear`, SwiGLU MLP
  dist           row / batch sharding across ranks
"""
from . import _lib, dtype, kernels, layout, op_metadatas  # noqa: F401
from ._lib import CudaKernelError  # noqa: F401
from .dtype import DType  # noqa: F401
from .layout import Layout  # noqa: F401

__all__ = ["DType", "Layout", "CudaKernelError", "kernels", "op_metadatas", "layout", "dtype"]
