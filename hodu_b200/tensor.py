"""Host-side mirror of the slice of `hodu_core::Tensor` that sits on the matmul
path: `matmul` / `dot` with the reference's rank dispatch and batch broadcasting
(crates/hodu_core/src/tensor/ops/matrix.rs:13-92,95-224,226-371), `transpose` as a
stride swap (tensor/ops/shape.rs:295-346), `to_dtype`
(tensor/ops/cast_memory.rs:11-38) and the CUDA storage dispatch underneath
(crates/hodu_core/src/be_cuda/storage/ops_matrix.rs:10-169, be_cuda/storage.rs:601-679).

Device memory and streams come from PyTorch (`torch.Tensor` is the `CudaSlice`
here); all arithmetic is done by libhodu_b200.so.  Forward only: no tape.
"""
from __future__ import annotations

from typing import Optional, Sequence

import torch

from . import kernels
from .dtype import DType, from_torch, to_torch
from .layout import Layout
from .op_metadatas import cast_metadata, dot_metadata, matmul_metadata


class HoduError(RuntimeError):
    pass


def _stream(device: torch.device) -> int:
    return torch.cuda.current_stream(device).cuda_stream


class Tensor:
    """A view (`Layout`) over a flat device buffer (`storage`, a 1-D torch tensor)."""

    def __init__(self, storage: torch.Tensor, layout: Layout):
        if storage.dim() != 1 or not storage.is_contiguous():
            raise HoduError("storage must be a flat contiguous buffer")
        if not storage.is_cuda:
            raise HoduError("this build only has the CUDA backend (Device::CUDA(n)); there is no CPU path")
        self.storage = storage
        self.layout = layout

    # ---- creation -------------------------------------------------------------------------
    @staticmethod
    def from_torch(t: torch.Tensor) -> "Tensor":
        """Wraps a contiguous CUDA tensor (no copy)."""
        if not t.is_contiguous():
            t = t.contiguous()
        return Tensor(t.reshape(-1), Layout.from_shape(tuple(t.shape)))

    def to_torch(self) -> torch.Tensor:
        """The viewed elements as a torch tensor sharing the storage (as_strided)."""
        return torch.as_strided(self.storage, self.layout.shape, self.layout.strides, self.layout.offset)

    # ---- properties -----------------------------------------------------------------------
    @property
    def shape(self):
        return self.layout.shape

    @property
    def dtype(self) -> DType:
        return from_torch(self.storage.dtype)

    @property
    def device_id(self) -> int:
        return self.storage.device.index or 0

    # ---- views ----------------------------------------------------------------------------
    def transpose(self, d0: int, d1: int) -> "Tensor":
        return Tensor(self.storage, self.layout.transpose(d0, d1))

    def broadcast(self, shape: Sequence[int]) -> "Tensor":
        return Tensor(self.storage, self.layout.broadcast_to(shape))

    def reshape(self, shape: Sequence[int]) -> "Tensor":
        return Tensor(self.storage, self.layout.reshape_contiguous(shape))

    # ---- matmul ---------------------------------------------------------------------------
    def matmul(self, other: "Tensor", out_dtype: Optional[DType] = None,
               scale_lhs: float = 1.0, scale_rhs: float = 1.0) -> "Tensor":
        """`Tensor::matmul` (matrix.rs:13-92).  `out_dtype` / scales are the mixed-dtype
        extension (f8e4m3 -> bf16, i8 -> i32); without them the result keeps the input dtype."""
        _validate_pair(self, other)
        ln, rn = len(self.shape), len(other.shape)
        if ln < 1 or rn < 1:
            raise HoduError(f"incompatible shapes {self.shape} x {other.shape}")
        if ln == 1 and rn == 1:
            raise HoduError("1-D x 1-D matmul is mul + sum_all in the reference; not on this path")
        if ln == 2 and rn == 1:
            if self.shape[1] != other.shape[0]:
                raise HoduError(f"incompatible shapes {self.shape} x {other.shape}")
            r = self.dot(other.reshape((other.shape[0], 1)), out_dtype, scale_lhs, scale_rhs)
            return r.reshape((self.shape[0],))
        if ln == 1 and rn == 2:
            if self.shape[0] != other.shape[0]:
                raise HoduError(f"incompatible shapes {self.shape} x {other.shape}")
            r = self.reshape((1, self.shape[0])).dot(other, out_dtype, scale_lhs, scale_rhs)
            return r.reshape((other.shape[1],))
        if ln == 2 and rn == 2:
            return self.dot(other, out_dtype, scale_lhs, scale_rhs)
        return self._matmul_batched(other, out_dtype, scale_lhs, scale_rhs)

    def dot(self, other: "Tensor", out_dtype: Optional[DType] = None,
            scale_lhs: float = 1.0, scale_rhs: float = 1.0) -> "Tensor":
        """`dot_2d` (matrix.rs:302-371) -> `call_ops_dot` (be_cuda/storage/ops_matrix.rs:95-169)."""
        _validate_pair(self, other)
        if len(self.shape) != 2 or len(other.shape) != 2 or self.shape[1] != other.shape[0]:
            raise HoduError(f"incompatible shapes {self.shape} x {other.shape}")
        m, n = self.shape[0], other.shape[1]
        md = dot_metadata(self.layout, other.layout)
        out = self._new_buffer(m * n, out_dtype)
        self._launch(other, out, md, out_dtype, scale_lhs, scale_rhs, is_dot=True)
        return Tensor(out, Layout.from_shape((m, n)))

    def _matmul_batched(self, other, out_dtype, scale_lhs, scale_rhs) -> "Tensor":
        lhs_dims, rhs_dims = self.shape, other.shape
        if len(lhs_dims) < 2 or len(rhs_dims) < 2 or lhs_dims[-1] != rhs_dims[-2]:
            raise HoduError(f"incompatible shapes {lhs_dims} x {rhs_dims}")
        lb, rb = lhs_dims[:-2], rhs_dims[:-2]
        nb = max(len(lb), len(rb))
        batch = []
        for i in range(nb):
            ld = lb[len(lb) - nb + i] if len(lb) - nb + i >= 0 else 1
            rd = rb[len(rb) - nb + i] if len(rb) - nb + i >= 0 else 1
            if ld != 1 and rd != 1 and ld != rd:
                raise HoduError(f"incompatible shapes {lhs_dims} x {rhs_dims}")
            batch.append(max(ld, rd))
        lhs_b = self.broadcast((*batch, lhs_dims[-2], lhs_dims[-1]))   # stride-0 views, matrix.rs:155-167
        rhs_b = other.broadcast((*batch, rhs_dims[-2], rhs_dims[-1]))
        out_layout = Layout.from_shape((*batch, lhs_dims[-2], rhs_dims[-1]))
        md = matmul_metadata(lhs_b.layout, rhs_b.layout, out_layout)
        out = self._new_buffer(out_layout.size(), out_dtype)
        lhs_b._launch(rhs_b, out, md, out_dtype, scale_lhs, scale_rhs, is_dot=False)
        return Tensor(out, out_layout)

    def _new_buffer(self, n: int, out_dtype: Optional[DType]) -> torch.Tensor:
        dt = to_torch(out_dtype) if out_dtype is not None else self.storage.dtype
        return torch.empty(n, dtype=dt, device=self.storage.device)  # uninitialised, like `new_buffer`

    def _launch(self, other, out, md, out_dtype, scale_lhs, scale_rhs, is_dot: bool) -> None:
        dev = self.device_id
        s = _stream(self.storage.device)
        if out_dtype is None and scale_lhs == 1.0 and scale_rhs == 1.0:
            fam = kernels.dot if is_dot else kernels.matmul
            call = kernels.call_ops_dot if is_dot else kernels.call_ops_matmul
            call(getattr(fam, str(self.dtype).upper()), dev, self.storage.data_ptr(),
                 other.storage.data_ptr(), out.data_ptr(), md, s)
        else:
            kernels.call_ops_matmul_ex(self.dtype, out_dtype if out_dtype is not None else self.dtype, dev,
                                       self.storage.data_ptr(), other.storage.data_ptr(), out.data_ptr(),
                                       md, scale_lhs, scale_rhs, s, is_dot=is_dot)

    def contiguous(self) -> "Tensor":
        """`CudaStorage::contiguous` (be_cuda/storage.rs:681-709): a dense copy of the view;
        the tensor itself when it already is contiguous."""
        if self.layout.is_contiguous() and self.layout.offset == 0 and self.storage.numel() == self.layout.size():
            return self
        out = torch.empty(self.layout.size(), dtype=self.storage.dtype, device=self.storage.device)
        k = getattr(kernels.contiguous, str(self.dtype).upper())
        kernels.call_ops_contiguous(k, self.device_id, self.storage.data_ptr(), out.data_ptr(),
                                    cast_metadata(self.layout), _stream(self.storage.device))
        return Tensor(out, Layout.from_shape(self.layout.shape))

    # ---- casts ----------------------------------------------------------------------------
    def to_dtype(self, dtype: DType) -> "Tensor":
        """`Tensor::to_dtype` -> `CudaStorage::to_dtype` -> `call_ops_cast`; output is contiguous."""
        dtype = DType(dtype)
        if dtype == self.dtype:
            return self
        out = torch.empty(self.layout.size(), dtype=to_torch(dtype), device=self.storage.device)
        k = getattr(kernels.cast, f"{str(self.dtype).upper()}_{str(dtype).upper()}")
        kernels.call_ops_cast(k, self.device_id, self.storage.data_ptr(), out.data_ptr(),
                              cast_metadata(self.layout), _stream(self.storage.device))
        return Tensor(out, Layout.from_shape(self.layout.shape))


def einsum(equation: str, tensors: Sequence[Tensor]) -> Tensor:
    """`Tensor::einsum` (crates/hodu_core/src/tensor/ops/einsum.rs:42-...) for the two-operand
    contractions that are matrix products ("ij,jk->ik", "bij,bjk->bik", "bhqd,bhkd->bhqk", ...).
    Other forms are the reference's own einsum kernel's business and raise `invalid kernel`."""
    from .einsum import ParsedEinsum, einsum_metadata
    if not tensors:
        raise HoduError("einsum requires at least one tensor")
    first = tensors[0]
    for t in tensors[1:]:
        _validate_pair(first, t)
    try:
        parsed = ParsedEinsum.parse(equation, [t.shape for t in tensors])
    except ValueError as e:
        raise HoduError(str(e)) from None
    out_layout = Layout.from_shape(tuple(parsed.compute_output_shape()))
    md = einsum_metadata(parsed, [t.layout for t in tensors], out_layout)
    out = first._new_buffer(max(out_layout.size(), 1), None)
    kernels.call_ops_einsum(getattr(kernels.einsum, str(first.dtype).upper()), first.device_id,
                            [t.storage.data_ptr() for t in tensors], out.data_ptr(), md,
                            _stream(first.storage.device))
    return Tensor(out, out_layout)


def matmul_vjp(a: Tensor, b: Tensor, grad_output: Tensor):
    """Vector-Jacobian products of `a.matmul(b)` as the reference computes them
    (crates/hodu_core/src/tensor/gradient/vjp_matrix.rs:17-66): dA = grad @ B^T and
    dB = A^T @ grad, both through transposed VIEWS (no copies), i.e. a K-contiguous rhs and an
    M-contiguous lhs for the kernels.  Operands whose batch dims were broadcast would need the
    reference's `sum_to_shape` reduction afterwards, which is not on this path: rejected."""
    if len(a.shape) < 2 or len(b.shape) < 2:
        raise HoduError("matmul_vjp takes operands of rank >= 2")
    grad_a = grad_output.matmul(b.transpose(-2, -1))
    grad_b = a.transpose(-2, -1).matmul(grad_output)
    if grad_a.shape != a.shape or grad_b.shape != b.shape:
        raise HoduError("broadcast batch dims need sum_to_shape, which is outside the matmul path")
    return grad_a, grad_b


def _validate_pair(a: Tensor, b: Tensor) -> None:
    if a.storage.device != b.storage.device:  # validate_same_device
        raise HoduError(f"device mismatch: {a.storage.device} vs {b.storage.device}")
    if a.storage.dtype != b.storage.dtype:    # validate_same_dtype
        raise HoduError(f"dtype mismatch: {a.dtype} vs {b.dtype}")
    if a.dtype == DType.BOOL:                 # validate_dtype_for_op (utils/valid.rs:259-264)
        raise HoduError("matmul does not take bool")
