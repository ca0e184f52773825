"""Builders of the flat `usize` metadata vectors the kernels take; same wire
formats as the reference (crates/hodu_core/src/op_metadatas.rs)."""
from __future__ import annotations

from typing import List

from .layout import Layout


def matmul_metadata(lhs: Layout, rhs: Layout, out: Layout) -> List[int]:
    """[num_els, lhs_ndim, rhs_ndim, batch_ndim, lhs_shape.., rhs_shape.., batch_shape..,
    lhs_strides.., rhs_strides.., lhs_off, rhs_off, M, K, N]  (op_metadatas.rs:192-290)."""
    ln, rn = lhs.ndim, rhs.ndim
    if ln < 2 or rn < 2:
        raise ValueError("matmul requires at least 2D tensors")
    m, k_l = lhs.shape[-2], lhs.shape[-1]
    k_r, n = rhs.shape[-2], rhs.shape[-1]
    if k_l != k_r:
        raise ValueError(f"matmul inner dimensions mismatch: {k_l} vs {k_r}")
    lb, rb = ln - 2, rn - 2
    bn = max(lb, rb)
    batch_shape = []
    for i in range(bn):
        li, ri = lb - bn + i, rb - bn + i
        ld = lhs.shape[li] if li >= 0 else 1
        rd = rhs.shape[ri] if ri >= 0 else 1
        if ld != rd and ld != 1 and rd != 1:
            raise ValueError(f"matmul batch dimension mismatch at index {i}: {ld} vs {rd}")
        batch_shape.append(max(ld, rd))
    md = [out.size(), ln, rn, bn]
    md += list(lhs.shape) + list(rhs.shape) + batch_shape
    md += list(lhs.strides) + list(rhs.strides)
    md += [lhs.offset, rhs.offset, m, k_l, n]
    return md


def dot_metadata(lhs: Layout, rhs: Layout) -> List[int]:
    """[M, K, N, lhs_stride_m, lhs_stride_k, rhs_stride_k, rhs_stride_n, lhs_off, rhs_off]
    (op_metadatas.rs:464-506)."""
    if lhs.ndim != 2 or rhs.ndim != 2:
        raise ValueError("dot requires 2D tensors")
    m, k = lhs.shape
    k2, n = rhs.shape
    if k != k2:
        raise ValueError(f"dot inner dimensions mismatch: {k} vs {k2}")
    return [m, k, n, lhs.strides[0], lhs.strides[1], rhs.strides[0], rhs.strides[1], lhs.offset, rhs.offset]


def cast_metadata(layout: Layout) -> List[int]:
    """[num_els, ndim, shape.., strides.., offset]  (op_metadatas.rs:1615-1640)."""
    return [layout.size(), layout.ndim, *layout.shape, *layout.strides, layout.offset]


def swiglu_metadata(x: Layout, w_gate: Layout, w_up: Layout) -> List[int]:
    """dot wire format with a second right-hand operand (see include/hodu_b200.h)."""
    if x.ndim != 2 or w_gate.ndim != 2 or w_up.ndim != 2:
        raise ValueError("swiglu requires 2D tensors")
    m, k = x.shape
    if w_gate.shape != w_up.shape or w_gate.shape[0] != k:
        raise ValueError(f"swiglu shape mismatch: x {x.shape}, gate {w_gate.shape}, up {w_up.shape}")
    n = w_gate.shape[1]
    return [m, k, n, x.strides[0], x.strides[1], w_gate.strides[0], w_gate.strides[1],
            w_up.strides[0], w_up.strides[1], x.offset, w_gate.offset, w_up.offset]


def conv2d_metadata(batch: int, in_channels: int, out_channels: int, in_hw, kernel_hw, stride=(1, 1),
                    padding=(0, 0), dilation=(1, 1), input_offset: int = 0, weight_offset: int = 0) -> List[int]:
    """[num_els, batch, in_channels, out_channels, in_h, in_w, kernel_h, kernel_w, out_h, out_w,
    stride_h, stride_w, padding_h, padding_w, dilation_h, dilation_w, input_offset, weight_offset]
    (op_metadatas.rs:1076-1123); the output extents follow from the others."""
    (h, w), (kh, kw), (sh, sw), (ph, pw), (dh, dw) = in_hw, kernel_hw, stride, padding, dilation
    oh = (h + 2 * ph - dh * (kh - 1) - 1) // sh + 1
    ow = (w + 2 * pw - dw * (kw - 1) - 1) // sw + 1
    if oh <= 0 or ow <= 0:
        raise ValueError("conv2d: kernel larger than the padded input")
    return [batch * out_channels * oh * ow, batch, in_channels, out_channels, h, w, kh, kw, oh, ow,
            sh, sw, ph, pw, dh, dw, input_offset, weight_offset]
