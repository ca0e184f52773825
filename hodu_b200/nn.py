"""`hodu_nn::Linear` (crates/hodu_nn/src/modules/linear.rs:38-47) and the SwiGLU MLP
a caller composes from three of them.  The reference has no SwiGLU module: the
composition is `down(silu(gate(x)) * up(x))`, five launches and three [M, hidden]
temporaries there; here gate, up, silu and mul are one kernel."""
from __future__ import annotations

from typing import Optional

import torch

from . import _lib, kernels
from .layout import Layout
from .op_metadatas import matmul_metadata, swiglu_metadata
from .tensor import HoduError, Tensor, _stream


class Linear:
    """weight is [out_features, in_features], bias [out_features] or None;
    forward = input.matmul(weight.transpose(-2,-1)) (+ bias), as one launch."""

    def __init__(self, weight: Tensor, bias: Optional[Tensor] = None, rounding: int = _lib.LINEAR_ROUND_EACH_OP):
        if len(weight.shape) != 2:
            raise HoduError("Linear weight must be 2-D [out, in]")
        if bias is not None:
            if tuple(bias.shape) != (weight.shape[0],):
                raise HoduError(f"Linear bias must be [{weight.shape[0]}], got {tuple(bias.shape)}")
            if bias.dtype != weight.dtype:
                raise HoduError("Linear bias and weight must have the same dtype")
        self.weight, self.bias, self.rounding = weight, bias, rounding

    def forward(self, input: Tensor) -> Tensor:
        wt = self.weight.transpose(-2, -1)
        if self.bias is None:
            return input.matmul(wt)
        if len(input.shape) < 2 or input.shape[-1] != wt.shape[0]:
            raise HoduError(f"incompatible shapes {input.shape} x {wt.shape}")
        if input.dtype != self.weight.dtype:
            raise HoduError("Linear input and weight must have the same dtype")
        batch = tuple(input.shape[:-2])
        out_layout = Layout.from_shape((*batch, input.shape[-2], wt.shape[1]))
        rhs = wt.broadcast((*batch, *wt.shape)) if batch else wt
        md = matmul_metadata(input.layout, rhs.layout, out_layout)
        md = [*md, self.bias.layout.strides[0], self.bias.layout.offset]
        out = torch.empty(out_layout.size(), dtype=input.storage.dtype, device=input.storage.device)
        kernels.call_ops_linear(input.dtype, input.device_id, input.storage.data_ptr(), wt.storage.data_ptr(),
                                self.bias.storage.data_ptr(), out.data_ptr(), md, self.rounding,
                                _stream(input.storage.device))
        return Tensor(out, out_layout)


class SwiGluMlp:
    """Y = down(silu(gate(X)) * up(X)) from three bias-free `Linear` layers."""

    def __init__(self, gate: Linear, up: Linear, down: Linear, rounding: int = _lib.SWIGLU_ROUND_EACH_OP):
        self.gate, self.up, self.down, self.rounding = gate, up, down, rounding

    def hidden(self, x: Tensor) -> Tensor:
        """silu(x.gate) * x.up as one launch (`hodu_b200_swiglu`)."""
        if len(x.shape) != 2:
            raise HoduError("SwiGluMlp takes a 2-D [tokens, features] input")
        wg = self.gate.weight.transpose(-2, -1)
        wu = self.up.weight.transpose(-2, -1)
        md = swiglu_metadata(x.layout, wg.layout, wu.layout)
        m, n = x.shape[0], wg.shape[1]
        out = torch.empty(m * n, dtype=x.storage.dtype, device=x.storage.device)
        kernels.call_ops_swiglu(x.dtype, x.device_id, x.storage.data_ptr(), wg.storage.data_ptr(),
                                wu.storage.data_ptr(), out.data_ptr(), md, self.rounding,
                                _stream(x.storage.device))
        return Tensor(out, Layout.from_shape((m, n)))

    def forward(self, x: Tensor) -> Tensor:
        return self.down.forward(self.hidden(x))

    def forward_host(self, x_host_ptr: int, y_host_ptr: int, tokens: int) -> None:
        """The same forward for activations that live in HOST memory (pinned for full copy speed):
        `x_host_ptr` -> [tokens, in_features] in, `y_host_ptr` -> [tokens, out_features] out, both
        contiguous and of the weights' dtype.  Row blocks of tokens are uploaded, multiplied and
        downloaded as one pipelined call; the weights stay on the device.  Returns when the result
        is complete in host memory."""
        g, u, d = self.gate.weight, self.up.weight, self.down.weight
        if any(l.bias is not None for l in (self.gate, self.up, self.down)):
            raise HoduError("forward_host takes bias-free layers")
        gt, ut, dt = (w.transpose(-2, -1) for w in (g, u, d))
        if not (gt.shape == ut.shape and gt.shape[1] == dt.shape[0]):
            raise HoduError(f"incompatible layer shapes {g.shape}, {u.shape}, {d.shape}")
        md = [tokens, gt.shape[0], gt.shape[1], dt.shape[1],
              gt.layout.strides[0], gt.layout.strides[1], ut.layout.strides[0], ut.layout.strides[1],
              dt.layout.strides[0], dt.layout.strides[1], gt.layout.offset, ut.layout.offset, dt.layout.offset]
        kernels.call_ops_swiglu_mlp_host(g.dtype, g.device_id, x_host_ptr, g.storage.data_ptr(), u.storage.data_ptr(),
                                         d.storage.data_ptr(), y_host_ptr, md, self.rounding)
