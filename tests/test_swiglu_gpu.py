"""Fused gate/up/silu/mul kernel and the SwiGLU MLP built from Linear layers (config 5)."""
import numpy as np
import pytest
import torch

from gpu_util import DEV, canary_intact, from_dev, new_out, to_dev
from hodu_b200 import DType, Layout, _lib
from hodu_b200 import kernels as K
from hodu_b200 import synthetic as S
from hodu_b200.nn import Linear, SwiGluMlp
from hodu_b200.op_metadatas import swiglu_metadata
from hodu_b200.tensor import Tensor
from oracle import oracle as O

pytestmark = pytest.mark.gpu


def run_swiglu(x, wg, wu, lx, lg, lu, dt, flags, path):
    tx, tg, tu = to_dev(x), to_dev(wg), to_dev(wu)
    m, n = lx.shape[0], lg.shape[1]
    out = new_out(m * n, dt)
    prev = K.force_path(path)
    try:
        K.call_ops_swiglu(DType(dt), 0, tx.data_ptr(), tg.data_ptr(), tu.data_ptr(), out.data_ptr(),
                          swiglu_metadata(lx, lg, lu), flags, 0)
        taken = K.last_path()
    finally:
        K.force_path(prev)
    want_path = _lib.PATH_SIMT if path == _lib.PATH_SIMT else _lib.PATH_TENSOR
    assert K.last_status(0) == 0 and canary_intact(out, m * n) and taken == want_path
    return from_dev(out[: m * n], dt)


@pytest.mark.parametrize("dt", [O.BF16, O.F16])
@pytest.mark.parametrize("weights_as_linear", [True, False])
@pytest.mark.parametrize("flags", [_lib.SWIGLU_ROUND_EACH_OP, _lib.SWIGLU_ROUND_ONCE])
def test_fused_hidden_matches_oracle(dt, weights_as_linear, flags):
    rng = np.random.default_rng(dt + flags)
    for (m, k, n) in [(128, 64, 128), (200, 264, 328), (384, 512, 1024)]:
        x = rng.standard_normal((m, k)).astype(np.float32)
        wg = (rng.standard_normal((k, n)) * 0.1).astype(np.float32)
        wu = (rng.standard_normal((k, n)) * 0.1).astype(np.float32)
        xb, gb, ub = O.narrow(x, dt), O.narrow(wg, dt), O.narrow(wu, dt)
        lx = Layout.from_shape((m, k))
        if weights_as_linear:  # stored [N,K], passed as a transposed view (hodu_nn::Linear)
            gs, us = np.ascontiguousarray(gb.T), np.ascontiguousarray(ub.T)
            lg = lu = Layout.from_shape((n, k)).transpose(0, 1)
        else:
            gs, us = gb, ub
            lg = lu = Layout.from_shape((k, n))
        want = O.swiglu_hidden(O.widen(xb, dt), O.widen(gb, dt), O.widen(ub, dt), dt,
                               round_each_op=(flags == _lib.SWIGLU_ROUND_EACH_OP))
        wf = O.widen(want, dt).reshape(-1)
        for path in (_lib.PATH_TENSOR_1CTA, _lib.PATH_TENSOR_2CTA, _lib.PATH_TENSOR_2CTA_512, _lib.PATH_SIMT):
            got = run_swiglu(xb, gs, us, lx, lg, lu, dt, flags, path)
            assert O.rel_err(O.widen(got, dt), wf) <= 1e-2


def test_config5_mlp_reduced_and_full_sampled_tokens():
    for scale, tokens in ((8, 16384), (1, 256)):
        c = S.config5(scale=scale, tokens=tokens)
        xb = O.f32_to_bf16(c["x"])
        # Linear stores weight as [out_features, in_features]
        wg, wu, wd = (O.f32_to_bf16(np.ascontiguousarray(c[k].T)) for k in ("w_gate", "w_up", "w_down"))
        dev = lambda bits, shape: Tensor(to_dev(bits).view(torch.bfloat16), Layout.from_shape(shape))
        x_t = dev(xb, xb.shape)
        mlp = SwiGluMlp(Linear(dev(wg, wg.shape)), Linear(dev(wu, wu.shape)), Linear(dev(wd, wd.shape)))
        y = mlp.forward(x_t)
        assert K.last_status(0) == 0 and K.last_path() == _lib.PATH_TENSOR
        got = O.widen(from_dev(y.storage.view(torch.int16), O.BF16), O.BF16).reshape(y.shape)
        xf = O.widen(xb, O.BF16)
        gf, uf, df = (O.widen(w, O.BF16).T for w in (wg, wu, wd))
        # reference composition: every op output rounded to bf16
        h = O.widen(O.swiglu_hidden(xf, gf, uf, O.BF16, round_each_op=True), O.BF16)
        want = O.widen(O.narrow(np.matmul(h, df).astype(np.float32), O.BF16), O.BF16)
        assert O.rel_err(got, want) <= 1e-2
        # single-rounding form, for information: also inside the bar
        h1 = O.widen(O.swiglu_hidden(xf, gf, uf, O.BF16, round_each_op=False), O.BF16)
        want1 = O.widen(O.narrow(np.matmul(h1, df).astype(np.float32), O.BF16), O.BF16)
        assert O.rel_err(got, want1) <= 1e-2
