"""Callers and data formats either side of the matmul path: the backward products through
transposed views, the strided -> contiguous copy, the remaining CUDA cast pairs, and attention's
two batched matmuls (4-D, broadcast)."""
import numpy as np
import pytest
import torch

from gpu_util import DEV, from_dev, to_dev
from hodu_b200 import DType, Layout, _lib
from hodu_b200 import kernels as K
from hodu_b200.tensor import HoduError, Tensor, matmul_vjp
from oracle import oracle as O

pytestmark = pytest.mark.gpu


def t_bf16(x):
    return Tensor.from_torch(torch.from_numpy(np.ascontiguousarray(x)).to(DEV).to(torch.bfloat16))


def t_f32(x):
    return Tensor.from_torch(torch.from_numpy(np.ascontiguousarray(x)).to(DEV))


def f32(t: Tensor):
    return t.to_torch().float().cpu().numpy()


def bf(x):
    return O.widen(O.f32_to_bf16(x), O.BF16)


@pytest.mark.parametrize("shape_a,shape_b", [((256, 384), (384, 320)), ((3, 136, 200), (3, 200, 72))])
def test_matmul_backward_products_through_views(shape_a, shape_b):
    """dA = G . B^T and dB = A^T . G (tensor/gradient/vjp_matrix.rs:31-37,58-63)."""
    rng = np.random.default_rng(12)
    a = rng.standard_normal(shape_a).astype(np.float32)
    b = rng.standard_normal(shape_b).astype(np.float32)
    g = rng.standard_normal((*shape_a[:-1], shape_b[-1])).astype(np.float32)
    # bf16 on the tensor cores
    ga, gb = matmul_vjp(t_bf16(a), t_bf16(b), t_bf16(g))
    assert K.last_path() == _lib.PATH_TENSOR and K.last_status(0) == 0
    want_a = bf(np.matmul(bf(g), np.swapaxes(bf(b), -1, -2)))
    want_b = bf(np.matmul(np.swapaxes(bf(a), -1, -2), bf(g)))
    assert ga.shape == shape_a and gb.shape == shape_b
    assert O.rel_err(f32(ga), want_a) <= 1e-2 and O.rel_err(f32(gb), want_b) <= 1e-2
    # f32 (split-TF32 tensor path or the generic kernel, whichever the size selects)
    ga, gb = matmul_vjp(t_f32(a), t_f32(b), t_f32(g))
    assert O.rel_err(f32(ga), np.matmul(g, np.swapaxes(b, -1, -2))) <= 1e-4
    assert O.rel_err(f32(gb), np.matmul(np.swapaxes(a, -1, -2), g)) <= 1e-4
    if len(shape_a) == 3:  # a broadcast rhs would need sum_to_shape afterwards: rejected
        with pytest.raises(HoduError):
            matmul_vjp(t_f32(a), t_f32(b[:1]), t_f32(g))


def test_attention_shaped_batched_matmuls():
    """scores = Q . K^T-view and out = P . V, 4-D [batch, heads, seq, dim]
    (crates/hodu_nn/src/modules/attention.rs:37,69)."""
    rng = np.random.default_rng(13)
    q = rng.standard_normal((2, 4, 128, 64)).astype(np.float32)
    k = rng.standard_normal((2, 4, 160, 64)).astype(np.float32)
    v = rng.standard_normal((2, 4, 160, 64)).astype(np.float32)
    Q, Kt, V = t_bf16(q), t_bf16(k).transpose(-2, -1), t_bf16(v)
    scores = Q.matmul(Kt)
    assert scores.shape == (2, 4, 128, 160) and K.last_path() == _lib.PATH_TENSOR
    want = bf(np.matmul(bf(q), np.swapaxes(bf(k), -1, -2)))
    assert O.rel_err(f32(scores), want) <= 1e-2
    out = scores.matmul(V)
    assert out.shape == (2, 4, 128, 64)
    assert O.rel_err(f32(out), np.matmul(bf(f32(scores)), bf(v))) <= 1e-2
    # key/value shared across heads: broadcast over the head dim
    k1 = rng.standard_normal((2, 1, 160, 64)).astype(np.float32)
    s2 = Q.matmul(t_bf16(k1).transpose(-2, -1))
    assert O.rel_err(f32(s2), np.matmul(bf(q), np.swapaxes(bf(k1), -1, -2))) <= 1e-2


@pytest.mark.parametrize("tdt", [torch.uint8, torch.bfloat16, torch.float32, torch.float64, torch.int64])
def test_contiguous_copy_of_views(tdt):
    rng = np.random.default_rng(14)
    base = torch.from_numpy(rng.integers(0, 200, size=(6, 40, 72))).to(DEV).to(tdt)
    t = Tensor.from_torch(base)
    views = [t.transpose(-2, -1), t.transpose(0, 2), t.transpose(0, 1),
             Tensor(t.storage, Layout((5, 30, 50), (40 * 72, 72, 1), 72 + 3)),        # a window with an offset
             Tensor(t.storage, Layout((4, 40, 72), (0, 72, 1), 0))]                    # broadcast (stride 0)
    for v in views:
        c = v.contiguous()
        assert c.layout.is_contiguous() and c.shape == v.shape
        assert torch.equal(c.to_torch(), v.to_torch())
    assert t.contiguous() is t


def test_remaining_cuda_cast_pairs():
    rng = np.random.default_rng(15)
    x = (rng.standard_normal(100003) * 1000).astype(np.float32)
    x[:6] = [0.0, -0.0, 0.99, -0.99, 2147483520.0, -2147483648.0]
    t = t_f32(x)
    assert np.array_equal(t.to_dtype(DType.I32).to_torch().cpu().numpy(), np.trunc(x).astype(np.int32))   # toward zero
    assert np.array_equal(t.to_dtype(DType.F64).to_torch().cpu().numpy(), x.astype(np.float64))
    xi = rng.integers(-2 ** 31, 2 ** 31 - 1, size=50001).astype(np.int32)
    ti = Tensor.from_torch(torch.from_numpy(xi).to(DEV))
    assert np.array_equal(ti.to_dtype(DType.F32).to_torch().cpu().numpy(), xi.astype(np.float32))          # RNE
    xd = rng.standard_normal(50001) * 1e3
    td = Tensor.from_torch(torch.from_numpy(xd).to(DEV))
    assert np.array_equal(td.to_dtype(DType.F32).to_torch().cpu().numpy(), xd.astype(np.float32))
    assert np.array_equal(td.transpose(0, 0).to_dtype(DType.F32).to_torch().cpu().numpy(), xd.astype(np.float32))
