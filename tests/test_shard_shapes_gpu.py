"""The launches the multi-GPU split produces, and config 5 at its full launch shape.

With g GPUs, rank r owns rows [r*M/g, (r+1)*M/g) of A (configs 3, 4) or of the tokens
(config 5), or 16/g whole batches (config 2); B and the weights are whole on every rank.
Each per-rank launch has its own tile count and raster, so each is checked here as such:
the shard of the full-size seeded problem that rank would get, run on this one GPU.

Bars: i8 -> i32 bit-exact (sampled rows against a float64 product, which is exact for these
magnitudes, plus the checksum of every row); e4m3 -> bf16 within 6e-2 of the output scale;
bf16 within 1e-2."""
import numpy as np
import pytest
import torch

from gpu_util import DEV, from_dev, to_dev
from hodu_b200 import DType, Layout, _lib
from hodu_b200 import kernels as K
from hodu_b200 import synthetic as S
from hodu_b200.dist import shard_range
from hodu_b200.nn import Linear, SwiGluMlp
from hodu_b200.op_metadatas import dot_metadata, matmul_metadata
from hodu_b200.tensor import Tensor
from oracle import oracle as O

pytestmark = pytest.mark.gpu

# (world, rank): the last rank of each split, and one from the middle
SHARDS = [(2, 1), (4, 2), (8, 7), (8, 3)]


def device_dot(ta, tb, m, k, n, in_dt, out_dt, scales=(1.0, 1.0)):
    out = torch.empty(m * n, dtype={O.BF16: torch.int16, O.I32: torch.int32}[out_dt], device=DEV)
    md = dot_metadata(Layout.from_shape((m, k)), Layout.from_shape((k, n)))
    K.call_ops_matmul_ex(DType(in_dt), DType(out_dt), 0, ta.data_ptr(), tb.data_ptr(), out.data_ptr(), md,
                         scales[0], scales[1], 0, is_dot=True)
    assert K.last_status(0) == 0 and K.last_path() == _lib.PATH_TENSOR
    return out


@pytest.fixture(scope="module")
def config3():
    c = S.config3()
    a, b = O.f32_to_e4m3(c["a"]), O.f32_to_e4m3(c["b"])
    return a, b, to_dev(b), c["scale_a"], c["scale_b"]


@pytest.mark.parametrize("world,rank", SHARDS)
def test_config3_row_shards(config3, world, rank):
    a, b, tb, sa, sb = config3
    d = a.shape[0]
    lo, hi = shard_range(d, rank, world)
    m = hi - lo
    out = device_dot(to_dev(a[lo:hi]), tb, m, d, d, O.F8E4M3, O.BF16, (sa, sb))
    rows = np.random.default_rng(100 * world + rank).choice(m, 16, replace=False)
    rows = np.concatenate([rows, [0, m - 1]])   # the first and last row of the shard as well
    got = from_dev(out.view(m, d)[torch.from_numpy(rows).to(DEV)], O.BF16).reshape(len(rows), d)
    want = np.matmul(O.e4m3_to_f32(a[lo:hi][rows]), O.e4m3_to_f32(b)) * np.float32(sa * sb)
    want = O.widen(O.narrow(want.astype(np.float32), O.BF16), O.BF16)
    assert O.rel_err(O.widen(got, O.BF16), want) <= 6e-2


@pytest.fixture(scope="module")
def config4():
    c = S.config4()
    b64 = c["b"].astype(np.int64)
    return c["a"], c["b"], to_dev(c["b"]), b64.sum(axis=1)


@pytest.mark.parametrize("world,rank", SHARDS)
def test_config4_row_shards_exact(config4, world, rank):
    a, b, tb, b_row_sums = config4
    d = a.shape[0]
    lo, hi = shard_range(d, rank, world)
    m = hi - lo
    out = device_dot(to_dev(a[lo:hi]), tb, m, d, d, O.I8, O.I32)
    rows = np.random.default_rng(200 * world + rank).choice(m, 16, replace=False)
    rows = np.concatenate([rows, [0, m - 1]])
    got = from_dev(out.view(m, d)[torch.from_numpy(rows).to(DEV)], O.I32).reshape(len(rows), d)
    want = np.rint(np.matmul(a[lo:hi][rows].astype(np.float64), b.astype(np.float64))).astype(np.int64)
    assert np.array_equal(got.astype(np.int64), want)
    # checksum of every row of the shard: C @ 1 == A @ (B @ 1), exact in int64
    row_sums = out.view(m, d).sum(dim=1, dtype=torch.int64).cpu().numpy()
    assert np.array_equal(row_sums, a[lo:hi].astype(np.int64) @ b_row_sums)


@pytest.mark.parametrize("world,rank", [(2, 1), (4, 3), (8, 5)])
def test_config2_batch_shards(world, rank):
    c = S.config2()
    lo, hi = shard_range(16, rank, world)
    a, b = O.f32_to_bf16(c["a"][lo:hi]), O.f32_to_bf16(c["b"][lo:hi])
    lay = Layout.from_shape(a.shape)
    md = matmul_metadata(lay, lay, lay)
    ta, tb = to_dev(a), to_dev(b)
    out = torch.empty(lay.size(), dtype=torch.int16, device=DEV)
    K.call_ops_matmul(K.matmul.BF16, 0, ta.data_ptr(), tb.data_ptr(), out.data_ptr(), md, 0)
    assert K.last_status(0) == 0 and K.last_path() == _lib.PATH_TENSOR
    got = O.widen(from_dev(out, O.BF16), O.BF16)
    want = O.widen(O.matmul(a, b, md, O.BF16), O.BF16)
    assert O.rel_err(got, want) <= 1e-2


@pytest.fixture(scope="module")
def config5():
    c = S.config5()
    xb = O.f32_to_bf16(c["x"])
    # hodu_nn::Linear stores its weight as [out_features, in_features]
    wg, wu, wd = (O.f32_to_bf16(np.ascontiguousarray(c[k].T)) for k in ("w_gate", "w_up", "w_down"))
    dev = lambda bits: Tensor(to_dev(bits).view(torch.bfloat16), Layout.from_shape(bits.shape))
    mlp = SwiGluMlp(Linear(dev(wg)), Linear(dev(wu)), Linear(dev(wd)))
    widened = tuple(O.widen(w, O.BF16).T for w in (wg, wu, wd))
    return xb, mlp, widened


def check_mlp_tokens(xb, mlp, widened, lo, hi, n_sample, seed):
    """Runs tokens [lo, hi) through SwiGluMlp.forward as one call and checks sampled tokens
    against both rounding forms of the oracle composition."""
    m = hi - lo
    x_t = Tensor(to_dev(xb[lo:hi]).view(torch.bfloat16), Layout.from_shape((m, xb.shape[1])))
    y = mlp.forward(x_t)
    assert K.last_status(0) == 0 and K.last_path() == _lib.PATH_TENSOR
    rows = np.random.default_rng(seed).choice(m, n_sample, replace=False)
    rows = np.concatenate([rows, [0, m - 1]])
    picked = y.storage.view(torch.int16).view(m, -1)[torch.from_numpy(rows).to(DEV)]
    got = O.widen(from_dev(picked, O.BF16), O.BF16).reshape(len(rows), -1)
    gf, uf, df = widened
    xf = O.widen(xb[lo:hi][rows], O.BF16)
    for each_op in (True, False):   # the reference's op-by-op roundings, and a single rounding
        h = O.widen(O.swiglu_hidden(xf, gf, uf, O.BF16, round_each_op=each_op), O.BF16)
        want = O.widen(O.narrow(np.matmul(h, df).astype(np.float32), O.BF16), O.BF16)
        assert O.rel_err(got, want) <= 1e-2


def test_config5_full_launch_sampled_tokens(config5):
    """All 16384 tokens in one forward: the launch shape the benchmark times (3584 SwiGLU tiles,
    then the K = 14336 down projection)."""
    xb, mlp, widened = config5
    check_mlp_tokens(xb, mlp, widened, 0, xb.shape[0], 64, 5)


@pytest.mark.parametrize("world,rank", [(2, 1), (4, 2), (8, 7)])
def test_config5_token_shards(config5, world, rank):
    xb, mlp, widened = config5
    lo, hi = shard_range(xb.shape[0], rank, world)
    check_mlp_tokens(xb, mlp, widened, lo, hi, 32, 300 * world + rank)
