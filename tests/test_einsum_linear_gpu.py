"""GPU parity of the two widened rows: einsum contractions routed to the GEMM
(`hodu_b200_einsum`) and `Linear` with its bias fused into the epilogue (`hodu_b200_linear`),
both through the C ABI, against the oracle and the golden outputs of the reference's C kernels."""
import os

import numpy as np
import pytest
import torch

from hodu_b200 import DType, Layout, kernels as K
from hodu_b200.einsum import ParsedEinsum, einsum_metadata
from hodu_b200.nn import Linear
from hodu_b200.op_metadatas import matmul_metadata
from hodu_b200.tensor import Tensor, einsum
from oracle import oracle as O
from tests.gpu_util import DEV, canary_intact, from_dev, new_out, to_dev

pytestmark = pytest.mark.gpu
GOLDEN_EL = np.load(os.path.join(os.path.dirname(__file__), "golden", "reference_einsum_linear.npz"))
TOL = {O.F32: 1e-4, O.BF16: 1e-2, O.F16: 1e-2}


def run_einsum(ins_bits, md, dt, path=K._lib.PATH_AUTO):
    n_out = int(md[0])
    out = new_out(n_out, dt)
    devs = [to_dev(b) for b in ins_bits]
    prev = K.force_path(path)
    try:
        K.call_ops_einsum(getattr(K.einsum, str(DType(dt)).upper()), 0, [d.data_ptr() for d in devs],
                          out.data_ptr(), md, 0)
        taken = K.last_path()
    finally:
        K.force_path(prev)
    assert K.last_status(0) == 0
    assert canary_intact(out, n_out)
    return from_dev(out[:n_out], dt), taken


EINSUM_GOLDEN = sorted({k.split("__")[0] for k in GOLDEN_EL.files if k.startswith("einsum_")})


@pytest.mark.parametrize("key", EINSUM_GOLDEN)
def test_einsum_golden_reference_outputs(key):
    md = [int(v) for v in GOLDEN_EL[key + "__md"]]
    ins = [GOLDEN_EL[key + "__in0"], GOLDEN_EL[key + "__in1"]]
    want = GOLDEN_EL[key + "__out"]
    if key.endswith("_i32"):
        got, _ = run_einsum(ins, md, O.I32)
        assert np.array_equal(got, want)
    else:
        got, _ = run_einsum(ins, md, O.F32)
        assert O.rel_err(got, want) <= 1e-5


def _storage_len(l: Layout) -> int:
    return l.offset + sum((n - 1) * s for n, s in zip(l.shape, l.strides)) + 1


BIG = [
    # equation, layouts (shape, strides|None, offset), dtype, forced path
    ("ij,jk->ik", [((384, 512), None, 0), ((512, 256), None, 0)], O.BF16, K._lib.PATH_TENSOR),
    ("ik,jk->ij", [((384, 512), None, 0), ((256, 512), None, 0)], O.BF16, K._lib.PATH_TENSOR),
    ("ij,jk->ki", [((384, 512), None, 0), ((512, 256), None, 0)], O.F16, K._lib.PATH_TENSOR),
    ("bij,bjk->bik", [((3, 256, 320), None, 0), ((3, 320, 128), None, 0)], O.BF16, K._lib.PATH_TENSOR),
    ("bhqd,bhkd->bhqk", [((2, 4, 256, 64), None, 0), ((2, 4, 384, 64), None, 0)], O.BF16, K._lib.PATH_TENSOR),
    ("bhqk,bhkd->bhqd", [((2, 4, 256, 384), None, 0), ((2, 4, 384, 64), None, 0)], O.F16, K._lib.PATH_TENSOR),
    ("abk,kn->abn", [((4, 96, 256), None, 0), ((256, 192), None, 0)], O.BF16, K._lib.PATH_TENSOR),
    ("bij,ijk->bk", [((256, 16, 32), None, 0), ((16, 32, 128), None, 0)], O.BF16, K._lib.PATH_TENSOR),
    ("ij,jk->ik", [((300, 520), (1048, 2), 3), ((520, 200), (1, 536), 8)], O.BF16, K._lib.PATH_AUTO),
    ("ij,jk->ik", [((512, 1024), None, 0), ((1024, 768), None, 0)], O.F32, K._lib.PATH_AUTO),
    ("bqd,bkd->bqk", [((6, 200, 72), None, 0), ((6, 136, 72), None, 0)], O.F32, K._lib.PATH_AUTO),
    ("i,i->", [((100000,), None, 0), ((100000,), None, 0)], O.F32, K._lib.PATH_AUTO),
    ("i,j->ij", [((700,), None, 0), ((900,), None, 0)], O.BF16, K._lib.PATH_AUTO),
    ("ij,jk->ik", [((64, 4096), None, 0), ((4096, 96), None, 0)], O.I8, K._lib.PATH_AUTO),
]


@pytest.mark.parametrize("case", BIG, ids=[f"{c[0]}-{DType(c[2])}-{i}" for i, c in enumerate(BIG)])
def test_einsum_vs_oracle(case):
    eq, spec, dt, path = case
    ls = [Layout.from_shape(s) if st is None else Layout(tuple(s), tuple(st), off) for s, st, off in spec]
    parsed = ParsedEinsum.parse(eq, [l.shape for l in ls])
    ol = Layout.from_shape(tuple(parsed.compute_output_shape()))
    md = einsum_metadata(parsed, ls, ol)
    import zlib
    rng = np.random.default_rng(zlib.crc32(eq.encode()) % 1000 + int(dt))   # the same data in every run
    if dt == O.I8:
        ins = [rng.integers(-127, 128, size=_storage_len(l), dtype=np.int8) for l in ls]
    else:
        # a single-element output (inner product) is kept well conditioned: all terms positive
        gen = (lambda n: np.abs(rng.standard_normal(n))) if ol.size() <= 1 else rng.standard_normal
        ins = [O.narrow(gen(_storage_len(l)).astype(np.float32), dt) for l in ls]
    got, taken = run_einsum(ins, md, dt, path)
    want = O.einsum(ins, md, dt)
    if dt == O.I8:
        assert np.array_equal(got, want)
    else:
        assert O.rel_err(O.widen(got, dt), O.widen(want, dt)) <= TOL[dt]
    if path == K._lib.PATH_TENSOR:
        assert taken == K._lib.PATH_TENSOR


def test_einsum_tensor_api_matches_matmul():
    rng = np.random.default_rng(3)
    a = torch.from_numpy(rng.standard_normal((2, 128, 256)).astype(np.float32)).to(DEV).bfloat16()
    b = torch.from_numpy(rng.standard_normal((2, 256, 64)).astype(np.float32)).to(DEV).bfloat16()
    ta, tb = Tensor.from_torch(a), Tensor.from_torch(b)
    c1 = einsum("bij,bjk->bik", [ta, tb]).to_torch()
    c2 = ta.matmul(tb).to_torch()
    assert c1.shape == (2, 128, 64)
    assert torch.equal(c1, c2)   # same kernel, same views
    # Q.K^T through einsum == through the transposed view
    q = torch.from_numpy(rng.standard_normal((2, 4, 128, 64)).astype(np.float32)).to(DEV).bfloat16()
    k = torch.from_numpy(rng.standard_normal((2, 4, 192, 64)).astype(np.float32)).to(DEV).bfloat16()
    s1 = einsum("bhqd,bhkd->bhqk", [Tensor.from_torch(q), Tensor.from_torch(k)]).to_torch()
    s2 = Tensor.from_torch(q).matmul(Tensor.from_torch(k).transpose(-2, -1)).to_torch()
    assert torch.equal(s1, s2)


# ------------------------------------------------------------------------------- Linear + bias
def run_linear(x_bits, w_bits, b_bits, x_l: Layout, w_l: Layout, b_l: Layout, dt, flags, path=K._lib.PATH_AUTO):
    """w_l is the [N,K] weight's layout; the call gets its transposed (and broadcast) view."""
    wt = w_l.transpose(0, 1)
    batch = tuple(x_l.shape[:-2])
    out_l = Layout.from_shape((*batch, x_l.shape[-2], wt.shape[1]))
    rhs = wt.broadcast_to((*batch, *wt.shape)) if batch else wt
    md = [*matmul_metadata(x_l, rhs, out_l), b_l.strides[0], b_l.offset]
    n_out = out_l.size()
    out = new_out(n_out, dt)
    dx, dw, db = to_dev(x_bits), to_dev(w_bits), to_dev(b_bits)
    prev = K.force_path(path)
    try:
        K.call_ops_linear(DType(dt), 0, dx.data_ptr(), dw.data_ptr(), db.data_ptr(), out.data_ptr(), md, flags, 0)
        taken = K.last_path()
    finally:
        K.force_path(prev)
    assert K.last_status(0) == 0
    assert canary_intact(out, n_out)
    return from_dev(out[:n_out], dt), taken


def test_linear_golden_reference_output():
    x, w, bias = GOLDEN_EL["linear_f32__x"], GOLDEN_EL["linear_f32__w"], GOLDEN_EL["linear_f32__bias"]
    got, _ = run_linear(x, w, bias, Layout.from_shape(x.shape), Layout.from_shape(w.shape),
                        Layout.from_shape(bias.shape), O.F32, K._lib.LINEAR_ROUND_EACH_OP)
    assert O.rel_err(got, GOLDEN_EL["linear_f32__out"]) <= 1e-5


LINEAR_CASES = [
    # x shape, out_features, dtype, path
    ((33, 72), 19, O.BF16, K._lib.PATH_AUTO),                 # generic kernel, odd extents
    ((256, 512), 384, O.BF16, K._lib.PATH_TENSOR_1CTA),
    ((512, 512), 512, O.BF16, K._lib.PATH_TENSOR_2CTA),
    ((1024, 256), 512, O.BF16, K._lib.PATH_TENSOR_2CTA_512),
    ((1000, 264), 488, O.F16, K._lib.PATH_TENSOR_2CTA_512),   # tails in M and N
    ((3, 200, 128), 320, O.BF16, K._lib.PATH_TENSOR),         # batched input, weight broadcast
    ((512, 1024), 768, O.F32, K._lib.PATH_AUTO),              # split-TF32 path
    ((40, 64), 24, O.F32, K._lib.PATH_AUTO),
]


@pytest.mark.parametrize("flags", [K._lib.LINEAR_ROUND_EACH_OP, K._lib.LINEAR_ROUND_ONCE], ids=["each_op", "once"])
@pytest.mark.parametrize("case", LINEAR_CASES, ids=[f"{c[0]}x{c[1]}-{DType(c[2])}-p{c[3]}" for c in LINEAR_CASES])
def test_linear_bias_vs_oracle(case, flags):
    xs, n, dt, path = case
    k = xs[-1]
    rng = np.random.default_rng(n + k)
    x = O.narrow(rng.standard_normal(xs).astype(np.float32), dt)
    w = O.narrow((rng.standard_normal((n, k)) / np.sqrt(k)).astype(np.float32), dt)
    b = O.narrow(rng.standard_normal(n).astype(np.float32), dt)
    got, taken = run_linear(x, w, b, Layout.from_shape(xs), Layout.from_shape((n, k)), Layout.from_shape((n,)),
                            dt, flags, path)
    want = O.linear(O.widen(x, dt).reshape(xs), O.widen(w, dt).reshape(n, k).T, O.widen(b, dt),
                    dt, round_each_op=(flags == K._lib.LINEAR_ROUND_EACH_OP))
    assert O.rel_err(O.widen(got, dt), O.widen(want, dt)) <= TOL[dt]
    if path != K._lib.PATH_AUTO:
        assert taken == K._lib.PATH_TENSOR
    if dt == O.BF16 and flags == K._lib.LINEAR_ROUND_EACH_OP and path != K._lib.PATH_AUTO:
        # the op-by-op form is a deterministic function of the rounded product: most elements
        # must agree bit for bit with the oracle (the rest sit on a rounding boundary of the
        # product, where f32 summation order decides)
        assert np.mean(got == want) > 0.97


def test_linear_strided_bias_and_no_bias():
    rng = np.random.default_rng(9)
    m, k, n = 256, 256, 256
    x = O.narrow(rng.standard_normal((m, k)).astype(np.float32), O.BF16)
    w = O.narrow((rng.standard_normal((n, k)) / 16).astype(np.float32), O.BF16)
    braw = O.narrow(rng.standard_normal(5 + 3 * n).astype(np.float32), O.BF16)
    got, _ = run_linear(x, w, braw, Layout.from_shape((m, k)), Layout.from_shape((n, k)), Layout((n,), (3,), 5),
                        O.BF16, K._lib.LINEAR_ROUND_ONCE, K._lib.PATH_TENSOR)
    want = O.linear(O.widen(x, O.BF16).reshape(m, k), O.widen(w, O.BF16).reshape(n, k).T,
                    O.widen(braw, O.BF16)[5::3][:n], O.BF16, round_each_op=False)
    assert O.rel_err(O.widen(got, O.BF16), O.widen(want, O.BF16)) <= 1e-2
    # module form: with and without bias
    tx = Tensor.from_torch(to_dev(x).view(torch.bfloat16).reshape(m, k))
    tw = Tensor.from_torch(to_dev(w).view(torch.bfloat16).reshape(n, k))
    tb = Tensor.from_torch(to_dev(braw[:n].copy()).view(torch.bfloat16))
    y0 = Linear(tw).forward(tx).to_torch().float()
    y1 = Linear(tw, tb).forward(tx).to_torch().float()
    ref = (y0 + tb.to_torch().float()[None, :]).bfloat16().float()   # product rounded, then add, rounded
    assert torch.equal(y1, ref)
