"""Randomised parity sweep: seeded random shapes, dtypes, layouts (transposed views, padded
pitches, element offsets, stride-0 broadcast), batch structures and kernel families for the
matmul / dot wire formats, plus random einsum contractions, Linear-with-bias and conv2d
geometries, each through the C ABI against the CPU oracle.  The seeds are fixed, so a failure
names a reproducible case."""
import numpy as np
import pytest

from gpu_util import canary_intact, check_close, from_dev, gpu_matmul, new_out, to_dev
from hodu_b200 import CudaKernelError, DType, Layout, _lib
from hodu_b200 import kernels as K
from hodu_b200.einsum import ParsedEinsum, einsum_metadata
from hodu_b200.op_metadatas import conv2d_metadata, dot_metadata, matmul_metadata
from oracle import oracle as O

pytestmark = pytest.mark.gpu

PAIRS = [(O.BF16, O.BF16), (O.BF16, O.F32), (O.F16, O.F16), (O.F16, O.F32), (O.F32, O.F32),
         (O.F8E4M3, O.BF16), (O.F8E4M3, O.F32), (O.F8E4M3, O.F8E4M3), (O.I8, O.I32), (O.I8, O.I8)]
TOL = {O.F32: 1e-4, O.BF16: 1e-2, O.F16: 1e-2, O.F8E4M3: 7e-2}


def values(rng, n, dt):
    if dt in (O.I8,):
        return rng.integers(-127, 128, size=n, dtype=np.int8)
    scale = 4.0 if dt == O.F8E4M3 else 1.0
    return O.narrow((rng.standard_normal(n) * scale).astype(np.float32), dt)


def random_matrix_layout(rng, rows, cols, align):
    """(strides, extent) of a [rows, cols] matrix: row- or column-contiguous, pitch padded by a
    random amount (a multiple of `align` elements, or odd: TMA cannot take that)."""
    pad = int(rng.choice([0, 0, align, 3 * align, 1, 5]))
    if rng.random() < 0.5:
        pitch = cols + pad
        return (pitch, 1), (rows - 1) * pitch + cols
    pitch = rows + pad
    return (1, pitch), (cols - 1) * pitch + rows


def random_operand(rng, batch_out, rows, cols, dt, allow_broadcast):
    """Layout [batch.., rows, cols] + backing storage; batch dims densely packed over the matrix
    extent, some of them broadcast (stride 0)."""
    align = 16 // np.dtype(O.NP_STORAGE[dt]).itemsize
    (sr, sc), extent = random_matrix_layout(rng, rows, cols, align)
    extent = (extent + align - 1) // align * align if rng.random() < 0.7 else extent
    shape, strides, acc = [], [], extent
    for b in reversed(batch_out):
        if allow_broadcast and rng.random() < 0.3:
            shape.append(b); strides.append(0)
        else:
            shape.append(b); strides.append(acc); acc *= b
    shape.reverse(); strides.reverse()
    offset = int(rng.choice([0, 0, align, 2 * align, 1, 7]))
    lay = Layout((*shape, rows, cols), (*strides, sr, sc), offset)
    return lay, values(rng, offset + acc, dt)


@pytest.mark.parametrize("seed", range(120))
def test_random_matmul_cases(seed):
    rng = np.random.default_rng(1000 + seed)
    in_dt, out_dt = PAIRS[seed % len(PAIRS)]
    big = rng.random() < 0.35
    m, k, n = (int(rng.integers(1, 700 if big else 96)) for _ in range(3))
    nb = int(rng.choice([0, 0, 1, 2]))
    batch = [int(rng.integers(1, 4)) for _ in range(nb)]
    la, a = random_operand(rng, batch, m, k, in_dt, allow_broadcast=True)
    lb, b = random_operand(rng, batch, k, n, in_dt, allow_broadcast=True)
    if nb == 0:
        md, is_dot = dot_metadata(la, lb), True
    else:
        md, is_dot = matmul_metadata(la, lb, Layout.from_shape((*batch, m, n))), False
    scales = (0.25, 0.5) if in_dt == O.F8E4M3 else (1.0, 1.0)
    path = int(rng.choice([_lib.PATH_AUTO, _lib.PATH_AUTO, _lib.PATH_SIMT, _lib.PATH_TENSOR, _lib.PATH_TENSOR_1CTA,
                           _lib.PATH_TENSOR_2CTA, _lib.PATH_TENSOR_2CTA_512]))
    want = O.matmul(a, b, md, in_dt, out_dt, scales[0] * scales[1], is_dot=is_dot)
    try:
        got, _ = gpu_matmul(a, b, md, in_dt, out_dt, scales=scales, is_dot=is_dot, path=path)
    except CudaKernelError as e:
        # forcing the tensor cores onto a layout they cannot take is an error by contract
        assert path >= _lib.PATH_TENSOR and "refused" in str(e), str(e)
        got, _ = gpu_matmul(a, b, md, in_dt, out_dt, scales=scales, is_dot=is_dot, path=_lib.PATH_AUTO)
    check_close(got, want, out_dt, TOL.get(out_dt, 0))


EINSUM_FORMS = ["ij,jk->ik", "ij,jk->ki", "ik,jk->ij", "ji,jk->ik", "bij,bjk->bik", "bij,bkj->bik", "bij,jk->bik",
                "abij,abjk->abik", "bhqd,bhkd->bhqk", "bhqk,bhkd->bhqd", "ij,j->i", "i,ij->j", "i,j->ij", "i,i->",
                "abk,kn->abn", "bij,ijk->bk", "ij,jk"]


@pytest.mark.parametrize("seed", range(51))
def test_random_einsum_cases(seed):
    rng = np.random.default_rng(2000 + seed)
    eq = EINSUM_FORMS[seed % len(EINSUM_FORMS)]
    dt = [O.BF16, O.F32, O.F16, O.I32][seed % 4]
    letters = sorted(set(c for c in eq if c.isalpha()))
    hi = 160 if seed % 3 == 0 else 24
    size = {c: int(rng.integers(1, hi)) for c in letters}
    while np.prod([float(v) for v in size.values()]) > 2e6:   # keep the oracle's work bounded
        big_c = max(size, key=size.get)
        size[big_c] = max(1, size[big_c] // 2)
    subs = eq.split("->")[0].split(",")
    shapes = [tuple(size[c] for c in s) for s in subs]
    lays = [Layout.from_shape(s) for s in shapes]
    parsed = ParsedEinsum.parse(eq, shapes)
    ol = Layout.from_shape(tuple(parsed.compute_output_shape()))
    md = einsum_metadata(parsed, lays, ol)
    if dt == O.I32:
        ins = [rng.integers(-50, 51, size=max(l.size(), 1), dtype=np.int32) for l in lays]
    else:
        gen = (lambda n: np.abs(rng.standard_normal(n))) if ol.size() <= 1 else rng.standard_normal
        ins = [O.narrow(gen(max(l.size(), 1)).astype(np.float32), dt) for l in lays]
    n_out = int(md[0])
    out = new_out(n_out, dt)
    devs = [to_dev(x) for x in ins]
    K.call_ops_einsum(getattr(K.einsum, str(DType(dt)).upper()), 0, [d.data_ptr() for d in devs], out.data_ptr(), md, 0)
    assert K.last_status(0) == 0 and canary_intact(out, n_out)
    got = from_dev(out[:n_out], dt)
    want = O.einsum(ins, md, dt)
    if dt == O.I32:
        assert np.array_equal(got, want)
    else:
        assert O.rel_err(O.widen(got, dt), O.widen(want, dt)) <= TOL[dt]


@pytest.mark.parametrize("seed", range(40))
def test_random_conv2d_cases(seed):
    rng = np.random.default_rng(3000 + seed)
    dt = [O.BF16, O.F16, O.F32][seed % 3]
    b, ci, co = int(rng.integers(1, 4)), int(rng.integers(1, 40)), int(rng.integers(1, 70))
    kh, kw = int(rng.choice([1, 1, 2, 3, 3, 5])), int(rng.choice([1, 1, 2, 3, 3, 7]))
    sh, sw = int(rng.integers(1, 3)), int(rng.integers(1, 3))
    ph, pw = int(rng.integers(0, 3)), int(rng.integers(0, 3))
    dh, dw = int(rng.integers(1, 3)), int(rng.integers(1, 3))
    h = int(rng.integers(dh * (kh - 1) + 1, dh * (kh - 1) + 40))
    w = int(rng.integers(dw * (kw - 1) + 1, dw * (kw - 1) + 40))
    offs = (int(rng.choice([0, 0, 8, 3])), int(rng.choice([0, 0, 8, 5])))
    md = conv2d_metadata(b, ci, co, (h, w), (kh, kw), (sh, sw), (ph, pw), (dh, dw), offs[0], offs[1])
    x = O.narrow(rng.standard_normal(offs[0] + b * ci * h * w).astype(np.float32), dt)
    wt = O.narrow((rng.standard_normal(offs[1] + co * ci * kh * kw) / np.sqrt(ci * kh * kw)).astype(np.float32), dt)
    n_out = int(md[0])
    out = new_out(n_out, dt)
    dx, dw_ = to_dev(x), to_dev(wt)
    K.call_ops_conv(getattr(K.conv2d, str(DType(dt)).upper()), 0, dx.data_ptr(), dw_.data_ptr(), out.data_ptr(), md, 0)
    assert K.last_status(0) == 0 and canary_intact(out, n_out)
    got = from_dev(out[:n_out], dt)
    want = O.conv2d(x, wt, md, dt)
    assert O.rel_err(O.widen(got, dt), O.widen(want, dt)) <= TOL[dt]


@pytest.mark.parametrize("seed", range(30))
def test_random_linear_cases(seed):
    rng = np.random.default_rng(4000 + seed)
    dt = [O.BF16, O.F16, O.F32][seed % 3]
    flags = seed % 2
    big = seed % 4 == 0
    m, k, n = (int(rng.integers(1, 600 if big else 80)) for _ in range(3))
    if big:
        k = (k + 7) // 8 * 8          # a Linear weight [N,K] the tensor cores can take as it lies
    batch = [int(rng.integers(1, 4))] if seed % 5 == 0 else []
    x = O.narrow(rng.standard_normal((*batch, m, k)).astype(np.float32), dt)
    w = O.narrow((rng.standard_normal((n, k)) / np.sqrt(k)).astype(np.float32), dt)
    bstride = int(rng.choice([1, 1, 2]))
    boff = int(rng.choice([0, 3]))
    braw = O.narrow(rng.standard_normal(boff + bstride * n).astype(np.float32), dt)
    x_l = Layout.from_shape((*batch, m, k))
    wt = Layout.from_shape((n, k)).transpose(0, 1)
    rhs = wt.broadcast_to((*batch, k, n)) if batch else wt
    out_l = Layout.from_shape((*batch, m, n))
    md = [*matmul_metadata(x_l, rhs, out_l), bstride, boff]
    n_out = out_l.size()
    out = new_out(n_out, dt)
    dx, dw_, db = to_dev(x), to_dev(w), to_dev(braw)
    K.call_ops_linear(DType(dt), 0, dx.data_ptr(), dw_.data_ptr(), db.data_ptr(), out.data_ptr(), md, flags, 0)
    assert K.last_status(0) == 0 and canary_intact(out, n_out)
    got = from_dev(out[:n_out], dt)
    bias = O.widen(braw, dt)[boff::bstride][:n]
    want = O.linear(O.widen(x, dt).reshape(*batch, m, k), O.widen(w, dt).reshape(n, k).T, bias, dt,
                    round_each_op=(flags == _lib.LINEAR_ROUND_EACH_OP))
    assert O.rel_err(O.widen(got, dt), O.widen(want, dt)) <= TOL[dt]


@pytest.mark.parametrize("seed", range(36))
def test_random_large_tails_on_the_pair_forms(seed):
    """Extents of 300..2100 that are multiples of nothing in particular, on the CTA-pair tile
    forms (256x256 and 512x256) and the automatic choice: M / N / K tails of every size."""
    rng = np.random.default_rng(5000 + seed)
    in_dt, out_dt = [(O.BF16, O.BF16), (O.I8, O.I32), (O.F8E4M3, O.BF16), (O.F16, O.F32)][seed % 4]
    esz = np.dtype(O.NP_STORAGE[in_dt]).itemsize
    unit = 16 // esz
    m = int(rng.integers(300, 2100))
    k = int(rng.integers(300, 2100)) // unit * unit        # pitches TMA can take
    n = int(rng.integers(300, 2100)) // 8 * 8
    b_kmajor = bool(rng.integers(0, 2))
    if esz == 1 and not b_kmajor:
        n = n // 16 * 16
    a = values(rng, m * k, in_dt)
    b = values(rng, k * n, in_dt)
    la = Layout.from_shape((m, k))
    lb = Layout.from_shape((n, k)).transpose(0, 1) if b_kmajor else Layout.from_shape((k, n))
    md = dot_metadata(la, lb)
    scales = (0.125, 0.25) if in_dt == O.F8E4M3 else (1.0, 1.0)
    path = [_lib.PATH_AUTO, _lib.PATH_TENSOR_2CTA, _lib.PATH_TENSOR_2CTA_512][seed % 3]
    got, taken = gpu_matmul(a, b, md, in_dt, out_dt, scales=scales, is_dot=True, path=path)
    assert taken == _lib.PATH_TENSOR
    want = O.matmul(a, b, md, in_dt, out_dt, scales[0] * scales[1], is_dot=True)
    check_close(got, want, out_dt, TOL.get(out_dt, 0))
