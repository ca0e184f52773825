"""Parity of the CUDA matmul / dot path with the CPU oracle, through the C ABI.

Bars: integer outputs bit-exact; bf16 / f16 max|got-want| / max|want| <= 1e-2; f8e4m3 inputs
<= 6e-2 of output scale; f32 <= 1e-4.  The oracle widens to f32, multiplies with sgemm and
narrows once with round-to-nearest-even."""
import numpy as np
import pytest

from gpu_util import check_close, gpu_matmul
from hodu_b200 import CudaKernelError, DType, Layout, _lib
from hodu_b200 import kernels as K
from hodu_b200.op_metadatas import dot_metadata, matmul_metadata
from oracle import oracle as O
from test_oracle import KNOWN

pytestmark = pytest.mark.gpu

TOL = {O.BF16: 1e-2, O.F16: 1e-2, O.F8E4M3: 6e-2, O.F32: 1e-4}
AUTO, SIMT, TENSOR = _lib.PATH_AUTO, _lib.PATH_SIMT, _lib.PATH_TENSOR


def rand_storage(rng, dtype, shape):
    if dtype in (O.I8,):
        return rng.integers(-127, 128, size=shape, dtype=np.int8)
    if dtype == O.I32:
        return rng.integers(-1000, 1000, size=shape).astype(np.int32)
    x = rng.standard_normal(shape).astype(np.float32)
    if dtype == O.F8E4M3:
        x = np.clip(x * 16, -448, 448)
    return O.narrow(x, dtype)


def operand(rng, dtype, rows, cols, contiguous_index):
    """A [rows, cols] operand whose `contiguous_index` ('r' or 'c') has stride 1."""
    if contiguous_index == "c":
        return rand_storage(rng, dtype, (rows, cols)), Layout.from_shape((rows, cols))
    return rand_storage(rng, dtype, (cols, rows)), Layout.from_shape((cols, rows)).transpose(0, 1)


@pytest.mark.parametrize("case", KNOWN, ids=[c[0] for c in KNOWN])
def test_reference_known_answers(case):
    """The reference's eight f32 known-answer tests, same metadata vectors, plain API."""
    _, is_dot, lhs, rhs, md, want = case
    got, _ = gpu_matmul(np.array(lhs, np.float32), np.array(rhs, np.float32), md, O.F32, is_dot=is_dot, plain_api=True)
    assert np.array_equal(np.round(got * 1e4) / 1e4, np.array(want, np.float32))


PAIRS = [(O.BF16, O.BF16), (O.F16, O.F16), (O.F8E4M3, O.BF16), (O.F8E4M3, O.F8E4M3), (O.F8E4M3, O.F32),
         (O.I8, O.I32), (O.I8, O.I8), (O.BF16, O.F32), (O.F16, O.F32), (O.F8E4M3, O.F16)]
SHAPES = [(128, 128, 256), (200, 136, 328), (1, 256, 128), (129, 2064, 72), (512, 512, 512), (130, 8, 16)]


@pytest.mark.parametrize("in_dt,out_dt", PAIRS)
@pytest.mark.parametrize("a_c,b_c", [("c", "c"), ("c", "r"), ("r", "c"), ("r", "r")])
def test_tensor_core_path_all_layouts(in_dt, out_dt, a_c, b_c):
    rng = np.random.default_rng(1000 * in_dt + 10 * out_dt + (a_c == "r") * 2 + (b_c == "r"))
    for (m, k, n) in SHAPES:
        # TMA needs 16-byte pitches: round the extent that becomes a pitch
        unit = 16 // O.NP_STORAGE[in_dt]().itemsize
        if (a_c == "c" and m > 1) or b_c == "r":
            k = (k + unit - 1) // unit * unit
        if a_c == "r":
            m = (m + unit - 1) // unit * unit if k > 1 else m
        if b_c == "c":
            n = (n + unit - 1) // unit * unit
        a, la = operand(rng, in_dt, m, k, a_c)
        b, lb = operand(rng, in_dt, k, n, b_c)
        md = dot_metadata(la, lb)
        scales = (0.5, 0.25) if in_dt == O.F8E4M3 else (1.0, 1.0)
        got, path = gpu_matmul(a, b, md, in_dt, out_dt, scales, is_dot=True, path=TENSOR)
        assert path == TENSOR
        want = O.matmul(a, b, md, in_dt, out_dt, scales[0] * scales[1], is_dot=True)
        tol = TOL.get(in_dt, 0) if out_dt != O.F8E4M3 else 7e-2  # e4m3 output: half an ulp at the top is 1/16
        check_close(got, want, out_dt, tol)


FORMS = [_lib.PATH_TENSOR_1CTA, _lib.PATH_TENSOR_2CTA, _lib.PATH_TENSOR_2CTA_512]


@pytest.mark.parametrize("form", FORMS)
@pytest.mark.parametrize("in_dt,out_dt", [(O.BF16, O.BF16), (O.F16, O.F32), (O.F8E4M3, O.BF16), (O.I8, O.I32), (O.F32, O.F32)])
@pytest.mark.parametrize("a_c,b_c", [("c", "c"), ("c", "r"), ("r", "c"), ("r", "r")])
def test_every_tile_form(form, in_dt, out_dt, a_c, b_c):
    """One CTA per 128xBN tile, CTA pair per 256x256 tile, CTA pair per 512x256 tile: same
    results, including M/N/K tails and tiles that are mostly out of range."""
    rng = np.random.default_rng(form * 100 + in_dt)
    for (m, k, n) in [(640, 272, 400), (512, 512, 512), (144, 128, 80), (1040, 64, 272)]:
        a, la = operand(rng, in_dt, m, k, a_c)
        b, lb = operand(rng, in_dt, k, n, b_c)
        md = dot_metadata(la, lb)
        got, taken = gpu_matmul(a, b, md, in_dt, out_dt, is_dot=True, path=form)
        assert taken == TENSOR
        check_close(got, O.matmul(a, b, md, in_dt, out_dt, is_dot=True), out_dt, TOL.get(in_dt, 0))


@pytest.mark.parametrize("form", FORMS)
def test_every_tile_form_batched(form):
    rng = np.random.default_rng(form)
    lshape, rshape = (3, 520, 136), (1, 136, 264)
    a, b = rand_storage(rng, O.BF16, lshape), rand_storage(rng, O.BF16, rshape)
    md = matmul_metadata(Layout.from_shape(lshape), Layout.from_shape(rshape), Layout.from_shape((3, 520, 264)))
    got, _ = gpu_matmul(a, b, md, O.BF16, path=form)
    check_close(got, O.matmul(a, b, md, O.BF16), O.BF16, 1e-2)


@pytest.mark.parametrize("in_dt,out_dt", PAIRS + [(O.F32, O.F32), (O.I32, O.I32)])
def test_simt_path_any_strides(in_dt, out_dt):
    """Pitches and offsets TMA cannot describe: odd extents, element offsets, padded rows."""
    rng = np.random.default_rng(77 + in_dt + out_dt)
    for (m, k, n, pad, off) in [(2, 3, 2, 0, 0), (37, 53, 29, 0, 0), (65, 70, 130, 3, 5), (1, 1, 1, 0, 1), (64, 16, 64, 1, 0)]:
        a = rand_storage(rng, in_dt, (off + m * (k + pad),))
        b = rand_storage(rng, in_dt, (off + k * (n + pad),))
        la = Layout((m, k), (k + pad, 1), off)
        lb = Layout((k, n), (n + pad, 1), off)
        md = dot_metadata(la, lb)
        got, path = gpu_matmul(a, b, md, in_dt, out_dt, is_dot=True, path=SIMT)
        assert path == SIMT
        want = O.matmul(a, b, md, in_dt, out_dt, is_dot=True)
        check_close(got, want, out_dt, TOL.get(in_dt, 0) if out_dt != O.F8E4M3 else 7e-2)
        # element-by-element C restatement on the small ones
        if m * n * k < 200000:
            want_c = O.matmul_c(a, b, md, in_dt, out_dt, is_dot=True)
            check_close(got, want_c, out_dt, TOL.get(in_dt, 0) if out_dt != O.F8E4M3 else 7e-2)


@pytest.mark.parametrize("in_dt,out_dt", [(O.BF16, O.BF16), (O.F8E4M3, O.BF16), (O.I8, O.I32)])
def test_both_gpu_paths_agree(in_dt, out_dt):
    rng = np.random.default_rng(5)
    a, la = operand(rng, in_dt, 256, 384, "c")
    b, lb = operand(rng, in_dt, 384, 256, "c")
    md = dot_metadata(la, lb)
    t, _ = gpu_matmul(a, b, md, in_dt, out_dt, is_dot=True, path=TENSOR)
    s, _ = gpu_matmul(a, b, md, in_dt, out_dt, is_dot=True, path=SIMT)
    check_close(t, s, out_dt, 4e-3)  # both accumulate in f32; they differ by summation order and one bf16 ulp


BATCH_CASES = [
    # (lhs shape, rhs shape) -- broadcasting over batch dims, right-aligned
    ((3, 128, 64), (3, 64, 128)),
    ((3, 128, 64), (64, 128)),            # rhs 2-D, as in the reference's CUDA batch test
    ((1, 136, 64), (4, 64, 72)),          # lhs broadcast
    ((2, 3, 128, 64), (2, 3, 64, 128)),
    ((2, 1, 128, 64), (1, 3, 64, 128)),   # both broadcast, different dims
    ((2, 3, 4, 40, 64), (4, 64, 48)),
]


@pytest.mark.parametrize("lshape,rshape", BATCH_CASES)
@pytest.mark.parametrize("in_dt,out_dt", [(O.BF16, O.BF16), (O.I8, O.I32), (O.F32, O.F32)])
@pytest.mark.parametrize("as_views", [False, True])
def test_batched_broadcast(lshape, rshape, in_dt, out_dt, as_views):
    """as_views: both operands broadcast to the full batch shape with stride-0 dims, which is
    what Tensor::matmul passes (tensor/ops/matrix.rs:155-167)."""
    rng = np.random.default_rng(len(lshape) * 100 + len(rshape) + in_dt)
    a, b = rand_storage(rng, in_dt, lshape), rand_storage(rng, in_dt, rshape)
    la, lb = Layout.from_shape(lshape), Layout.from_shape(rshape)
    nb = max(len(lshape), len(rshape)) - 2
    lb_dims = (1,) * (nb - (len(lshape) - 2)) + tuple(lshape[:-2])
    rb_dims = (1,) * (nb - (len(rshape) - 2)) + tuple(rshape[:-2])
    batch = tuple(max(x, y) for x, y in zip(lb_dims, rb_dims))
    if as_views:
        la = la.broadcast_to((*batch, *lshape[-2:]))
        lb = lb.broadcast_to((*batch, *rshape[-2:]))
    out_l = Layout.from_shape((*batch, lshape[-2], rshape[-1]))
    md = matmul_metadata(la, lb, out_l)
    want = O.matmul(a, b, md, in_dt, out_dt)
    paths = [SIMT, TENSOR]  # pitches TMA cannot take are re-laid into scratch on the tensor path
    for path in paths:
        got, taken = gpu_matmul(a, b, md, in_dt, out_dt, path=path)
        assert taken == path
        check_close(got, want, out_dt, TOL.get(in_dt, 0))
    if int(np.prod(out_l.shape)) * lshape[-1] < 300000:
        check_close(want, O.matmul_c(a, b, md, in_dt, out_dt), out_dt, TOL.get(in_dt, 0))


@pytest.mark.parametrize("a_c,b_c", [("c", "c"), ("c", "r"), ("r", "c"), ("r", "r")])
def test_f32_on_tensor_cores_keeps_f32_accuracy(a_c, b_c):
    """Three TF32 products of split operands: far inside the 1e-4 bar (one plain TF32 product
    would sit near 1e-3), for any strides, offsets and odd extents."""
    rng = np.random.default_rng(31)
    for (m, k, n) in [(512, 1024, 768), (130, 37, 29), (257, 515, 130), (1, 300, 64)]:
        a, la = operand(rng, O.F32, m, k, a_c)
        b, lb = operand(rng, O.F32, k, n, b_c)
        md = dot_metadata(la, lb)
        for path in (TENSOR, _lib.PATH_TENSOR_2CTA, _lib.PATH_TENSOR_2CTA_512):
            got, taken = gpu_matmul(a, b, md, O.F32, is_dot=True, path=path)
            assert taken == TENSOR
            want = np.matmul(O._strided(a.reshape(-1), la.shape, la.strides, 0).astype(np.float64),
                             O._strided(b.reshape(-1), lb.shape, lb.strides, 0).astype(np.float64))
            assert O.rel_err(got, want.reshape(-1)) <= 2e-5
        assert O.rel_err(got, O.matmul(a, b, md, O.F32, is_dot=True)) <= 1e-4   # the reference's sgemm
    # padded pitch + element offset that no TMA map could take directly
    a = rand_storage(rng, O.F32, (5 + 70 * 67,))
    b = rand_storage(rng, O.F32, (3 + 64 * 131,))
    md = dot_metadata(Layout((70, 64), (67, 1), 5), Layout((64, 130), (131, 1), 3))
    got, _ = gpu_matmul(a, b, md, O.F32, is_dot=True, path=TENSOR)
    assert O.rel_err(got, O.matmul(a, b, md, O.F32, is_dot=True)) <= 1e-5


@pytest.mark.parametrize("in_dt,out_dt", [(O.BF16, O.BF16), (O.F16, O.F32), (O.F8E4M3, O.BF16), (O.I8, O.I32)])
def test_layout_front_door_relays_what_tma_cannot_take(in_dt, out_dt):
    """Odd pitches, odd element offsets and doubly-strided operands on the tensor path: the
    operand is copied into scratch as a dense K-contiguous matrix first."""
    rng = np.random.default_rng(41 + in_dt)
    cases = [
        # (M, K, N, lhs layout maker, rhs layout maker)
        (200, 301, 136, lambda m, k: Layout((m, k), (k + 3, 1), 5), lambda k, n: Layout((k, n), (n + 1, 1), 7)),
        (136, 264, 200, lambda m, k: Layout((m, k), (1, m + 5), 1), lambda k, n: Layout((k, n), (1, k + 9), 3)),   # transposed, odd pitch
        (130, 96, 70, lambda m, k: Layout((m, k), (2 * k, 2), 0), lambda k, n: Layout((k, n), (3 * n, 3), 0)),     # no contiguous index
    ]
    for m, k, n, mk_a, mk_b in cases:
        la, lb = mk_a(m, k), mk_b(k, n)
        size_a = la.offset + sum((s - 1) * st for s, st in zip(la.shape, la.strides)) + 1
        size_b = lb.offset + sum((s - 1) * st for s, st in zip(lb.shape, lb.strides)) + 1
        a, b = rand_storage(rng, in_dt, (size_a,)), rand_storage(rng, in_dt, (size_b,))
        md = dot_metadata(la, lb)
        want = O.matmul(a, b, md, in_dt, out_dt, is_dot=True)
        for path in (TENSOR, _lib.PATH_TENSOR_2CTA):
            got, taken = gpu_matmul(a, b, md, in_dt, out_dt, is_dot=True, path=path)
            assert taken == TENSOR
            check_close(got, want, out_dt, TOL.get(in_dt, 0))


def test_offsets_on_tensor_path():
    """Views into a larger buffer: 16-byte-aligned element offsets and padded pitches."""
    rng = np.random.default_rng(3)
    m, k, n, pitch_a, pitch_b = 160, 192, 136, 200, 144
    a = rand_storage(rng, O.BF16, (64 + m * pitch_a,))
    b = rand_storage(rng, O.BF16, (24 + k * pitch_b,))
    md = dot_metadata(Layout((m, k), (pitch_a, 1), 64), Layout((k, n), (pitch_b, 1), 24))
    got, path = gpu_matmul(a, b, md, O.BF16, is_dot=True, path=TENSOR)
    check_close(got, O.matmul(a, b, md, O.BF16, is_dot=True), O.BF16, 1e-2)


def test_auto_path_selection_and_refusal():
    rng = np.random.default_rng(4)
    # large aligned -> tensor cores
    a, la = operand(rng, O.BF16, 256, 256, "c")
    b, lb = operand(rng, O.BF16, 256, 256, "c")
    _, path = gpu_matmul(a, b, dot_metadata(la, lb), O.BF16, is_dot=True)
    assert path == TENSOR
    # K = 297: a row pitch of 594 bytes cannot be a TMA stride.  Large enough to pay for a copy:
    # the operands are re-laid into scratch and the tensor cores still run
    a, la = operand(rng, O.BF16, 256, 37 * 8 + 1, "c")
    b, lb = operand(rng, O.BF16, 37 * 8 + 1, 256, "r")
    md = dot_metadata(la, lb)
    got, path = gpu_matmul(a, b, md, O.BF16, is_dot=True)
    assert path == TENSOR
    check_close(got, O.matmul(a, b, md, O.BF16, is_dot=True), O.BF16, 1e-2)
    # the same kind of layout, small: the generic CUDA-core kernel, same answer bar
    a, la = operand(rng, O.BF16, 64, 37, "c")
    b, lb = operand(rng, O.BF16, 37, 64, "c")
    md = dot_metadata(la, lb)
    got, path = gpu_matmul(a, b, md, O.BF16, is_dot=True)
    assert path == SIMT
    check_close(got, O.matmul(a, b, md, O.BF16, is_dot=True), O.BF16, 1e-2)
    # a dtype with no tensor-core kernel is refused when the tensor path is forced, never re-routed
    ai = rand_storage(rng, O.I32, (64, 64))
    with pytest.raises(CudaKernelError) as e:
        gpu_matmul(ai, ai, dot_metadata(Layout.from_shape((64, 64)), Layout.from_shape((64, 64))), O.I32,
                   is_dot=True, path=TENSOR)
    assert e.value.kind == "invalid input" and "tensor-core path refused" in str(e.value)
    # f32: tiny products stay on the CUDA cores, the rest runs as split TF32 on the tensor cores
    # (one kernel for small products, the operand-split path for large ones)
    a, la = operand(rng, O.F32, 32, 32, "c")
    _, path = gpu_matmul(a, a, dot_metadata(la, la), O.F32, is_dot=True)
    assert path == SIMT
    for d, launches in ((128, 1), (512, 1), (2048, 2)):
        a, la = operand(rng, O.F32, d, d, "c")
        before = K.launch_count()
        got, path = gpu_matmul(a, a, dot_metadata(la, la), O.F32, is_dot=True)
        assert path == TENSOR and K.launch_count() - before == launches
        assert O.rel_err(got, O.matmul(a, a, dot_metadata(la, la), O.F32, is_dot=True)) <= 1e-4


def test_aliased_inputs_and_k_zero():
    rng = np.random.default_rng(6)
    a, la = operand(rng, O.BF16, 128, 128, "c")
    md = dot_metadata(la, la)
    got, _ = gpu_matmul(a, a, md, O.BF16, is_dot=True, path=TENSOR)  # a.matmul(&a)
    check_close(got, O.matmul(a, a, md, O.BF16, is_dot=True), O.BF16, 1e-2)
    # K == 0: an empty sum is zero
    md0 = dot_metadata(Layout.from_shape((4, 0)), Layout.from_shape((0, 5)))
    got, _ = gpu_matmul(np.zeros(1, np.float32), np.zeros(1, np.float32), md0, O.F32, is_dot=True)
    assert np.array_equal(got, np.zeros(20, np.float32))


def test_saturation_of_e4m3_output():
    """Sums beyond +-448 saturate to the largest finite e4m3, they do not become NaN."""
    k = 128
    a = O.narrow(np.full((128, k), 16.0, np.float32), O.F8E4M3)
    b = O.narrow(np.full((k, 128), 16.0, np.float32), O.F8E4M3)
    b[:, 64:] ^= 0x80  # negative half
    md = dot_metadata(Layout.from_shape((128, k)), Layout.from_shape((k, 128)))
    for path in (TENSOR, SIMT):
        got, _ = gpu_matmul(a, b, md, O.F8E4M3, O.F8E4M3, is_dot=True, path=path)
        g = got.reshape(128, 128)
        assert np.all(g[:, :64] == 0x7E) and np.all(g[:, 64:] == 0xFE)


# ---------------------------------------------------------------- split over K for small outputs
SPLITK = [
    # M, K, N, in dtype, out dtype, lhs K-contiguous?, rhs N-contiguous?, launches expected
    # (one launch: K slices across the CTAs of a cluster; two: slices as batches plus a reduction)
    (256, 8192, 256, O.BF16, O.BF16, True, True, 1),
    (256, 8192, 256, O.BF16, O.F32, False, False, 1),     # transposed views of both operands
    (128, 4096, 192, O.F16, O.F16, True, False, 1),
    (128, 16384, 64, O.F8E4M3, O.BF16, True, True, 1),
    (256, 8192, 2048, O.BF16, O.BF16, True, True, 2),     # K long enough for eight slices of 16 k-blocks
    (512, 1024, 768, O.F32, O.F32, True, True, 1),         # config 1: the one-kernel f32 form (K slices added inside the cluster)
    (512, 1024, 768, O.F32, O.F32, True, False, 1),        # the same with a K-contiguous rhs (a Linear weight view)
    (256, 16384, 256, O.F32, O.F32, True, True, 3),        # K too long for that form: operand split, product, reduction
    (256, 8192, 250, O.BF16, O.BF16, True, False, 1),      # N not a multiple of 4: runs whole
]


@pytest.mark.parametrize("case", SPLITK, ids=[f"{c[0]}x{c[1]}x{c[2]}-{DType(c[3])}-{DType(c[4])}-{int(c[5])}{int(c[6])}" for c in SPLITK])
def test_small_outputs_with_long_k_are_split_over_k(case):
    m, k, n, in_dt, out_dt, a_kmajor, b_nmajor, launches = case
    rng = np.random.default_rng(m + k + n)
    scale = 8.0 if in_dt == O.F8E4M3 else 1.0
    a = O.narrow((rng.standard_normal((m, k)) * scale).astype(np.float32), in_dt).reshape(m, k)
    b = O.narrow((rng.standard_normal((k, n)) * scale).astype(np.float32), in_dt).reshape(k, n)
    la = Layout.from_shape((m, k)) if a_kmajor else Layout.from_shape((k, m)).transpose(0, 1)
    lb = Layout.from_shape((k, n)) if b_nmajor else Layout.from_shape((n, k)).transpose(0, 1)
    a_store = a if a_kmajor else np.ascontiguousarray(a.T)
    b_store = b if b_nmajor else np.ascontiguousarray(b.T)
    md = dot_metadata(la, lb)
    scales = (1 / 16, 1 / 4) if in_dt == O.F8E4M3 else (1.0, 1.0)
    before = K.launch_count()
    got, taken = gpu_matmul(a_store, b_store, md, in_dt, out_dt, scales=scales, is_dot=True)
    assert K.launch_count() - before == launches
    assert taken == K._lib.PATH_TENSOR
    want = O.matmul(a_store, b_store, md, in_dt, out_dt, scales[0] * scales[1], is_dot=True)
    tol = {O.F32: 1e-4, O.BF16: 1e-2, O.F16: 1e-2}[out_dt] if in_dt != O.F8E4M3 else 6e-2
    check_close(got, want, out_dt, tol)


@pytest.mark.parametrize("m,k,n", [(256, 16384, 512), (512, 40000, 256), (1024, 8192, 1024)])
def test_f32_long_k_stays_inside_the_bar(m, k, n):
    """The tensor core adds into its f32 accumulator with truncation; one accumulator over a long
    K drifts past the 1e-4 bar (2.8e-4 measured at K = 32768).  The f32 path restarts the
    accumulator every 4096 (2048) elements of K and adds the generations in f32 on the way out."""
    rng = np.random.default_rng(k)
    a = rng.standard_normal((m, k)).astype(np.float32)
    b = rng.standard_normal((k, n)).astype(np.float32)
    md = dot_metadata(Layout.from_shape((m, k)), Layout.from_shape((k, n)))
    got, taken = gpu_matmul(a, b, md, O.F32, O.F32, is_dot=True)
    assert taken == K._lib.PATH_TENSOR
    want = (a.astype(np.float64) @ b.astype(np.float64)).astype(np.float32).reshape(-1)
    assert O.rel_err(got, want) <= 2e-5


@pytest.mark.parametrize("m,k,n,out_shift", [(256, 40000, 250, 0), (300, 40000, 253, 0), (256, 40000, 256, 1),
                                             (512, 16384, 130, 3)])
def test_f32_long_k_with_outputs_that_rule_out_vector_stores(m, k, n, out_shift):
    """The same bar when the output rows cannot take 16-byte stores (N not a multiple of 4, or an
    output pointer at an odd element): the accumulator generations still run, through the
    element-wise store path."""
    import torch
    from gpu_util import DEV, to_dev
    rng = np.random.default_rng(k + n)
    a = rng.standard_normal((m, k)).astype(np.float32)
    b = rng.standard_normal((k, n)).astype(np.float32)
    md = dot_metadata(Layout.from_shape((m, k)), Layout.from_shape((k, n)))
    ta, tb = to_dev(a), to_dev(b)
    buf = torch.full((m * n + out_shift + 64,), 7.0, dtype=torch.float32, device=DEV)
    out = buf[out_shift:]
    prev = K.force_path(TENSOR)
    try:
        K.call_ops_dot(K.dot.F32, 0, ta.data_ptr(), tb.data_ptr(), out.data_ptr(), md, 0)
        assert K.last_path() == TENSOR
    finally:
        K.force_path(prev)
    assert K.last_status(0) == 0
    host = buf.cpu().numpy()
    assert (host[:out_shift] == 7.0).all() and (host[out_shift + m * n:] == 7.0).all()
    want = (a.astype(np.float64) @ b.astype(np.float64)).astype(np.float32).reshape(-1)
    assert O.rel_err(host[out_shift:out_shift + m * n], want) <= 2e-5


def test_output_beyond_two_to_the_31_elements():
    """Maximum sizes: an output of 66000 x 33000 = 2.18e9 elements (4.4 GB of bf16), so element
    and byte offsets pass 2^31 and 2^32; rows sampled from both ends and the middle are checked
    against the oracle, and the element after the last one is untouched."""
    import torch
    m, k, n = 66000, 32, 33000
    rng = np.random.default_rng(7)
    a = O.narrow(rng.standard_normal((m, k)).astype(np.float32), O.BF16)
    b = O.narrow(rng.standard_normal((k, n)).astype(np.float32), O.BF16)
    md = dot_metadata(Layout.from_shape((m, k)), Layout.from_shape((k, n)))
    dev = torch.device("cuda:0")
    ta = torch.from_numpy(a.view(np.int16)).to(dev)
    tb = torch.from_numpy(b.view(np.int16)).to(dev)
    out = torch.empty(m * n + 64, dtype=torch.int16, device=dev)
    out[m * n:] = 0x5A5A
    K.call_ops_dot(K.dot.BF16, 0, ta.data_ptr(), tb.data_ptr(), out.data_ptr(), md, 0)
    assert K.last_status(0) == 0 and K.last_path() == K._lib.PATH_TENSOR
    assert bool((out[m * n:] == 0x5A5A).all().item())
    af, bf = O.widen(a, O.BF16).reshape(m, k), O.widen(b, O.BF16).reshape(k, n)
    for r in (0, 1, 32767, 32768, 65535, 65536, m - 1):
        got = out[r * n:(r + 1) * n].cpu().numpy().view(np.uint16)
        want = O.narrow(af[r:r + 1] @ bf, O.BF16).reshape(-1)
        assert O.rel_err(O.widen(got, O.BF16), O.widen(want, O.BF16)) <= 1e-2, r
    del out
    torch.cuda.empty_cache()


def test_empty_extents_on_every_entry_point():
    """Empty inputs: every entry point returns success, launches nothing and leaves the output alone."""
    import torch
    from hodu_b200.einsum import ParsedEinsum, einsum_metadata
    from hodu_b200.op_metadatas import cast_metadata, conv2d_metadata, swiglu_metadata
    dev = torch.device("cuda:0")
    buf = torch.full((256,), 7, dtype=torch.int16, device=dev)
    p = buf.data_ptr()
    before = K.launch_count()
    for (m, k, n) in ((0, 8, 8), (8, 8, 0), (0, 0, 0)):
        K.call_ops_dot(K.dot.BF16, 0, p, p, p, dot_metadata(Layout.from_shape((m, k)), Layout.from_shape((k, n))), 0)
        K.call_ops_matmul_ex(DType.I8, DType.I32, 0, p, p, p,
                             dot_metadata(Layout.from_shape((m, k)), Layout.from_shape((k, n))), is_dot=True)
    for bshape in ((0, 4, 4), (3, 0, 4)):
        la = Layout.from_shape(bshape)
        lb = Layout.from_shape((bshape[0], bshape[2], 5))
        K.call_ops_matmul(K.matmul.F16, 0, p, p, p, matmul_metadata(la, lb, Layout.from_shape((bshape[0], bshape[1], 5))), 0)
    K.call_ops_cast(K.cast.F32_BF16, 0, p, p, cast_metadata(Layout.from_shape((0,))), 0)
    K.call_ops_contiguous(K.contiguous.BF16, 0, p, p, cast_metadata(Layout.from_shape((4, 0))), 0)
    K.call_ops_swiglu(DType.BF16, 0, p, p, p, p,
                      swiglu_metadata(Layout.from_shape((0, 8)), Layout.from_shape((8, 16)), Layout.from_shape((8, 16))))
    K.call_ops_linear(DType.BF16, 0, p, p, p, p,
                      [*matmul_metadata(Layout.from_shape((0, 8)), Layout.from_shape((8, 4)), Layout.from_shape((0, 4))), 1, 0])
    shapes = [(0, 3), (3, 4)]
    parsed = ParsedEinsum.parse("ij,jk->ik", shapes)
    K.call_ops_einsum(K.einsum.BF16, 0, [p, p], p,
                      einsum_metadata(parsed, [Layout.from_shape(s) for s in shapes], Layout.from_shape((0, 4))), 0)
    K.call_ops_conv(K.conv2d.BF16, 0, p, p, p, conv2d_metadata(0, 3, 4, (5, 5), (3, 3)), 0)
    torch.cuda.synchronize()
    assert K.launch_count() == before
    assert K.last_status(0) == 0
    assert bool((buf == 7).all().item())
