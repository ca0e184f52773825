"""Pins the CPU oracle (oracle/) before anything is checked against it:
  1. the reference's own known-answer tests for matmul / dot, re-expressed on the same
     metadata wire format (values and metadata from
     crates/hodu_cpu_kernels/tests/ops_matrix.rs:9-147 and
     crates/hodu_cuda_kernels/tests/ops_matrix.rs:18-262);
  2. golden outputs of the reference's C kernels (tests/golden/reference_cpu_kernels.npz,
     made by tests/golden/make_golden.py);
  3. where oracle/_ref is present, the compiled reference kernels on fresh random cases.
No GPU involved."""
import ctypes
import os

import numpy as np
import pytest

from hodu_b200.layout import Layout
from hodu_b200.op_metadatas import cast_metadata, dot_metadata, matmul_metadata
from oracle import oracle as O

GOLDEN = np.load(os.path.join(os.path.dirname(__file__), "golden", "reference_cpu_kernels.npz"))

# (name, is_dot, lhs, rhs, metadata, expected) -- the reference's eight f32 cases
KNOWN = [
    ("cpu_matmul_f32_2d", False, [1, 2, 3, 4, 5, 6], [7, 8, 9, 10, 11, 12],
     [4, 2, 2, 0, 2, 3, 3, 2, 3, 1, 2, 1, 0, 0, 2, 3, 2], [58, 64, 139, 154]),
    ("cpu_matmul_f32_batch", False, [1, 2, 3, 4, 2, 3, 4, 5], [5, 6, 7, 8, 6, 7, 8, 9],
     [8, 3, 3, 1, 2, 2, 2, 2, 2, 2, 2, 4, 2, 1, 4, 2, 1, 0, 0, 2, 2, 2], [19, 22, 43, 50, 36, 41, 64, 73]),
    ("cpu_dot_f32_simple", True, [1, 2, 3, 4, 5, 6], [7, 8, 9, 10, 11, 12],
     [2, 3, 2, 3, 1, 2, 1, 0, 0], [58, 64, 139, 154]),
    ("cuda_dot_f32_simple", True, [1, 2, 3, 4, 5, 6], [7, 8, 9, 10, 11, 12],
     [2, 3, 2, 3, 1, 2, 1, 0, 0], [58, 64, 139, 154]),
    ("cuda_matmul_f32_2d", False, [1, 2, 3, 4, 5, 6], [7, 8, 9, 10, 11, 12],
     [4, 2, 2, 0, 2, 3, 3, 2, 3, 1, 2, 1, 0, 0, 2, 3, 2], [58, 64, 139, 154]),
    ("cuda_matmul_f32_square", False, [1, 2, 3, 4, 5, 6, 7, 8, 9], [9, 8, 7, 6, 5, 4, 3, 2, 1],
     [9, 2, 2, 0, 3, 3, 3, 3, 3, 1, 3, 1, 0, 0, 3, 3, 3], [30, 24, 18, 84, 69, 54, 138, 114, 90]),
    ("cuda_dot_f32_identity", True, [1, 0, 0, 0, 1, 0, 0, 0, 1], [1, 0, 0, 0, 1, 0, 0, 0, 1],
     [3, 3, 3, 3, 1, 3, 1, 0, 0], [1, 0, 0, 0, 1, 0, 0, 0, 1]),
    ("cuda_matmul_f32_batch_rhs2d", False, [1, 2, 3, 4, 5, 6, 7, 8, 9, 10, 11, 12], [1, 0, 0, 1, 1, 1],
     [8, 3, 2, 1, 2, 2, 3, 3, 2, 2, 6, 3, 1, 2, 1, 0, 0, 2, 3, 2], [4, 5, 10, 11, 16, 17, 22, 23]),
]


@pytest.mark.parametrize("case", KNOWN, ids=[c[0] for c in KNOWN])
def test_reference_known_answers(case):
    _, is_dot, lhs, rhs, md, want = case
    lhs, rhs = np.array(lhs, dtype=np.float32), np.array(rhs, dtype=np.float32)
    want = np.array(want, dtype=np.float32)
    assert np.array_equal(O.matmul(lhs, rhs, md, O.F32, is_dot=is_dot), want)      # numpy form
    assert np.array_equal(O.matmul_c(lhs, rhs, md, O.F32, is_dot=is_dot), want)    # C restatement


def _golden_case(name):
    return (GOLDEN[name + "__lhs"], GOLDEN[name + "__rhs"], [int(x) for x in GOLDEN[name + "__md"]],
            GOLDEN[name + "__out"], str(GOLDEN[name + "__fn"]))


@pytest.mark.parametrize("name", ["dot_f32_blas", "dot_f32_fallback", "dot_f32_blas_rhs_t", "dot_f32_fallback_rhs_t",
                                  "matmul_f32_fallback_bcast", "matmul_f32_blas_bcast_view",
                                  "matmul_f32_fallback_2batch"])
def test_golden_f32(name):
    lhs, rhs, md, want, fn = _golden_case(name)
    is_dot = "_dot_" in fn
    got_c = O.matmul_c(lhs, rhs, md, O.F32, is_dot=is_dot)
    got_np = O.matmul(lhs, rhs, md, O.F32, is_dot=is_dot)
    # same products, possibly another summation order (sgemm, blocked fallback): 1e-5 of scale
    assert O.rel_err(got_c, want) < 1e-5
    assert O.rel_err(got_np, want) < 1e-5
    if fn.startswith("hodu_cpu_matmul_f32_fallback"):
        assert np.array_equal(got_c, want)  # identical k-ordered sum


@pytest.mark.parametrize("name,out_dt", [("dot_i32", O.I32), ("matmul_i32", O.I32)])
def test_golden_i32(name, out_dt):
    lhs, rhs, md, want, fn = _golden_case(name)
    is_dot = "_dot_" in fn
    assert np.array_equal(O.matmul_c(lhs, rhs, md, O.I32, O.I32, is_dot=is_dot), want)
    assert np.array_equal(O.matmul(lhs, rhs, md, O.I32, O.I32, is_dot=is_dot), want)


def test_golden_i8_paths():
    # i8 -> i32 of the oracle == reference cast_i8_to_i32 + dot_i32 on the same i8 operands
    lhs32, rhs32, md, want32, _ = _golden_case("dot_i32")
    lhs8, rhs8, md8, want8, _ = _golden_case("dot_i8_wrapped")
    assert np.array_equal(lhs32, lhs8.astype(np.int32).reshape(-1))
    assert np.array_equal(GOLDEN["cast_i8_to_i32__out"], O.widen(GOLDEN["cast_i8_to_i32__in"], O.I8).reshape(-1))
    assert np.array_equal(O.matmul(lhs8, rhs8, md8, O.I8, O.I32, is_dot=True), want32)
    assert np.array_equal(O.matmul_c(lhs8, rhs8, md8, O.I8, O.I32, is_dot=True), want32)
    # i8 -> i8: the reference CPU kernel's own output is the exact sum wrapped to 8 bits
    assert np.array_equal(O.matmul(lhs8, rhs8, md8, O.I8, O.I8, is_dot=True), want8)
    assert np.array_equal(O.matmul_c(lhs8, rhs8, md8, O.I8, O.I8, is_dot=True), want8)


def test_golden_widening_casts():
    assert np.array_equal(O.bf16_to_f32(GOLDEN["cast_bf16_to_f32__in"]).view(np.uint32),
                          GOLDEN["cast_bf16_to_f32__out"].view(np.uint32))
    got, want = O.f16_to_f32(GOLDEN["cast_f16_to_f32__in"]), GOLDEN["cast_f16_to_f32__out"]
    nan = np.isnan(want)
    assert np.array_equal(np.isnan(got), nan)
    assert np.array_equal(got[~nan], want[~nan])
    # e4m3 codes with exponent field < 15 mean the same in the reference's C codec and in OCP e4m3fn
    assert np.array_equal(O.e4m3_to_f32(GOLDEN["cast_f8e4m3_to_f32__in"]), GOLDEN["cast_f8e4m3_to_f32__out"])


def test_golden_silu():
    got, want = O.silu(GOLDEN["silu_f32__in"]), GOLDEN["silu_f32__out"]
    assert np.max(np.abs(got - want)) <= 2e-7 * max(1.0, float(np.max(np.abs(want))))
    out = np.zeros_like(want)
    O.clib().oracle_silu_f32(GOLDEN["silu_f32__in"].ctypes.data_as(ctypes.c_void_p),
                             out.ctypes.data_as(ctypes.c_void_p), ctypes.c_size_t(out.size))
    assert np.max(np.abs(out - want)) <= 2e-7 * max(1.0, float(np.max(np.abs(want))))


def test_narrowing_codecs_agree_c_numpy_torch():
    """The three independent statements of RNE (+ saturation for e4m3) agree bit for bit."""
    import torch
    rng = np.random.default_rng(7)
    x = np.concatenate([rng.standard_normal(20000).astype(np.float32) * s for s in (1e-6, 1e-3, 1.0, 64.0, 500.0, 7e4)])
    x = np.concatenate([x, np.array([0.0, -0.0, 448, 449, 464, 480, -448, -1e9, 1e9, np.inf, -np.inf, 65504, 65520,
                                     2.0 ** -9, 2.0 ** -10, 1.5 * 2.0 ** -10, 2.0 ** -24, 2.0 ** -25, 3 * 2.0 ** -26],
                                    dtype=np.float32)])
    c = O.clib()
    sub = x[::13]
    assert np.array_equal(O.f32_to_bf16(x), torch.from_numpy(x).bfloat16().view(torch.int16).numpy().view(np.uint16))
    assert np.array_equal(O.f32_to_f16(x), torch.from_numpy(x).half().view(torch.int16).numpy().view(np.uint16))
    assert np.array_equal(O.f32_to_e4m3(x),
                          torch.from_numpy(np.clip(x, -448, 448)).to(torch.float8_e4m3fn).view(torch.uint8).numpy())
    assert np.array_equal(np.array([c.oracle_f32_to_bf16(ctypes.c_float(v)) for v in sub], dtype=np.uint16),
                          O.f32_to_bf16(sub))
    assert np.array_equal(np.array([c.oracle_f32_to_f16(ctypes.c_float(v)) for v in sub], dtype=np.uint16),
                          O.f32_to_f16(sub))
    assert np.array_equal(np.array([c.oracle_f32_to_e4m3(ctypes.c_float(v)) for v in sub], dtype=np.uint8),
                          O.f32_to_e4m3(sub))
    # NaN: quiet NaN out, sign kept
    nan = np.array([np.nan, -np.nan], dtype=np.float32)
    assert np.all(np.isnan(O.bf16_to_f32(O.f32_to_bf16(nan))))
    assert np.array_equal(O.f32_to_e4m3(nan) & 0x7F, np.array([0x7F, 0x7F], dtype=np.uint8))
    # e4m3 decode of all 256 codes == torch's float8_e4m3fn
    codes = np.arange(256, dtype=np.uint8)
    t = torch.from_numpy(codes).view(torch.float8_e4m3fn).float().numpy()
    mine = O.e4m3_to_f32(codes)
    assert np.array_equal(np.isnan(t), np.isnan(mine)) and np.array_equal(t[~np.isnan(t)], mine[~np.isnan(t)])
    assert float(np.nanmax(mine)) == 448.0


def test_cast_indices_strided():
    lay = Layout((3, 4), (1, 3), 2)  # a transposed view with an offset
    md = cast_metadata(lay)
    idx = np.zeros(12, dtype=np.uint64)
    O.clib().oracle_cast_indices((ctypes.c_size_t * len(md))(*md), idx.ctypes.data_as(ctypes.c_void_p))
    want = [2 + i * 1 + j * 3 for i in range(3) for j in range(4)]
    assert idx.tolist() == want


needs_ref = pytest.mark.skipif(O.ref() is None, reason="oracle/_ref not built (no reference tree on this machine)")


@needs_ref
@pytest.mark.parametrize("seed", range(4))
def test_against_compiled_reference_random(seed):
    rng = np.random.default_rng(100 + seed)
    ref = O.ref()
    bdims = [(), (3,), (2, 3)][seed % 3]
    m, k, n = [int(v) for v in rng.integers(1, 40, size=3)]
    lshape = (*bdims, m, k)
    rshape = ((1,) * len(bdims) if seed % 2 else bdims) + (k, n)
    a = rng.standard_normal(lshape).astype(np.float32)
    b = rng.standard_normal(rshape).astype(np.float32)
    la, lb = Layout.from_shape(lshape), Layout.from_shape(rshape)
    if seed >= 2:  # transposed inner view of the rhs
        b = np.ascontiguousarray(np.swapaxes(b, -1, -2))
        lb = Layout.from_shape(b.shape).transpose(-1, -2)
    out_l = Layout.from_shape((*bdims, m, n))
    md = matmul_metadata(la, lb, out_l)
    want = np.zeros(out_l.size(), dtype=np.float32)
    ref.call("hodu_cpu_matmul_f32_fallback", a, b, want, md)
    assert np.array_equal(O.matmul_c(a, b, md, O.F32), want)
    assert O.rel_err(O.matmul(a, b, md, O.F32), want) < 1e-5
    # integer twin
    ai = rng.integers(-127, 128, size=lshape, dtype=np.int8).astype(np.int32)
    bi = rng.integers(-127, 128, size=b.shape, dtype=np.int8).astype(np.int32)
    wi = np.zeros(out_l.size(), dtype=np.int32)
    ref.call("hodu_cpu_matmul_i32", ai, bi, wi, md)
    assert np.array_equal(O.matmul_c(ai, bi, md, O.I32), wi)
    assert np.array_equal(O.matmul(ai, bi, md, O.I32), wi)


@needs_ref
def test_reference_per_dtype_kernels_are_not_the_oracle():
    """Documents why: the reference's bf16 CPU matmul re-rounds (by truncation) at every k, so
    it drifts from the widened-f32 result far beyond the parity bar at K = 2048."""
    rng = np.random.default_rng(5)
    a = (rng.standard_normal((8, 2048)) / np.sqrt(2048)).astype(np.float32)
    b = (rng.standard_normal((2048, 8)) / np.sqrt(2048)).astype(np.float32)
    ab, bb = O.f32_to_bf16(a), O.f32_to_bf16(b)
    md = dot_metadata(Layout.from_shape(a.shape), Layout.from_shape(b.shape))
    ref_out = np.zeros(64, dtype=np.uint16)
    O.ref().call("hodu_cpu_dot_bf16", ab, bb, ref_out, md)
    want = O.widen(O.matmul(ab, bb, md, O.BF16, is_dot=True), O.BF16)
    assert O.rel_err(O.bf16_to_f32(ref_out), want) > 1e-2


# ---------------------------------------------------------------- einsum and Linear-with-bias
from hodu_b200.einsum import ParsedEinsum, einsum_metadata  # noqa: E402

GOLDEN_EL = np.load(os.path.join(os.path.dirname(__file__), "golden", "reference_einsum_linear.npz"))

# The reference's own einsum known answers that are matrix products
# (crates/hodu_cpu_kernels/tests/ops_einsum.rs:87-143,233-280,282-326,330-395).
EINSUM_KNOWN = [
    ("ij,jk->ik", [(2, 3), (3, 4)], [1, 2, 3, 4, 5, 6], list(range(1, 13)), [38, 44, 50, 56, 83, 98, 113, 128]),
    ("i,j->ij", [(3,), (2,)], [1, 2, 3], [4, 5], [4, 5, 8, 10, 12, 15]),
    ("i,i->", [(3,), (3,)], [1, 2, 3], [4, 5, 6], [32]),
    ("bij,bjk->bik", [(2, 2, 3), (2, 3, 2)], list(range(1, 13)), list(range(1, 13)),
     [22, 28, 49, 64, 220, 244, 301, 334]),
]


@pytest.mark.parametrize("case", EINSUM_KNOWN, ids=[c[0] for c in EINSUM_KNOWN])
def test_reference_einsum_known_answers(case):
    eq, shapes, a, b, want = case
    parsed = ParsedEinsum.parse(eq, shapes)
    md = einsum_metadata(parsed, [Layout.from_shape(s) for s in shapes],
                         Layout.from_shape(tuple(parsed.compute_output_shape())))
    got = O.einsum([np.array(a, dtype=np.float32), np.array(b, dtype=np.float32)], md, O.F32)
    assert np.array_equal(got, np.array(want, dtype=np.float32))


EINSUM_GOLDEN = sorted({k.split("__")[0] for k in GOLDEN_EL.files if k.startswith("einsum_")})


@pytest.mark.parametrize("key", EINSUM_GOLDEN)
def test_golden_einsum(key):
    md = [int(v) for v in GOLDEN_EL[key + "__md"]]
    ins = [GOLDEN_EL[key + "__in0"], GOLDEN_EL[key + "__in1"]]
    want = GOLDEN_EL[key + "__out"]
    if key.endswith("_i32"):
        assert np.array_equal(O.einsum(ins, md, O.I32), want)
    else:
        # same sum, numpy's order of additions instead of the reference's k-order
        assert O.rel_err(O.einsum(ins, md, O.F32), want) <= 2e-6


def test_golden_linear_f32():
    x, w, bias = GOLDEN_EL["linear_f32__x"], GOLDEN_EL["linear_f32__w"], GOLDEN_EL["linear_f32__bias"]
    for each in (True, False):  # f32 storage: both rounding forms are the same arithmetic
        got = O.linear(x, w.T, bias, O.F32, round_each_op=each)
        assert O.rel_err(got, GOLDEN_EL["linear_f32__out"]) <= 2e-6


def test_linear_rounding_forms_differ_for_bf16():
    rng = np.random.default_rng(5)
    x = O.widen(O.narrow(rng.standard_normal((8, 64)).astype(np.float32), O.BF16), O.BF16)
    w = O.widen(O.narrow(rng.standard_normal((64, 16)).astype(np.float32), O.BF16), O.BF16)
    b = O.widen(O.narrow(rng.standard_normal(16).astype(np.float32), O.BF16), O.BF16)
    each, once = O.linear(x, w, b, O.BF16, True), O.linear(x, w, b, O.BF16, False)
    assert O.rel_err(O.widen(each, O.BF16), O.widen(once, O.BF16)) <= 1e-2
    assert not np.array_equal(each, once)  # two roundings vs one


def test_einsum_against_compiled_reference_random():
    ref = O.ref()
    if ref is None or not hasattr(ref.base, "hodu_cpu_einsum_f32"):
        pytest.skip("oracle/_ref not built (reference tree not mounted)")
    rng = np.random.default_rng(11)
    for eq, shapes in [("ij,jk->ik", [(9, 14), (14, 5)]), ("bhqd,bhkd->bhqk", [(2, 2, 3, 4), (2, 2, 5, 4)]),
                       ("ik,jk->ji", [(6, 7), (4, 7)])]:
        parsed = ParsedEinsum.parse(eq, shapes)
        ol = Layout.from_shape(tuple(parsed.compute_output_shape()))
        md = einsum_metadata(parsed, [Layout.from_shape(s) for s in shapes], ol)
        ins = [rng.standard_normal(s).astype(np.float32) for s in shapes]
        want = np.zeros(ol.size(), dtype=np.float32)
        ref.einsum("hodu_cpu_einsum_f32", ins, want, md)
        assert O.rel_err(O.einsum(ins, md, O.F32), want) <= 2e-6


# ---------------------------------------------------------------- conv2d
from hodu_b200.op_metadatas import conv2d_metadata  # noqa: E402

GOLDEN_CONV = np.load(os.path.join(os.path.dirname(__file__), "golden", "reference_conv2d.npz"))
CONV_GOLDEN = sorted({k.split("__")[0] for k in GOLDEN_CONV.files})


def test_reference_conv2d_known_answers():
    # crates/hodu_cpu_kernels/tests/ops_conv.rs:95-147 and :150-202
    x = np.arange(1, 10, dtype=np.float32)
    md = conv2d_metadata(1, 1, 1, (3, 3), (2, 2))
    assert md == [4, 1, 1, 1, 3, 3, 2, 2, 2, 2, 1, 1, 0, 0, 1, 1, 0, 0]
    assert np.array_equal(O.conv2d(x, np.array([1, 0, 0, 1], dtype=np.float32), md, O.F32), [6, 8, 12, 14])
    md = conv2d_metadata(1, 1, 1, (3, 3), (3, 3), padding=(1, 1))
    assert md[8:10] == [3, 3]
    w = np.array([0, 0, 0, 0, 1, 0, 0, 0, 0], dtype=np.float32)
    assert np.array_equal(O.conv2d(x, w, md, O.F32), x)


@pytest.mark.parametrize("name", CONV_GOLDEN)
def test_golden_conv2d(name):
    md = [int(v) for v in GOLDEN_CONV[name + "__md"]]
    got = O.conv2d(GOLDEN_CONV[name + "__in"], GOLDEN_CONV[name + "__w"], md, O.F32)
    assert O.rel_err(got, GOLDEN_CONV[name + "__out"]) <= 2e-6
