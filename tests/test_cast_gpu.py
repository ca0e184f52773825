"""f32 <-> bf16 | f16 | f8e4m3 and i8 -> i32 on the device, bit-exact against the oracle's
codecs (round to nearest even; e4m3 saturating to +-448, NaN kept)."""
import numpy as np
import pytest

from gpu_util import canary_intact, from_dev, new_out, to_dev
from hodu_b200 import Layout
from hodu_b200 import kernels as K
from hodu_b200.op_metadatas import cast_metadata
from oracle import oracle as O

pytestmark = pytest.mark.gpu

NAMES = {O.F32: "F32", O.BF16: "BF16", O.F16: "F16", O.F8E4M3: "F8E4M3", O.I8: "I8", O.I32: "I32"}
SPECIAL = np.array([0.0, -0.0, 1.0, -1.0, 448, 449, 464, 480, -448, -500, 1e9, -1e9, np.inf, -np.inf, np.nan, 65504,
                    65520, 65536, 2.0 ** -9, 2.0 ** -10, 1.5 * 2.0 ** -10, 2.0 ** -24, 2.0 ** -25, 3 * 2.0 ** -26,
                    2.0 ** -126, 1e-40, 3.3895314e38, 1.0 + 2.0 ** -8, 1.0 + 3 * 2.0 ** -9], dtype=np.float32)


def run_cast(src_bits, layout, src_dt, dst_dt):
    t = to_dev(src_bits)
    n = layout.size()
    out = new_out(n, dst_dt)
    k = getattr(K.cast, f"{NAMES[src_dt]}_{NAMES[dst_dt]}")
    K.call_ops_cast(k, 0, t.data_ptr(), out.data_ptr(), cast_metadata(layout), 0)
    assert K.last_status(0) == 0
    assert canary_intact(out, n)
    return from_dev(out[:n], dst_dt)


def gather(src_bits, layout):
    flat = np.ascontiguousarray(src_bits).reshape(-1)
    v = np.lib.stride_tricks.as_strided(flat[layout.offset:], shape=layout.shape,
                                        strides=tuple(s * flat.itemsize for s in layout.strides))
    return np.ascontiguousarray(v).reshape(-1)


def equal_mod_nan(got, want, dt):
    if dt in (O.I32, O.I8):
        return np.array_equal(got, want)
    g, w = O.widen(got, dt), O.widen(want, dt)
    nan = np.isnan(w)
    return np.array_equal(np.isnan(g), nan) and np.array_equal(got[~nan], want[~nan])


@pytest.mark.parametrize("dst", [O.BF16, O.F16, O.F8E4M3])
@pytest.mark.parametrize("n", [1, 7, 16, 1000, (1 << 20) + 3])
def test_narrowing_contiguous(dst, n):
    rng = np.random.default_rng(n + dst)
    x = (rng.standard_normal(n) * rng.choice([1e-6, 1e-3, 1.0, 30.0, 600.0, 7e4], size=n)).astype(np.float32)
    x[: min(n, SPECIAL.size)] = SPECIAL[: min(n, SPECIAL.size)]
    got = run_cast(x, Layout.from_shape((n,)), O.F32, dst)
    assert equal_mod_nan(got, O.narrow(x, dst), dst)


@pytest.mark.parametrize("src", [O.BF16, O.F16, O.F8E4M3])
def test_widening_every_bit_pattern(src):
    bits = np.arange(256, dtype=np.uint8) if src == O.F8E4M3 else np.arange(65536, dtype=np.uint16)
    got = run_cast(bits, Layout.from_shape(bits.shape), src, O.F32)
    want = O.widen(bits, src)
    nan = np.isnan(want)
    assert np.array_equal(np.isnan(got), nan)
    assert np.array_equal(got[~nan].view(np.uint32), want[~nan].view(np.uint32))


def test_i8_to_i32():
    x = np.arange(-128, 128, dtype=np.int8).repeat(33)
    assert np.array_equal(run_cast(x, Layout.from_shape(x.shape), O.I8, O.I32), x.astype(np.int32))


@pytest.mark.parametrize("src,dst", [(O.F32, O.BF16), (O.F32, O.F8E4M3), (O.BF16, O.F32), (O.F8E4M3, O.F32), (O.F32, O.F16)])
def test_strided_and_offset_inputs(src, dst):
    rng = np.random.default_rng(9)
    base = O.narrow(rng.standard_normal(4 + 64 * 48).astype(np.float32) * 20, src)
    for lay in (Layout((48, 64), (1, 48), 0),            # transposed view
                Layout((64, 48), (48, 1), 3),            # offset that breaks 16-byte alignment
                Layout((5, 16, 3), (0, 48, 2), 1),       # broadcast (stride 0) outer dim, stepped inner
                Layout((64, 1, 48), (48, 7777, 1), 0)):  # extent-1 dim with a junk stride: still contiguous
        got = run_cast(base, lay, src, dst)
        want = O.narrow(O.widen(gather(base, lay), src), dst) if dst != O.F32 else O.widen(gather(base, lay), src)
        assert equal_mod_nan(got, want, dst)


def test_round_trip_is_idempotent():
    """narrow(widen(narrow(x))) == narrow(x): a property that holds at any size."""
    rng = np.random.default_rng(11)
    x = (rng.standard_normal(1 << 22) * 50).astype(np.float32)
    for dt in (O.BF16, O.F16, O.F8E4M3):
        once = run_cast(x, Layout.from_shape(x.shape), O.F32, dt)
        back = run_cast(once, Layout.from_shape(x.shape), dt, O.F32)
        twice = run_cast(back, Layout.from_shape(x.shape), O.F32, dt)
        assert np.array_equal(once, twice)


# The reference's six cast known answers (crates/hodu_cuda_kernels/tests/ops_cast.rs:48-89).
REF_CAST_KNOWN = [
    ("F32_I32", np.array([1.5, -2.7, 3.2, -4.9], dtype=np.float32), np.array([1, -2, 3, -4], dtype=np.int32)),
    ("I32_F32", np.array([1, -2, 3, -4], dtype=np.int32), np.array([1.0, -2.0, 3.0, -4.0], dtype=np.float32)),
    ("F32_U32", np.array([1.5, 2.7, 3.2, 4.9], dtype=np.float32), np.array([1, 2, 3, 4], dtype=np.uint32)),
    ("U32_F32", np.array([1, 2, 3, 4], dtype=np.uint32), np.array([1.0, 2.0, 3.0, 4.0], dtype=np.float32)),
    ("F64_F32", np.array([1.5, 2.7, 3.2, 4.9], dtype=np.float64), np.array([1.5, 2.7, 3.2, 4.9], dtype=np.float32)),
    ("F32_F64", np.array([1.5, 2.7, 3.2, 4.9], dtype=np.float32),
     np.array([1.5, 2.7, 3.2, 4.9], dtype=np.float32).astype(np.float64)),
]


@pytest.mark.parametrize("case", REF_CAST_KNOWN, ids=[c[0] for c in REF_CAST_KNOWN])
def test_reference_cast_known_answers(case):
    import torch
    name, src, want = case
    view = {np.dtype(np.uint32): np.int32}
    s_np = src.view(view.get(src.dtype, src.dtype))
    d_src = torch.from_numpy(s_np.copy()).to("cuda:0")
    d_out = torch.zeros(want.size * want.itemsize + 16, dtype=torch.uint8, device="cuda:0")
    K.call_ops_cast(getattr(K.cast, name), 0, d_src.data_ptr(), d_out.data_ptr(),
                    cast_metadata(Layout.from_shape(src.shape)), 0)
    assert K.last_status(0) == 0
    got = d_out.cpu().numpy()[: want.size * want.itemsize].view(want.dtype)
    assert np.array_equal(got, want)
    assert not d_out.cpu().numpy()[want.size * want.itemsize:].any()   # nothing written past the end


def test_cast_of_more_than_two_to_the_32_elements():
    """Maximum sizes: 2^32 + 4096 contiguous f32 elements to bf16 (the reference's CUDA cast indexes
    with uint32_t, crates/hodu_cuda_kernels/kernels/ops_cast.cu:7-30).  Slices at the start, around
    the 2^32 boundary and at the very end must equal round-to-nearest-even bit for bit."""
    import torch
    n = (1 << 32) + 4096
    dev = torch.device("cuda:0")
    src = torch.empty(n, dtype=torch.float32, device=dev)
    step = 1 << 28
    g = torch.Generator(device=dev).manual_seed(3)
    for lo in range(0, n, step):                     # filled in pieces: no 17 GB temporary
        hi = min(n, lo + step)
        src[lo:hi].normal_(generator=g)
    out = torch.zeros(n + 64, dtype=torch.int16, device=dev)
    K.call_ops_cast(K.cast.F32_BF16, 0, src.data_ptr(), out.data_ptr(), cast_metadata(Layout.from_shape((n,))), 0)
    assert K.last_status(0) == 0
    for lo, hi in ((0, 4096), ((1 << 31) - 2048, (1 << 31) + 2048), ((1 << 32) - 2048, (1 << 32) + 2048), (n - 4096, n)):
        want = src[lo:hi].to(torch.bfloat16).view(torch.int16)
        assert torch.equal(out[lo:hi], want), (lo, hi)
    assert not bool(out[n:].any().item())            # nothing written past the end
    del src, out
    torch.cuda.empty_cache()
