"""GPU parity of conv2d as im2col + GEMM (`hodu_b200_conv2d`), through the C ABI, against the
oracle and the golden outputs of the reference's C kernel."""
import os

import numpy as np
import pytest

from hodu_b200 import CudaKernelError, DType, kernels as K
from hodu_b200.op_metadatas import conv2d_metadata
from oracle import oracle as O
from tests.gpu_util import canary_intact, from_dev, new_out, to_dev

pytestmark = pytest.mark.gpu
GOLDEN_CONV = np.load(os.path.join(os.path.dirname(__file__), "golden", "reference_conv2d.npz"))
TOL = {O.F32: 1e-4, O.BF16: 1e-2, O.F16: 1e-2}


def run_conv(x_bits, w_bits, md, dt):
    n_out = int(md[0])
    out = new_out(n_out, dt)
    dx, dw = to_dev(x_bits), to_dev(w_bits)
    K.call_ops_conv(getattr(K.conv2d, str(DType(dt)).upper()), 0, dx.data_ptr(), dw.data_ptr(), out.data_ptr(), md, 0)
    taken = K.last_path()
    assert K.last_status(0) == 0
    assert canary_intact(out, n_out)
    return from_dev(out[:n_out], dt), taken


@pytest.mark.parametrize("name", sorted({k.split("__")[0] for k in GOLDEN_CONV.files}))
def test_conv2d_golden_reference_outputs(name):
    md = [int(v) for v in GOLDEN_CONV[name + "__md"]]
    got, _ = run_conv(GOLDEN_CONV[name + "__in"], GOLDEN_CONV[name + "__w"], md, O.F32)
    assert O.rel_err(got, GOLDEN_CONV[name + "__out"]) <= 1e-5


CASES = [
    # batch, Cin, Cout, (H, W), (KH, KW), stride, padding, dilation, dtype
    (4, 64, 128, (56, 56), (3, 3), (1, 1), (1, 1), (1, 1), O.BF16),     # ResNet-style 3x3
    (2, 128, 256, (28, 28), (3, 3), (2, 2), (1, 1), (1, 1), O.BF16),    # strided
    (2, 256, 512, (14, 14), (1, 1), (1, 1), (0, 0), (1, 1), O.F16),     # pointwise: no unfolding, N pitch 392 B not 16-aligned... relaid
    (2, 256, 512, (16, 16), (1, 1), (1, 1), (0, 0), (1, 1), O.BF16),    # pointwise, aligned: input is the rhs as it lies
    (1, 3, 64, (224, 224), (7, 7), (2, 2), (3, 3), (1, 1), O.BF16),     # stem: K = 147 (unaligned weight rows)
    (2, 32, 48, (33, 29), (3, 5), (1, 2), (2, 0), (2, 1), O.F16),       # odd everything, dilation
    (2, 64, 64, (32, 32), (3, 3), (1, 1), (1, 1), (1, 1), O.F32),       # f32 through split TF32
    (1, 2, 3, (5, 5), (3, 3), (1, 1), (0, 0), (1, 1), O.BF16),          # tiny: generic kernel
    # in_channels a multiple of 64, bf16 / f16: the implicit form (no unfolded copy)
    (3, 128, 96, (17, 13), (3, 3), (2, 1), (1, 2), (1, 2), O.F16),      # tiles straddle images, odd extents, stride, dilation, ragged Cout
    (2, 64, 256, (20, 24), (5, 5), (1, 1), (2, 2), (1, 1), O.BF16),     # 5x5; few pixel tiles: 64-wide channel tiles, four per pixel tile
    (8, 64, 256, (56, 56), (3, 3), (1, 1), (1, 1), (1, 1), O.BF16),     # 196 pixel tiles: 256-wide channel tiles
    (16, 64, 128, (28, 28), (3, 3), (1, 1), (1, 1), (1, 1), O.F16),     # 98 pixel tiles: 128-wide channel tiles (two k-blocks per stage)
    (4, 512, 512, (7, 7), (3, 3), (1, 1), (1, 1), (1, 1), O.BF16),      # deep layer: 2 pixel tiles x 8 channel tiles, 72 k-blocks
    (40, 64, 64, (9, 9), (3, 3), (1, 1), (0, 0), (1, 1), O.BF16),       # no padding; 1960 pixels: a ragged last tile
    (2, 192, 64, (31, 31), (3, 3), (3, 3), (1, 1), (1, 1), O.F16),      # three channel blocks, stride 3
]
IMPLICIT = lambda c: c[1] % 64 == 0 and c[8] in (O.BF16, O.F16) and c[4] != (1, 1)


@pytest.mark.parametrize("case", CASES, ids=[f"b{c[0]}c{c[1]}-{c[2]}_{c[3][0]}x{c[3][1]}_k{c[4][0]}x{c[4][1]}-{DType(c[8])}" for c in CASES])
def test_conv2d_vs_oracle(case):
    b, ci, co, hw, k, s, p, d, dt = case
    md = conv2d_metadata(b, ci, co, hw, k, s, p, d)
    rng = np.random.default_rng(ci * 7 + co)
    x = O.narrow(rng.standard_normal(b * ci * hw[0] * hw[1]).astype(np.float32), dt)
    w = O.narrow((rng.standard_normal(co * ci * k[0] * k[1]) / np.sqrt(ci * k[0] * k[1])).astype(np.float32), dt)
    before = K.launch_count()
    got, taken = run_conv(x, w, md, dt)
    launches = K.launch_count() - before
    want = O.conv2d(x, w, md, dt)
    assert O.rel_err(O.widen(got, dt), O.widen(want, dt)) <= TOL[dt]
    work = b * co * md[8] * md[9] * ci * k[0] * k[1]
    if work >= (1 << 24):
        assert taken == K._lib.PATH_TENSOR   # large enough: the tcgen05 kernel, relaid if need be
        if IMPLICIT(case):
            assert launches == 2             # re-lay input and weights, then the implicit GEMM: no unfolding pass


def test_conv2d_implicit_and_explicit_forms_agree():
    """The same convolution through both forms (the switch is read once per process, so the
    explicit form runs in a child process): equal within the bf16 bar, and equal to the oracle."""
    import subprocess
    import sys
    code = r'''
import sys, numpy as np
sys.path.insert(0, %r); sys.path.insert(0, %r)
from test_conv2d_gpu import run_conv
from hodu_b200.op_metadatas import conv2d_metadata
from oracle import oracle as O
md = conv2d_metadata(4, 64, 128, (28, 28), (3, 3), (1, 1), (1, 1), (1, 1))
rng = np.random.default_rng(1)
x = O.narrow(rng.standard_normal(4 * 64 * 28 * 28).astype(np.float32), O.BF16)
w = O.narrow((rng.standard_normal(128 * 64 * 9) / 24).astype(np.float32), O.BF16)
got, _ = run_conv(x, w, md, O.BF16)
np.save(sys.argv[1], got)
''' % (os.path.dirname(os.path.dirname(os.path.abspath(__file__))), os.path.dirname(os.path.abspath(__file__)))
    import tempfile
    outs = []
    for implicit in ("1", "0"):
        with tempfile.NamedTemporaryFile(suffix=".npy") as f:
            env = dict(os.environ, HODU_B200_CONV_IMPLICIT=implicit)
            r = subprocess.run([sys.executable, "-c", code, f.name], capture_output=True, text=True, timeout=600, env=env)
            assert r.returncode == 0, r.stderr[-2000:]
            outs.append(np.load(f.name))
    a, b = (O.widen(o, O.BF16) for o in outs)
    assert O.rel_err(a, b) <= 1e-2


def test_conv2d_argument_errors():
    md = conv2d_metadata(1, 1, 1, (3, 3), (2, 2))
    bad = list(md)
    bad[8] = 3                                     # wrong out_h
    with pytest.raises(CudaKernelError) as e:
        K.call_ops_conv(K.conv2d.F32, 0, 0x1000, 0x1000, 0x2000, bad)
    assert e.value.code == -2
    with pytest.raises(CudaKernelError) as e:
        K.call_ops_conv(K.conv2d.I8, 0, 0x1000, 0x1000, 0x2000, md)
    assert e.value.code == -1
    with pytest.raises(CudaKernelError) as e:
        K.call_ops_conv(K.conv2d.F32, 0, 0x1000, 0x1000, 0x2000, md[:-1])
    assert e.value.code == -2
