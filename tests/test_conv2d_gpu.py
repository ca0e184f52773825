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
]


@pytest.mark.parametrize("case", CASES, ids=[f"b{c[0]}c{c[1]}-{c[2]}_{c[3][0]}x{c[3][1]}_k{c[4][0]}x{c[4][1]}-{DType(c[8])}" for c in CASES])
def test_conv2d_vs_oracle(case):
    b, ci, co, hw, k, s, p, d, dt = case
    md = conv2d_metadata(b, ci, co, hw, k, s, p, d)
    rng = np.random.default_rng(ci * 7 + co)
    x = O.narrow(rng.standard_normal(b * ci * hw[0] * hw[1]).astype(np.float32), dt)
    w = O.narrow((rng.standard_normal(co * ci * k[0] * k[1]) / np.sqrt(ci * k[0] * k[1])).astype(np.float32), dt)
    got, taken = run_conv(x, w, md, dt)
    want = O.conv2d(x, w, md, dt)
    assert O.rel_err(O.widen(got, dt), O.widen(want, dt)) <= TOL[dt]
    if b * co * md[8] * md[9] * ci * k[0] * k[1] >= (1 << 24):
        assert taken == K._lib.PATH_TENSOR   # large enough: the tcgen05 kernel, relaid if need be


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
