"""The five benchmark configurations: reduced sizes against the full oracle, and the full
sizes through properties that do not need a full CPU product (sampled rows against the
oracle, an exact checksum identity for the integer case)."""
import numpy as np
import pytest
import torch

from gpu_util import DEV, check_close, from_dev, gpu_matmul, to_dev
from hodu_b200 import DType, Layout, _lib
from hodu_b200 import kernels as K
from hodu_b200 import synthetic as S
from hodu_b200.op_metadatas import dot_metadata, matmul_metadata
from oracle import oracle as O

pytestmark = pytest.mark.gpu


def test_config1_f32_full_size():
    c = S.config1()
    a, b = c["a"], c["b"]
    md = dot_metadata(Layout.from_shape(a.shape), Layout.from_shape(b.shape))
    got, _ = gpu_matmul(a, b, md, O.F32, is_dot=True, plain_api=True)
    want = O.matmul(a, b, md, O.F32, is_dot=True)  # sgemm, as the reference's openblas build
    assert O.rel_err(got, want) <= 1e-4


def test_config2_bf16_batched_reduced_and_full():
    for scale, batches in ((8, 16), (1, 16)):
        c = S.config2(scale=scale, batches=batches)
        a, b = O.f32_to_bf16(c["a"]), O.f32_to_bf16(c["b"])
        l = Layout.from_shape(a.shape)
        md = matmul_metadata(l, l, l)
        got, path = gpu_matmul(a, b, md, O.BF16, plain_api=True)
        assert path == _lib.PATH_TENSOR
        want = O.matmul(a, b, md, O.BF16)
        assert O.rel_err(O.widen(got, O.BF16), O.widen(want, O.BF16)) <= 1e-2


def _device_dot(ta, tb, m, k, n, in_dt, out_dt, scales=(1.0, 1.0)):
    out = torch.empty(m * n, dtype={O.BF16: torch.int16, O.I32: torch.int32}[out_dt], device=DEV)
    md = dot_metadata(Layout.from_shape((m, k)), Layout.from_shape((k, n)))
    K.call_ops_matmul_ex(DType(in_dt), DType(out_dt), 0, ta.data_ptr(), tb.data_ptr(), out.data_ptr(), md,
                         scales[0], scales[1], 0, is_dot=True)
    assert K.last_status(0) == 0 and K.last_path() == _lib.PATH_TENSOR
    return out


def test_config3_e4m3_reduced_and_full_sampled_rows():
    c = S.config3(scale=8)
    a, b = O.f32_to_e4m3(c["a"]), O.f32_to_e4m3(c["b"])
    md = dot_metadata(Layout.from_shape(a.shape), Layout.from_shape(b.shape))
    got, _ = gpu_matmul(a, b, md, O.F8E4M3, O.BF16, (c["scale_a"], c["scale_b"]), is_dot=True)
    want = O.matmul(a, b, md, O.F8E4M3, O.BF16, c["scale_a"] * c["scale_b"], is_dot=True)
    assert O.rel_err(O.widen(got, O.BF16), O.widen(want, O.BF16)) <= 6e-2
    # full size: 64 sampled rows of C against the oracle
    c = S.config3()
    a, b = O.f32_to_e4m3(c["a"]), O.f32_to_e4m3(c["b"])
    d = a.shape[0]
    out = _device_dot(to_dev(a), to_dev(b), d, d, d, O.F8E4M3, O.BF16, (c["scale_a"], c["scale_b"]))
    rows = np.random.default_rng(0).choice(d, 64, replace=False)
    got = from_dev(out.view(d, d)[torch.from_numpy(rows).to(DEV)], O.BF16).reshape(64, d)
    want = np.matmul(O.e4m3_to_f32(a[rows]), O.e4m3_to_f32(b)) * np.float32(c["scale_a"] * c["scale_b"])
    want = O.widen(O.narrow(want.astype(np.float32), O.BF16), O.BF16)
    assert O.rel_err(O.widen(got, O.BF16), want) <= 6e-2
    assert abs(float(np.std(want)) - 90.5) < 3.0  # C ~ N(0, 8192) after scaling


def test_config4_i8_reduced_and_full_exact():
    c = S.config4(scale=8)
    a, b = c["a"], c["b"]
    md = dot_metadata(Layout.from_shape(a.shape), Layout.from_shape(b.shape))
    got, path = gpu_matmul(a, b, md, O.I8, O.I32, is_dot=True)
    assert path == _lib.PATH_TENSOR
    assert np.array_equal(got, O.matmul(a, b, md, O.I8, O.I32, is_dot=True))
    rows8 = dot_metadata(Layout.from_shape((8, a.shape[1])), Layout.from_shape(b.shape))
    assert np.array_equal(got.reshape(a.shape[0], -1)[:8].reshape(-1),
                          O.matmul_c(a[:8].copy(), b, rows8, O.I8, O.I32, is_dot=True))  # C restatement
    # full size: sampled rows bit-exact, plus the identity sum(C) == colsum(A) . rowsum(B)
    c = S.config4()
    a, b = c["a"], c["b"]
    d = a.shape[0]
    out = _device_dot(to_dev(a), to_dev(b), d, d, d, O.I8, O.I32)
    rows = np.random.default_rng(1).choice(d, 64, replace=False)
    got = from_dev(out.view(d, d)[torch.from_numpy(rows).to(DEV)], O.I32).reshape(64, d)
    want = np.rint(np.matmul(a[rows].astype(np.float64), b.astype(np.float64))).astype(np.int64)
    assert np.array_equal(got.astype(np.int64), want)
    total = int(out.sum(dtype=torch.int64).item())
    assert total == int(np.dot(a.astype(np.int64).sum(axis=0), b.astype(np.int64).sum(axis=1)))
    # every row checksum: C @ 1 == A @ (B @ 1)
    row_sums = out.view(d, d).sum(dim=1, dtype=torch.int64).cpu().numpy()
    assert np.array_equal(row_sums, a.astype(np.int64) @ b.astype(np.int64).sum(axis=1))
