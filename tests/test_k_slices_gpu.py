"""Products with too few output tiles for the SMs: the tensor-core kernel cuts K into slices that
the CTAs of a cluster share, and adds the slices through distributed shared memory.  Parity
against the CPU oracle over operand layouts, dtypes, tails in M, N and K, batches, scale and
bias; one launch each, and (in a child process with the debug prints on) proof that slices
were in fact used."""
import os
import subprocess
import sys

import numpy as np
import pytest

from hodu_b200 import kernels as K
from hodu_b200.dtype import DType
from hodu_b200.layout import Layout
from hodu_b200.op_metadatas import dot_metadata, matmul_metadata
from oracle import oracle as O
from gpu_util import check_close, gpu_matmul
from test_einsum_linear_gpu import run_linear
from test_gemm_gpu import rand_storage

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

CASES = [
    # M, K, N, batches, in dtype, out dtype, lhs K-contiguous?, rhs N-contiguous?
    (512, 2048, 512, 0, O.BF16, O.BF16, True, True),
    (1024, 4096, 1024, 0, O.BF16, O.BF16, True, True),      # 32 tiles of 128 x 256, four slices
    (1536, 1536, 1536, 0, O.BF16, O.BF16, True, True),      # on the border: sliced or whole, one launch either way
    (1000, 3000, 776, 0, O.BF16, O.BF16, True, True),       # tails in M, N and K
    (320, 1000, 200, 0, O.F16, O.F32, False, True),         # lhs M-contiguous, 4-byte output
    (128, 4096, 520, 0, O.BF16, O.BF16, True, False),       # rhs K-contiguous, 8 columns in the last tile
    (384, 2048, 384, 0, O.F16, O.F16, False, False),
    (512, 4096, 512, 4, O.BF16, O.BF16, True, True),        # batched: tiles x batches clusters
    (512, 8192, 1024, 0, O.I8, O.I32, True, True),          # integer partial sums add exactly
    (256, 4096, 256, 0, O.I8, O.I8, True, False),
    (256, 4096, 384, 0, O.F8E4M3, O.BF16, True, True),
    (128, 8192, 128, 0, O.F8E4M3, O.F8E4M3, True, False),
    (64, 8192, 2048, 0, O.BF16, O.F32, True, True),
]


def _ids(c):
    return f"{c[0]}x{c[1]}x{c[2]}b{c[3]}-{DType(c[4])}-{DType(c[5])}-{int(c[6])}{int(c[7])}"


@pytest.mark.parametrize("case", CASES, ids=[_ids(c) for c in CASES])
def test_k_slices_match_oracle(case):
    m, k, n, batches, in_dt, out_dt, a_kmajor, b_nmajor = case
    rng = np.random.default_rng(m * 7 + k * 3 + n)
    bshape = (batches,) if batches else ()
    a_shape = (*bshape, m, k) if a_kmajor else (*bshape, k, m)
    b_shape = (*bshape, k, n) if b_nmajor else (*bshape, n, k)
    a = rand_storage(rng, in_dt, a_shape)
    b = rand_storage(rng, in_dt, b_shape)
    la = Layout.from_shape(a_shape) if a_kmajor else Layout.from_shape(a_shape).transpose(-2 % len(a_shape), -1 % len(a_shape))
    lb = Layout.from_shape(b_shape) if b_nmajor else Layout.from_shape(b_shape).transpose(-2 % len(b_shape), -1 % len(b_shape))
    if batches:
        md = matmul_metadata(la, lb, Layout.from_shape((batches, m, n)))
    else:
        md = dot_metadata(la, lb)
    scales = (1 / 16, 1 / 8) if in_dt == O.F8E4M3 else (1.0, 1.0)
    before = K.launch_count()
    got, taken = gpu_matmul(a, b, md, in_dt, out_dt, scales=scales, is_dot=not batches)
    assert K.launch_count() - before == 1
    assert taken == K._lib.PATH_TENSOR
    want = O.matmul(a, b, md, in_dt, out_dt, scales[0] * scales[1], is_dot=not batches)
    if in_dt == O.I8:
        assert np.array_equal(got, want)
    else:
        tol = {O.F32: 1e-4, O.BF16: 1e-2, O.F16: 1e-2, O.F8E4M3: 7e-2}[out_dt] if in_dt != O.F8E4M3 else 7e-2
        check_close(got, want, out_dt, tol)


def _random_cases(n_cases, seed):
    rng = np.random.default_rng(seed)
    out = []
    while len(out) < n_cases:
        m = int(rng.choice([64, 128, 200, 256, 384, 500, 512, 768, 1000]))
        n = int(rng.choice([64, 128, 192, 256, 320, 512, 776, 1024, 1536]))
        k = int(rng.choice([512, 1000, 1024, 2048, 3000, 4096, 6144]))
        a_kmajor, b_nmajor = bool(rng.integers(2)), bool(rng.integers(2))
        dt = int(rng.choice([O.BF16, O.F16]))
        # TMA takes the operand as it lies only when the pitch of its contiguous index is a multiple of 16 bytes
        if ((m if not a_kmajor else k) * 2) % 16 or ((n if b_nmajor else k) * 2) % 16:
            continue
        out.append((m, k, n, dt, a_kmajor, b_nmajor))
    return out


RANDOM = _random_cases(24, 20241)


@pytest.mark.parametrize("case", RANDOM, ids=[f"{c[0]}x{c[1]}x{c[2]}-{DType(c[3])}-{int(c[4])}{int(c[5])}" for c in RANDOM])
def test_random_products_with_few_tiles(case):
    """Fixed-seed sweep over shapes with few output tiles (most run with 2, 4 or 8 K slices) and all
    four layout combinations: one launch each, oracle parity."""
    m, k, n, dt, a_kmajor, b_nmajor = case
    rng = np.random.default_rng(m + 3 * k + 5 * n)
    a = rand_storage(rng, dt, (m, k) if a_kmajor else (k, m))
    b = rand_storage(rng, dt, (k, n) if b_nmajor else (n, k))
    la = Layout.from_shape((m, k)) if a_kmajor else Layout.from_shape((k, m)).transpose(0, 1)
    lb = Layout.from_shape((k, n)) if b_nmajor else Layout.from_shape((n, k)).transpose(0, 1)
    md = dot_metadata(la, lb)
    before = K.launch_count()
    got, taken = gpu_matmul(a, b, md, dt, dt, is_dot=True)
    assert K.launch_count() - before == 1 and taken == K._lib.PATH_TENSOR
    check_close(got, O.matmul(a, b, md, dt, dt, 1.0, is_dot=True), dt, 1e-2)


@pytest.mark.parametrize("flags", [K._lib.LINEAR_ROUND_EACH_OP, K._lib.LINEAR_ROUND_ONCE], ids=["each_op", "once"])
def test_k_slices_with_bias(flags):
    """hodu_nn::Linear on few tokens: the bias is added once, by the slice that stores the chunk."""
    m, k, n = 192, 4096, 1024
    rng = np.random.default_rng(5)
    x = O.narrow(rng.standard_normal((m, k)).astype(np.float32), O.BF16)
    w = O.narrow((rng.standard_normal((n, k)) / np.sqrt(k)).astype(np.float32), O.BF16)
    b = O.narrow(rng.standard_normal(n).astype(np.float32), O.BF16)
    before = K.launch_count()
    got, taken = run_linear(x, w, b, Layout.from_shape((m, k)), Layout.from_shape((n, k)), Layout.from_shape((n,)),
                            O.BF16, flags)
    assert K.launch_count() - before == 1 and taken == K._lib.PATH_TENSOR
    want = O.linear(O.widen(x, O.BF16).reshape(m, k), O.widen(w, O.BF16).reshape(n, k).T, O.widen(b, O.BF16),
                    O.BF16, round_each_op=(flags == K._lib.LINEAR_ROUND_EACH_OP))
    assert O.rel_err(O.widen(got, O.BF16), O.widen(want, O.BF16)) <= 1e-2


def test_k_slices_are_deterministic():
    """The slices are added in a fixed order: repeated calls give the same bits."""
    m, k, n = 512, 4096, 512
    rng = np.random.default_rng(11)
    a = rand_storage(rng, O.BF16, (m, k))
    b = rand_storage(rng, O.BF16, (k, n))
    md = dot_metadata(Layout.from_shape((m, k)), Layout.from_shape((k, n)))
    first, _ = gpu_matmul(a, b, md, O.BF16, O.F32, is_dot=True)
    for _ in range(5):
        again, _ = gpu_matmul(a, b, md, O.BF16, O.F32, is_dot=True)
        assert np.array_equal(first, again)


CHILD = r"""
import sys
import numpy as np, torch
from hodu_b200 import kernels as K
from hodu_b200.layout import Layout
from hodu_b200.op_metadatas import dot_metadata
for (m, k, n) in [(512, 2048, 512), (1024, 4096, 1024), (128, 4096, 4096)]:
    a = (torch.randn(m, k, device="cuda") / 8).bfloat16(); b = (torch.randn(k, n, device="cuda") / 8).bfloat16()
    c = torch.zeros(m, n, device="cuda", dtype=torch.bfloat16)
    md = dot_metadata(Layout.from_shape((m, k)), Layout.from_shape((k, n)))
    K.call_ops_dot(K.dot.BF16, 0, a.data_ptr(), b.data_ptr(), c.data_ptr(), md, 0)
    torch.cuda.synchronize()
    ref = a.float() @ b.float()
    assert (c.float() - ref).abs().max().item() <= 2e-2 * ref.abs().max().item()
print("ok")
"""


def test_debug_prints_show_the_slices():
    env = dict(os.environ, HODU_B200_DEBUG="1", PYTHONPATH=ROOT)
    r = subprocess.run([sys.executable, "-c", CHILD], cwd=ROOT, env=env, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    lines = [l for l in r.stderr.splitlines() if "K slice(s)" in l]
    assert len(lines) == 3
    sliced = [int(l.split(" K slice(s)")[0].rsplit(" ", 1)[1]) for l in lines]
    assert all(s in (2, 4, 8) for s in sliced), lines
