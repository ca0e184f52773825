"""hodu_b200_dot_f32_static: the f32 product with its scratch in a fixed array of the library
instead of allocated memory, for callers that must not allocate while they run (real-time loops,
fixed memory reservations, hosts that forbid allocation in compute callbacks).

The file name sorts last on purpose: a run that stops at the first failure has then already
run every other test.  The test needs nothing from the other tests and initialises nothing
through them: it passes alone in a fresh process (where the entry point's first call does its
own one-time set-up on the device) and after the rest of the suite."""
import ctypes

import numpy as np
import pytest
import torch

from hodu_b200 import CudaKernelError, Layout, _lib
from hodu_b200 import kernels as K
from hodu_b200.op_metadatas import dot_metadata
from oracle import oracle as O

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda:0")


def static_dot(ta, tb, out, md):
    arr = _lib.metadata_array(md)
    _lib.check(_lib.lib().hodu_b200_dot_f32_static(0, None, ta.data_ptr(), tb.data_ptr(), out.data_ptr(), arr, len(md)))


def static_status() -> int:
    """The status word private to the entry point (synchronises the device, clears the word)."""
    w = ctypes.c_uint32(0xFFFFFFFF)
    _lib.check(_lib.lib().hodu_b200_dot_f32_static_status(0, ctypes.byref(w)))
    return w.value


def test_static_scratch_entry_point_matches_the_allocating_one():
    rng = np.random.default_rng(2024)
    # two calls in a row on the shared array: the config-1 shape first, then a smaller product with
    # padded pitches, an element offset and a transposed rhs view, so that anything the second
    # call failed to overwrite would still hold the first call's operands
    cases = [
        (rng.standard_normal((512, 1024)).astype(np.float32), Layout.from_shape((512, 1024)),
         rng.standard_normal((1024, 768)).astype(np.float32), Layout.from_shape((1024, 768))),
        (rng.standard_normal(3 + 130 * 75).astype(np.float32), Layout((130, 70), (75, 1), 3),
         rng.standard_normal((52, 70)).astype(np.float32), Layout.from_shape((52, 70)).transpose(0, 1)),
    ]
    for a, la, b, lb in cases:
        md = dot_metadata(la, lb)
        m, n = la.shape[0], lb.shape[1]
        ta, tb = torch.from_numpy(a).to(DEV), torch.from_numpy(b).to(DEV)
        got = torch.full((m * n + 64,), 123.0, dtype=torch.float32, device=DEV)
        static_dot(ta, tb, got, md)
        torch.cuda.synchronize()
        assert bool((got[m * n:] == 123.0).all().item()), "wrote past the end of the output"
        # the existing entry point, pinned to the same (tensor-core) algorithm
        want = torch.empty(m * n, dtype=torch.float32, device=DEV)
        prev = K.force_path(_lib.PATH_TENSOR)
        try:
            K.call_ops_dot(K.dot.F32, 0, ta.data_ptr(), tb.data_ptr(), want.data_ptr(), md, 0)
        finally:
            K.force_path(prev)
        assert K.last_status(0) == 0
        assert static_status() == 0   # no bounded wait of the static call gave up
        g, w = got[: m * n].cpu().numpy(), want.cpu().numpy()
        # same kernels; the allocating entry point may add the three product terms as separate
        # K slices (it has scratch for the partial sums), so only the order of the sums differs
        assert O.rel_err(g, w) <= 2e-5
        assert O.rel_err(g, O.matmul(a, b, md, O.F32, is_dot=True)) <= 1e-4  # and the f32 bar against the oracle


def test_static_scratch_entry_point_rejects_what_does_not_fit():
    limit = 32 << 20
    m = n = k = 2048                      # 12*(M+N)*K = 96 MiB of split operands
    assert 12 * (m + n) * k > limit
    t = torch.zeros(8, dtype=torch.float32, device=DEV)
    md = dot_metadata(Layout.from_shape((m, k)), Layout.from_shape((k, n)))
    with pytest.raises(CudaKernelError) as e:
        static_dot(t, t, t, md)            # rejected from the sizes alone: the buffers are never touched
    assert e.value.kind == "invalid input" and "fixed array holds" in str(e.value)
    with pytest.raises(CudaKernelError):
        static_dot(t, t, t, md[:-1])       # malformed metadata


def test_static_scratch_entry_point_limit_is_exact_and_k_zero_clears():
    limit = 32 << 20
    # 12*(M+N)*K with K = 1024 (rows of 3K floats are already 16-byte multiples): M + N = 2730 fits
    # by 8192 bytes, one more row does not
    k, n = 1024, 730
    m_fit = limit // (12 * k) - n
    assert 12 * (m_fit + n) * k <= limit < 12 * (m_fit + 1 + n) * k
    rng = np.random.default_rng(77)
    a = rng.standard_normal((m_fit + 1, k)).astype(np.float32)
    b = rng.standard_normal((k, n)).astype(np.float32)
    ta, tb = torch.from_numpy(a).to(DEV), torch.from_numpy(b).to(DEV)
    out = torch.empty((m_fit + 1) * n, dtype=torch.float32, device=DEV)
    static_dot(ta, tb, out, dot_metadata(Layout.from_shape((m_fit, k)), Layout.from_shape((k, n))))
    assert static_status() == 0
    want = a[:m_fit].astype(np.float64) @ b.astype(np.float64)
    assert O.rel_err(out[: m_fit * n].cpu().numpy(), want.astype(np.float32).reshape(-1)) <= 2e-5
    with pytest.raises(CudaKernelError) as e:
        static_dot(ta, tb, out, dot_metadata(Layout.from_shape((m_fit + 1, k)), Layout.from_shape((k, n))))
    assert e.value.kind == "invalid input"
    # K == 0: an empty sum, so the output is cleared (a memset: still no allocation)
    z = torch.full((6 * 5 + 8,), 3.0, dtype=torch.float32, device=DEV)
    static_dot(ta, tb, z, dot_metadata(Layout.from_shape((6, 0)), Layout.from_shape((0, 5))))
    torch.cuda.synchronize()
    assert bool((z[:30] == 0).all().item()) and bool((z[30:] == 3.0).all().item())


def test_static_scratch_entry_point_takes_no_device_memory():
    """What the entry point exists for: after its one-time set-up a call changes neither the
    amount of free device memory nor anything the library's other entry points have allocated."""
    rng = np.random.default_rng(5)
    a = rng.standard_normal((384, 512)).astype(np.float32)
    b = rng.standard_normal((512, 256)).astype(np.float32)
    md = dot_metadata(Layout.from_shape(a.shape), Layout.from_shape(b.shape))
    ta, tb = torch.from_numpy(a).to(DEV), torch.from_numpy(b).to(DEV)
    out = torch.empty(384 * 256, dtype=torch.float32, device=DEV)
    static_dot(ta, tb, out, md)             # warm call: symbol addresses, kernel attributes, module load
    torch.cuda.synchronize()
    free0, _ = torch.cuda.mem_get_info(DEV)
    launches0 = K.launch_count()
    for _ in range(3):
        static_dot(ta, tb, out, md)
    torch.cuda.synchronize()
    free1, _ = torch.cuda.mem_get_info(DEV)
    assert free1 == free0, f"free device memory changed by {free0 - free1} bytes over three calls"
    assert K.launch_count() - launches0 == 6   # split pass + product per call, nothing else
    assert static_status() == 0


def test_static_scratch_entry_point_alone_in_a_fresh_process():
    """The first thing a process does with the library: no hodu_b200_init, no other entry point
    before it, so nothing of the library's allocated per-device state exists."""
    import os
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    code = r"""
import ctypes, sys
import numpy as np, torch
sys.path.insert(0, %r)
from hodu_b200 import Layout, _lib
from hodu_b200.op_metadatas import dot_metadata
dev = torch.device("cuda:0")
rng = np.random.default_rng(9)
a = rng.standard_normal((200, 300)).astype(np.float32)
b = rng.standard_normal((300, 136)).astype(np.float32)
ta, tb = torch.from_numpy(a).to(dev), torch.from_numpy(b).to(dev)
out = torch.empty(200 * 136, dtype=torch.float32, device=dev)
md = dot_metadata(Layout.from_shape(a.shape), Layout.from_shape(b.shape))
arr = _lib.metadata_array(md)
lib = _lib.lib()
for _ in range(2):
    assert lib.hodu_b200_dot_f32_static(0, None, ta.data_ptr(), tb.data_ptr(), out.data_ptr(), arr, len(md)) == 0
w = ctypes.c_uint32(1)
assert lib.hodu_b200_dot_f32_static_status(0, ctypes.byref(w)) == 0 and w.value == 0
want = (a.astype(np.float64) @ b.astype(np.float64)).reshape(-1)
err = float(np.abs(out.cpu().numpy() - want).max() / np.abs(want).max())
assert err <= 2e-5, err
print("ok", err)
""" % root
    r = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, timeout=600)
    assert r.returncode == 0 and "ok" in r.stdout, r.stdout + r.stderr
