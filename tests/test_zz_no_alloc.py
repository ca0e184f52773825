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
