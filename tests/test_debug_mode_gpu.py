"""HODU_B200_DEBUG=1: host-side checks of every tensor-core launch (tile arithmetic, stage sizes,
TMEM columns, TMA coordinate ranges) before it runs, a synchronisation and a read of the device
status word after it.  Run in a child process because the switch is read once per process."""
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

CODE = r"""
import sys
sys.path.insert(0, %r)
sys.path.insert(0, %r)
import numpy as np
from gpu_util import gpu_matmul, check_close
from hodu_b200 import Layout, _lib
from hodu_b200.op_metadatas import dot_metadata, matmul_metadata
from oracle import oracle as O
rng = np.random.default_rng(3)
n = 0
for form in (_lib.PATH_TENSOR_1CTA, _lib.PATH_TENSOR_2CTA, _lib.PATH_TENSOR_2CTA_512, _lib.PATH_TENSOR):
    for (m, k, n_) in ((300, 264, 520), (128, 64, 64), (1024, 2048, 768)):
        a = O.narrow(rng.standard_normal((m, k)).astype(np.float32), O.BF16)
        b = O.narrow(rng.standard_normal((k, n_)).astype(np.float32), O.BF16)
        md = dot_metadata(Layout.from_shape((m, k)), Layout.from_shape((k, n_)))
        got, _ = gpu_matmul(a, b, md, O.BF16, is_dot=True, path=form)
        check_close(got, O.matmul(a, b, md, O.BF16, is_dot=True), O.BF16, 1e-2)
        n += 1
a = rng.standard_normal((512, 1024)).astype(np.float32)
b = rng.standard_normal((1024, 768)).astype(np.float32)
md = dot_metadata(Layout.from_shape(a.shape), Layout.from_shape(b.shape))
got, _ = gpu_matmul(a, b, md, O.F32, is_dot=True, path=_lib.PATH_TENSOR)
assert O.rel_err(got, O.matmul(a, b, md, O.F32, is_dot=True)) <= 1e-4
print("checked", n + 1)
"""


def test_debug_mode_checks_every_launch_and_results_stay_right():
    env = dict(os.environ, HODU_B200_DEBUG="1")
    r = subprocess.run([sys.executable, "-c", CODE % (ROOT, os.path.join(ROOT, "tests"))], capture_output=True,
                       text=True, timeout=900, env=env)
    assert r.returncode == 0 and "checked 13" in r.stdout, r.stdout[-800:] + r.stderr[-2000:]
    lines = [l for l in r.stderr.splitlines() if l.startswith("[hodu_b200] gemm_")]
    assert len(lines) >= 13, r.stderr[-1500:]       # one line per tensor-core launch
    assert any("pair" in l for l in lines) and any("1-CTA" in l for l in lines)
    assert any("gemm_f32_fused" in l for l in lines)   # the f32 product took the one-kernel form
