"""The metadata parsers under AddressSanitizer + UndefinedBehaviorSanitizer, fed hostile metadata
(short arrays, huge ranks, overflowing extents).  Host code only: nothing is launched and no GPU
is needed; nvcc compiles the library's sources with the sanitizers switched on for the host side
and links them with tests/sanitize/parsers_fuzz.cu into one program."""
import concurrent.futures as cf
import os
import shutil
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
CSRC = os.path.join(ROOT, "hodu_b200", "csrc")
# one -Xcompiler per flag: nvcc splits a single argument at its commas
SAN = [x for f in ("-fsanitize=address", "-fsanitize=undefined", "-fno-sanitize-recover=undefined",
                      "-fno-omit-frame-pointer") for x in ("-Xcompiler", f)]


def test_parsers_survive_hostile_metadata_under_sanitizers(tmp_path):
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(nvcc):
        pytest.skip("nvcc not installed")
    from hodu_b200.build import SOURCES
    srcs = [os.path.join(CSRC, s) for s in SOURCES] + [os.path.join(ROOT, "tests", "sanitize", "parsers_fuzz.cu")]
    common = [nvcc, "-gencode", "arch=compute_100a,code=sm_100a", "-O1", "-g", "-std=c++17", "--expt-relaxed-constexpr", *SAN]

    def compile_one(src):
        obj = str(tmp_path / (os.path.basename(src) + ".o"))
        r = subprocess.run(common + ["-c", src, "-o", obj], capture_output=True, text=True)
        assert r.returncode == 0, r.stderr[-2000:]
        return obj

    with cf.ThreadPoolExecutor(max_workers=8) as ex:
        objs = list(ex.map(compile_one, srcs))
    exe = str(tmp_path / "parsers_fuzz")
    r = subprocess.run([nvcc, "-gencode", "arch=compute_100a,code=sm_100a", "-o", exe, *objs, *SAN, "-lpthread"], capture_output=True, text=True)
    assert r.returncode == 0, r.stderr[-2000:]
    env = dict(os.environ, ASAN_OPTIONS="protect_shadow_gap=0:detect_leaks=0:abort_on_error=0",
               UBSAN_OPTIONS="print_stacktrace=1:halt_on_error=1", CUDA_VISIBLE_DEVICES="")
    r = subprocess.run([exe, "60000"], capture_output=True, text=True, timeout=900, env=env)
    assert r.returncode == 0 and "no sanitizer finding" in r.stdout, (r.stdout[-1500:] + r.stderr[-3000:])
