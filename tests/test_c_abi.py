"""include/hodu_b200.h compiled as C11 and the ABI called from a C program (no Python between the
caller and the library): what the reference's Rust crate would do through its FFI declarations."""
import os
import shutil
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
SRC = os.path.join(ROOT, "tests", "c_abi", "abi_smoke.c")
CUDA = os.environ.get("CUDA_HOME", "/usr/local/cuda")


@pytest.fixture(scope="module")
def abi_smoke(built_lib, tmp_path_factory):
    gcc = shutil.which("gcc")
    if gcc is None or not os.path.exists(os.path.join(CUDA, "include", "cuda_runtime_api.h")):
        pytest.skip("gcc or the CUDA headers are not installed")
    exe = str(tmp_path_factory.mktemp("c_abi") / "abi_smoke")
    libdir = os.path.join(ROOT, "hodu_b200", "lib")
    cmd = [gcc, "-std=c11", "-Wall", "-Wextra", "-Werror", "-pedantic", "-O1", SRC, "-o", exe,
           "-I", os.path.join(ROOT, "include"), "-I", os.path.join(CUDA, "include"),
           "-L", libdir, "-lhodu_b200", "-L", os.path.join(CUDA, "lib64"), "-lcudart",
           f"-Wl,-rpath,{libdir}", f"-Wl,-rpath,{os.path.join(CUDA, 'lib64')}"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    assert r.returncode == 0, r.stderr
    return exe


def test_header_is_valid_c11_and_host_side_calls_work(abi_smoke):
    r = subprocess.run([abi_smoke, "host"], capture_output=True, text=True, timeout=120)
    assert r.returncode == 0 and "host checks ok" in r.stdout, r.stdout + r.stderr


@pytest.mark.gpu
def test_c_program_runs_both_kernel_families_on_the_gpu(abi_smoke):
    r = subprocess.run([abi_smoke, "gpu"], capture_output=True, text=True, timeout=600)
    assert r.returncode == 0 and "gpu checks ok" in r.stdout, r.stdout + r.stderr
