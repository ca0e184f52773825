"""TEST INFRASTRUCTURE.  Builds the CPU checkers:

  oracle/_build/liboracle.so        the C restatement in hodu_oracle.c (gcc)
  oracle/_ref/libhodu_ref.so        the REFERENCE's own C kernels for this path, compiled
                                    from the sources where they lie (never copied here):
                                    ops_matrix.c, ops_cast.c, ops_unary.c, ops_binary.c, ops_einsum.c, ops_conv.c
  oracle/_ref/libhodu_ref_blas.so   the reference's OpenBLAS variant ops_matrix_openblas.c
                                    (hodu_cpu_matmul_f32 / hodu_cpu_dot_f32 = cblas_sgemm),
                                    linked against an OpenBLAS found in site-packages

The reference libraries are built only where the reference tree is present; on a
machine without it the prebuilt files are used as they are.

Flags follow the reference's build (crates/hodu_cpu_kernels/build.rs:37-65:
-std=c11 -O3 -DENABLE_THREADS) except -march=native, replaced by -march=x86-64-v3 so
that a library built on one host runs on another.

    python oracle/build.py [--ref-root /path/to/reference]
"""
from __future__ import annotations

import argparse
import glob
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
BUILD = os.path.join(HERE, "_build")
REF = os.path.join(HERE, "_ref")


def default_ref_root() -> str:
    """Where the reference checkout is looked for: $HODU_REFERENCE_ROOT, else a directory named
    `reference` beside this repository.  Neither present: the prebuilt files are used as they are."""
    env = os.environ.get("HODU_REFERENCE_ROOT")
    if env:
        return env
    return os.path.normpath(os.path.join(HERE, "..", "..", "reference"))


def _run(cmd):
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError("failed: " + " ".join(cmd) + "\n" + r.stdout + r.stderr)


def find_openblas():
    """(path, symbol_prefix) of an LP64 OpenBLAS shipped inside a wheel.  scipy's copy
    (0.3.31, the reference asks for 0.3.30+) prefixes its symbols with `scipy_`."""
    import site
    for root in site.getsitepackages():
        hits = sorted(glob.glob(os.path.join(root, "scipy.libs", "libscipy_openblas-*.so")))
        if hits:
            return hits[0], "scipy_"
    for p in ("/usr/lib/x86_64-linux-gnu/libopenblas.so.0", "/usr/lib64/libopenblas.so.0"):
        if os.path.exists(p):
            return p, ""
    return None, ""


def build_oracle() -> str:
    os.makedirs(BUILD, exist_ok=True)
    out = os.path.join(BUILD, "liboracle.so")
    src = os.path.join(HERE, "hodu_oracle.c")
    if not os.path.exists(out) or os.path.getmtime(out) < os.path.getmtime(src):
        _run(["gcc", "-std=c11", "-O2", "-fPIC", "-shared", "-ffp-contract=off", src, "-o", out, "-lm"])
    return out


def _exports(path: str, symbol: str) -> bool:
    import ctypes
    try:
        return hasattr(ctypes.CDLL(path), symbol)
    except OSError:
        return False


def build_ref(ref_root: str = ""):
    ref_root = ref_root or default_ref_root()
    kdir = os.path.join(ref_root, "crates", "hodu_cpu_kernels", "kernels")
    if not os.path.isdir(kdir):
        return None
    os.makedirs(REF, exist_ok=True)
    flags = ["-std=c11", "-O3", "-march=x86-64-v3", "-DENABLE_THREADS", "-fPIC", "-shared", "-I", kdir]
    out = os.path.join(REF, "libhodu_ref.so")
    srcs = [os.path.join(kdir, f) for f in ("ops_matrix.c", "ops_cast.c", "ops_unary.c", "ops_binary.c",
                                            "ops_einsum.c", "ops_conv.c")]
    if os.path.exists(out) and not _exports(out, "hodu_cpu_conv2d_f32_fallback"):
        os.remove(out)  # built from an earlier, shorter source list
    if not os.path.exists(out):
        _run(["gcc", *flags, *srcs, "-o", out, "-lpthread", "-lm"])
    blas, prefix = find_openblas()
    out_blas = os.path.join(REF, "libhodu_ref_blas.so")
    if blas and not os.path.exists(out_blas):
        # cblas.h is the small header next to this script; the fallbacks the file
        # forward-declares come from ops_matrix.c.  A prefixed OpenBLAS is reached by
        # renaming the four BLAS symbols on the command line; the source is untouched.
        renames = [f"-D{n}={prefix}{n}" for n in ("cblas_sgemm", "cblas_dgemm", "openblas_set_num_threads",
                                                  "openblas_get_num_threads")] if prefix else []
        _run(["gcc", *flags, *renames, "-I", HERE, os.path.join(kdir, "ops_matrix_openblas.c"),
              os.path.join(kdir, "ops_matrix.c"), "-o", out_blas, blas,
              "-Wl,--disable-new-dtags,-rpath," + os.path.dirname(blas), "-lpthread", "-lm"])
        with open(os.path.join(REF, "blas.txt"), "w") as f:
            f.write(f"{blas}\n{prefix}\n")
    return out


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--ref-root", default="")
    a = ap.parse_args()
    print(build_oracle())
    print(build_ref(a.ref_root) or "reference tree not present: oracle/_ref left as it is")
