"""Generates tests/golden/*.npz by running the REFERENCE's own C kernels (compiled from its
sources into oracle/_ref by oracle/build.py) on small seeded inputs.  Needs the reference
tree; the committed .npz files are what the tests read.

    python tests/golden/make_golden.py

Each case stores the raw operand storage, the metadata vector, the name of the reference
entry point that produced the output, and that output.
"""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
from hodu_b200.layout import Layout  # noqa: E402
from hodu_b200.op_metadatas import cast_metadata, dot_metadata, matmul_metadata  # noqa: E402
from oracle import oracle as O  # noqa: E402

HERE = os.path.dirname(os.path.abspath(__file__))


def main():
    ref = O.ref()
    if ref is None:
        raise SystemExit("oracle/_ref is missing and the reference tree is not mounted")
    rng = np.random.Generator(np.random.Philox(key=1234))
    cases = {}

    def add(name, fn, lhs, rhs, md, out_dtype):
        out = np.zeros(int(md[0]) if fn.startswith("hodu_cpu_matmul") else int(md[0]) * int(md[2]), dtype=out_dtype)
        ref.call(fn, lhs, rhs, out, md)
        cases[name + "__lhs"] = lhs
        cases[name + "__rhs"] = rhs
        cases[name + "__md"] = np.array(md, dtype=np.int64)
        cases[name + "__out"] = out
        cases[name + "__fn"] = np.array(fn)

    # f32, through cblas_sgemm (hodu_cpu_matmul_f32 / hodu_cpu_dot_f32) and the fallbacks
    a = rng.standard_normal((37, 53), dtype=np.float32)
    b = rng.standard_normal((53, 29), dtype=np.float32)
    la, lb = Layout.from_shape(a.shape), Layout.from_shape(b.shape)
    add("dot_f32_blas", "hodu_cpu_dot_f32", a, b, dot_metadata(la, lb), np.float32)
    add("dot_f32_fallback", "hodu_cpu_dot_f32_fallback", a, b, dot_metadata(la, lb), np.float32)
    # transposed rhs view (Linear: weight [N,K] seen as [K,N] with strides (1,K))
    w = rng.standard_normal((29, 53), dtype=np.float32)
    lw = Layout.from_shape(w.shape).transpose(0, 1)
    add("dot_f32_blas_rhs_t", "hodu_cpu_dot_f32", a, w, dot_metadata(la, lw), np.float32)
    add("dot_f32_fallback_rhs_t", "hodu_cpu_dot_f32_fallback", a, w, dot_metadata(la, lw), np.float32)
    # batched with a broadcast rhs and an offset lhs
    a3 = rng.standard_normal((1 + 3 * 11 * 17,), dtype=np.float32)
    la3 = Layout((3, 11, 17), (11 * 17, 17, 1), 1)
    b2 = rng.standard_normal((17, 13), dtype=np.float32)
    lb2 = Layout.from_shape(b2.shape)
    out_l = Layout.from_shape((3, 11, 13))
    add("matmul_f32_fallback_bcast", "hodu_cpu_matmul_f32_fallback", a3, b2, matmul_metadata(la3, lb2, out_l), np.float32)
    # both 3-D (what Tensor::matmul passes after broadcasting both operands)
    lb3 = lb2.broadcast_to((3, 17, 13))
    add("matmul_f32_blas_bcast_view", "hodu_cpu_matmul_f32", a3, b2, matmul_metadata(la3, lb3, out_l), np.float32)
    # 2 batch dims, lhs broadcast over the outer one
    a4 = rng.standard_normal((1, 4, 6, 8), dtype=np.float32)
    b4 = rng.standard_normal((2, 4, 8, 5), dtype=np.float32)
    la4 = Layout.from_shape(a4.shape).broadcast_to((2, 4, 6, 8))
    lb4 = Layout.from_shape(b4.shape)
    add("matmul_f32_fallback_2batch", "hodu_cpu_matmul_f32_fallback", a4, b4,
        matmul_metadata(la4, lb4, Layout.from_shape((2, 4, 6, 5))), np.float32)

    # integers: the widened-integer matmul (cast_i8_to_i32 then dot_i32 / matmul_i32) and the wrapped i8 one
    ai = rng.integers(-127, 128, size=(19, 300), dtype=np.int8)
    bi = rng.integers(-127, 128, size=(300, 23), dtype=np.int8)
    lai, lbi = Layout.from_shape(ai.shape), Layout.from_shape(bi.shape)
    ai32 = np.zeros(ai.size, dtype=np.int32)
    bi32 = np.zeros(bi.size, dtype=np.int32)
    ref.cast("hodu_cpu_cast_i8_to_i32", ai, ai32, cast_metadata(lai))
    ref.cast("hodu_cpu_cast_i8_to_i32", bi, bi32, cast_metadata(lbi))
    cases["cast_i8_to_i32__in"] = ai
    cases["cast_i8_to_i32__out"] = ai32
    add("dot_i32", "hodu_cpu_dot_i32", ai32, bi32, dot_metadata(lai, lbi), np.int32)
    add("dot_i8_wrapped", "hodu_cpu_dot_i8", ai, bi, dot_metadata(lai, lbi), np.int8)
    ai3 = rng.integers(-127, 128, size=(2, 5, 40), dtype=np.int8).astype(np.int32)
    bi3 = rng.integers(-127, 128, size=(2, 40, 7), dtype=np.int8).astype(np.int32)
    add("matmul_i32", "hodu_cpu_matmul_i32", ai3, bi3,
        matmul_metadata(Layout.from_shape(ai3.shape), Layout.from_shape(bi3.shape), Layout.from_shape((2, 5, 7))), np.int32)

    # widening casts of every bf16 / f16 bit pattern step 7, and e4m3 codes the reference's
    # C codec shares with OCP e4m3fn (exponent field < 15)
    for name, fn, src in (("cast_bf16_to_f32", "hodu_cpu_cast_bf16_to_f32", np.arange(0, 65536, 7, dtype=np.uint16)),
                          ("cast_f16_to_f32", "hodu_cpu_cast_f16_to_f32", np.arange(0, 65536, 7, dtype=np.uint16))):
        dst = np.zeros(src.size, dtype=np.float32)
        ref.cast(fn, src, dst, cast_metadata(Layout.from_shape(src.shape)))
        cases[name + "__in"] = src
        cases[name + "__out"] = dst
    codes = np.array([c for c in range(256) if ((c >> 3) & 0xF) != 0xF], dtype=np.uint8)
    dst = np.zeros(codes.size, dtype=np.float32)
    ref.cast("hodu_cpu_cast_f8e4m3_to_f32", codes, dst, cast_metadata(Layout.from_shape(codes.shape)))
    cases["cast_f8e4m3_to_f32__in"] = codes
    cases["cast_f8e4m3_to_f32__out"] = dst

    # silu f32 (used by the SwiGLU oracle)
    x = np.linspace(-12, 12, 97, dtype=np.float32)
    y = np.zeros_like(x)
    fn = getattr(ref.base, "hodu_cpu_silu_f32")
    fn.restype = None
    import ctypes
    md = (ctypes.c_size_t * 5)(x.size, 1, x.size, 1, 0)
    fn(x.ctypes.data_as(ctypes.c_void_p), y.ctypes.data_as(ctypes.c_void_p), md)
    cases["silu_f32__in"] = x
    cases["silu_f32__out"] = y

    np.savez_compressed(os.path.join(HERE, "reference_cpu_kernels.npz"), **cases)
    print("wrote", len(cases), "arrays")


if __name__ == "__main__":
    main()
