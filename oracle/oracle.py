"""TEST INFRASTRUCTURE -- not part of the product.  Only tests/, the smoke check and the
cpu_baseline / reference legs of bench.py import this module.

Python face of the CPU oracle:
  * `C`   : ctypes access to oracle/_build/liboracle.so (hodu_oracle.c, the restatement)
  * `Ref` : ctypes access to oracle/_ref/*.so, the reference's own C kernels compiled from
            its sources (None when neither the prebuilt files nor the reference tree exist)
  * numpy forms of the same definitions for sizes where per-element C loops are too slow:
    widening is exact, the f32 product is numpy's sgemm (the reference's `openblas`
    build calls cblas_sgemm, crates/hodu_cpu_kernels/kernels/ops_matrix_openblas.c:91-141),
    narrowing is round-to-nearest-even.

Arrays hold RAW STORAGE: bf16/f16 as uint16, f8e4m3 as uint8, i8 as int8, f32 as float32.
"""
from __future__ import annotations

import ctypes as C_
import os
from typing import Optional, Sequence

import numpy as np

from . import build as _build

HERE = os.path.dirname(os.path.abspath(__file__))

# DType discriminants (crates/hodu_core/src/types/dtype.rs:6-30)
F8E4M3, BF16, F16, F32, I8, I32 = 1, 3, 4, 5, 11, 13
NP_STORAGE = {F8E4M3: np.uint8, BF16: np.uint16, F16: np.uint16, F32: np.float32, I8: np.int8, I32: np.int32}

_c = None
_ref = None
_ref_tried = False


def _ptr(a: np.ndarray):
    return a.ctypes.data_as(C_.c_void_p)


def _md(md: Sequence[int]):
    return (C_.c_size_t * len(md))(*[int(x) for x in md])


def clib() -> C_.CDLL:
    global _c
    if _c is None:
        path = os.path.join(HERE, "_build", "liboracle.so")
        if not os.path.exists(path) or os.path.getmtime(path) < os.path.getmtime(os.path.join(HERE, "hodu_oracle.c")):
            path = _build.build_oracle()
        _c = C_.CDLL(path)
        for n in ("oracle_bf16_to_f32", "oracle_f16_to_f32", "oracle_e4m3_to_f32"):
            getattr(_c, n).restype = C_.c_float
        _c.oracle_f32_to_bf16.restype = C_.c_uint16
        _c.oracle_f32_to_f16.restype = C_.c_uint16
        _c.oracle_f32_to_e4m3.restype = C_.c_uint8
        for n in ("oracle_f32_to_bf16", "oracle_f32_to_f16", "oracle_f32_to_e4m3"):
            getattr(_c, n).argtypes = [C_.c_float]
    return _c


class _Ref:
    """The reference's compiled C kernels (see oracle/build.py)."""

    def __init__(self, base: C_.CDLL, blas: Optional[C_.CDLL]):
        self.base, self.blas = base, blas

    def call(self, name: str, lhs: np.ndarray, rhs: np.ndarray, out: np.ndarray, md: Sequence[int]) -> None:
        lib = self.blas if (self.blas is not None and hasattr(self.blas, name)) else self.base
        fn = getattr(lib, name)
        fn.restype = None
        fn(_ptr(lhs), _ptr(rhs), _ptr(out), _md(md))

    def cast(self, name: str, src: np.ndarray, dst: np.ndarray, md: Sequence[int]) -> None:
        fn = getattr(self.base, name)
        fn.restype = None
        fn(_ptr(src), _ptr(dst), _md(md))

    def einsum(self, name: str, inputs: Sequence[np.ndarray], out: np.ndarray, md: Sequence[int]) -> None:
        """hodu_cpu_einsum_{dtype}(const void** inputs, void* output, const size_t* metadata)."""
        fn = getattr(self.base, name)
        fn.restype = None
        ptrs = (C_.c_void_p * len(inputs))(*[a.ctypes.data for a in inputs])
        fn(ptrs, _ptr(out), _md(md))

    def set_blas_threads(self, n: int) -> int:
        """openblas_set_num_threads(n) on the OpenBLAS behind hodu_cpu_{matmul,dot}_f32 (launchers
        such as torchrun export OMP_NUM_THREADS=1, which OpenBLAS would otherwise obey).
        Returns the thread count in effect afterwards (0 if there is no BLAS build)."""
        note = os.path.join(HERE, "_ref", "blas.txt")
        if self.blas is None or not os.path.exists(note):
            return 0
        path, prefix = [l.strip() for l in open(note).read().split("\n")[:2]]
        try:
            ob = C_.CDLL(path)
            getattr(ob, prefix + "openblas_set_num_threads")(C_.c_int(int(n)))
            return int(getattr(ob, prefix + "openblas_get_num_threads")())
        except (OSError, AttributeError):
            return 0

    def blas_info(self) -> dict:
        """Thread count and build string of the OpenBLAS behind hodu_cpu_{matmul,dot}_f32."""
        info = {"threads": 0, "config": "none", "path": ""}
        note = os.path.join(HERE, "_ref", "blas.txt")
        if self.blas is None or not os.path.exists(note):
            return info
        path, prefix = [l.strip() for l in open(note).read().split("\n")[:2]]
        try:
            ob = C_.CDLL(path)
            info["path"] = path
            info["threads"] = int(getattr(ob, prefix + "openblas_get_num_threads")())
            cfg = getattr(ob, prefix + "openblas_get_config")
            cfg.restype = C_.c_char_p
            info["config"] = cfg().decode()
        except (OSError, AttributeError):
            pass
        return info


def ref() -> Optional[_Ref]:
    """oracle/_ref if present (built here when the reference tree is mounted)."""
    global _ref, _ref_tried
    if not _ref_tried:
        _ref_tried = True
        base = os.path.join(HERE, "_ref", "libhodu_ref.so")
        if not os.path.exists(base):
            try:
                _build.build_ref()
            except Exception:
                pass
        if os.path.exists(base):
            blas_path = os.path.join(HERE, "_ref", "libhodu_ref_blas.so")
            blas = None
            if os.path.exists(blas_path):
                try:
                    blas = C_.CDLL(blas_path)
                except OSError:
                    blas = None
            _ref = _Ref(C_.CDLL(base), blas)
    return _ref


# ------------------------------------------------------------------ codecs (numpy forms)

def bf16_to_f32(bits: np.ndarray) -> np.ndarray:
    return (bits.astype(np.uint32) << 16).view(np.float32)


def f32_to_bf16(x: np.ndarray) -> np.ndarray:
    """Round to nearest even; NaN stays NaN (quiet bit forced)."""
    b = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32)
    nan = (b & 0x7FFFFFFF) > 0x7F800000
    r = ((b + (0x7FFF + ((b >> 16) & 1))) >> 16).astype(np.uint16)
    return np.where(nan, ((b >> 16) | 0x40).astype(np.uint16), r)


def f16_to_f32(bits: np.ndarray) -> np.ndarray:
    return bits.view(np.float16).astype(np.float32)


def f32_to_f16(x: np.ndarray) -> np.ndarray:
    with np.errstate(over="ignore"):
        return np.ascontiguousarray(x, dtype=np.float32).astype(np.float16).view(np.uint16)


_E4M3_LUT = None


def e4m3_lut() -> np.ndarray:
    global _E4M3_LUT
    if _E4M3_LUT is None:
        c = clib()
        _E4M3_LUT = np.array([c.oracle_e4m3_to_f32(C_.c_uint8(i)) for i in range(256)], dtype=np.float32)
    return _E4M3_LUT


def e4m3_to_f32(bits: np.ndarray) -> np.ndarray:
    return e4m3_lut()[bits]


def f32_to_e4m3(x: np.ndarray) -> np.ndarray:
    """Round to nearest even, saturate finite values to +-448, NaN -> 0x7F | sign."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    sign = ((x.view(np.uint32) >> 24) & 0x80).astype(np.uint8)
    a = np.abs(x)
    nan = np.isnan(x)
    a = np.minimum(np.where(nan, 0.0, a), np.float32(512.0)).astype(np.float32)  # +-inf saturate too
    with np.errstate(divide="ignore"):
        exp = np.floor(np.log2(np.maximum(a, np.float32(2.0 ** -20)))).astype(np.int32)
    # log2 can be off by one ulp at powers of two: fix with exact comparisons
    exp = np.where(np.ldexp(np.float32(1), exp + 1) <= a, exp + 1, exp)
    exp = np.where(np.ldexp(np.float32(1), exp) > a, exp - 1, exp)
    exp = np.maximum(exp, -6)
    scaled = np.ldexp(a, 3 - exp).astype(np.float64)      # units of the last mantissa bit; exact
    q = np.rint(scaled).astype(np.int64)                  # rint = round half to even
    carry = q == 16
    q = np.where(carry, 8, q)
    exp = np.where(carry, exp + 1, exp)
    sub = (exp == -6) & (q < 8)
    out = np.where(sub, q, ((exp + 7) << 3) | (q - 8))
    out = np.where(a >= 448.0, 0x7E, out)
    out = np.clip(out, 0, 0x7E).astype(np.uint8)
    out = np.where(nan, 0x7F, out).astype(np.uint8)
    return (out | sign).astype(np.uint8)


def widen(bits: np.ndarray, dtype: int) -> np.ndarray:
    """Storage -> f32 (floating dtypes) or int32 (i8), exactly."""
    if dtype == BF16:
        return bf16_to_f32(bits)
    if dtype == F16:
        return f16_to_f32(bits)
    if dtype == F8E4M3:
        return e4m3_to_f32(bits)
    if dtype == F32:
        return np.asarray(bits, dtype=np.float32)
    if dtype in (I8, I32):
        return bits.astype(np.int32)
    raise ValueError(dtype)


def narrow(x: np.ndarray, dtype: int) -> np.ndarray:
    """f32 -> storage with round to nearest even; int32 -> i32 / wrapped i8."""
    if dtype == BF16:
        return f32_to_bf16(x)
    if dtype == F16:
        return f32_to_f16(x)
    if dtype == F8E4M3:
        return f32_to_e4m3(x)
    if dtype == F32:
        return np.asarray(x, dtype=np.float32)
    if dtype == I32:
        return np.asarray(x).astype(np.int32)
    if dtype == I8:
        return (np.asarray(x).astype(np.int64) & 0xFF).astype(np.uint8).view(np.int8)
    raise ValueError(dtype)


# ------------------------------------------------------------------ views from wire formats

def _strided(flat: np.ndarray, shape, strides, offset) -> np.ndarray:
    item = flat.itemsize
    return np.lib.stride_tricks.as_strided(flat[offset:], shape=tuple(shape), strides=tuple(s * item for s in strides),
                                           writeable=False)


def operands_from_matmul_md(lhs: np.ndarray, rhs: np.ndarray, md: Sequence[int]):
    """Strided numpy views [batch.., M, K] and [batch.., K, N] described by matmul metadata,
    broadcast to the output batch shape exactly as the reference indexes them
    (crates/hodu_cpu_kernels/kernels/ops_matrix.c:144-193)."""
    md = [int(x) for x in md]
    ln, rn, bn = md[1], md[2], md[3]
    p = 4
    lshape = md[p:p + ln]; p += ln
    rshape = md[p:p + rn]; p += rn
    bshape = md[p:p + bn]; p += bn
    lstr = md[p:p + ln]; p += ln
    rstr = md[p:p + rn]; p += rn
    loff, roff = md[p], md[p + 1]

    def view(flat, shape, strides, off, nd):
        strides = [0 if s == 1 else st for s, st in zip(shape[:nd - 2], strides[:nd - 2])] + list(strides[nd - 2:])
        pad = bn - (nd - 2)
        full_shape = list(bshape) + list(shape[nd - 2:])
        full_str = [0] * pad + strides
        return _strided(flat, full_shape, full_str, off)

    return view(lhs.reshape(-1), lshape, lstr, loff, ln), view(rhs.reshape(-1), rshape, rstr, roff, rn)


def operands_from_dot_md(lhs: np.ndarray, rhs: np.ndarray, md: Sequence[int]):
    m, k, n, lsm, lsk, rsk, rsn, lo, ro = [int(x) for x in md]
    return _strided(lhs.reshape(-1), (m, k), (lsm, lsk), lo), _strided(rhs.reshape(-1), (k, n), (rsk, rsn), ro)


# ------------------------------------------------------------------ the oracle product

def matmul(lhs: np.ndarray, rhs: np.ndarray, md: Sequence[int], in_dtype: int, out_dtype: Optional[int] = None,
           scale: float = 1.0, is_dot: bool = False) -> np.ndarray:
    """Oracle result (raw storage of `out_dtype`, flat) for one call of the matmul / dot
    wire format.  Floating inputs: widen -> f32 sgemm -> * scale -> one RNE narrowing.
    i8 / i32 inputs: exact integer product (computed in float64, exact while |sum| < 2^53),
    returned as i32 or wrapped to i8."""
    out_dtype = in_dtype if out_dtype is None else out_dtype
    a, b = (operands_from_dot_md if is_dot else operands_from_matmul_md)(lhs, rhs, md)
    if in_dtype in (I8, I32):
        c = np.matmul(a.astype(np.float64), b.astype(np.float64))
        ci = np.rint(c).astype(np.int64)
        if out_dtype == I32:
            return (ci & 0xFFFFFFFF).astype(np.uint32).view(np.int32).reshape(-1)
        return narrow(ci, I8).reshape(-1)
    af, bf = widen(np.ascontiguousarray(a), in_dtype), widen(np.ascontiguousarray(b), in_dtype)
    c = np.matmul(af, bf)
    if scale != 1.0:
        c = c * np.float32(scale)
    return narrow(c.astype(np.float32), out_dtype).reshape(-1)


def matmul_c(lhs: np.ndarray, rhs: np.ndarray, md: Sequence[int], in_dtype: int, out_dtype: Optional[int] = None,
             scale: float = 1.0, is_dot: bool = False) -> np.ndarray:
    """Same definition through the element-by-element C restatement (small cases)."""
    out_dtype = in_dtype if out_dtype is None else out_dtype
    c = clib()
    md_c = _md(md)
    n_out = int(md[0]) * int(md[2]) if is_dot else int(md[0])
    if in_dtype in (I8, I32):
        a32 = widen(lhs.reshape(-1), I8 if in_dtype == I8 else I32).astype(np.int32)
        b32 = widen(rhs.reshape(-1), I8 if in_dtype == I8 else I32).astype(np.int32)
        out = np.zeros(n_out, dtype=np.int32)
        (c.oracle_dot_i32 if is_dot else c.oracle_matmul_i32)(_ptr(a32), _ptr(b32), _ptr(out), md_c)
        return out if out_dtype == I32 else narrow(out, I8)
    af = np.ascontiguousarray(widen(lhs.reshape(-1), in_dtype))
    bf = np.ascontiguousarray(widen(rhs.reshape(-1), in_dtype))
    out = np.zeros(n_out, dtype=np.float32)
    (c.oracle_dot_f32 if is_dot else c.oracle_matmul_f32)(_ptr(af), _ptr(bf), _ptr(out), md_c)
    if scale != 1.0:
        out = out * np.float32(scale)
    return narrow(out, out_dtype)


def silu(x: np.ndarray) -> np.ndarray:
    """x / (1 + expf(-x)) in f32 (crates/hodu_cpu_kernels/kernels/math_utils.h:184)."""
    x = np.asarray(x, dtype=np.float32)
    with np.errstate(over="ignore"):
        return (x / (np.float32(1.0) + np.exp(-x, dtype=np.float32))).astype(np.float32)


def swiglu_hidden(x: np.ndarray, wg: np.ndarray, wu: np.ndarray, dtype: int, round_each_op: bool = True) -> np.ndarray:
    """silu(x.wg) * (x.wu) for 2-D widened-f32 views x[M,K], wg[K,N], wu[K,N] holding values
    of storage dtype `dtype`.  round_each_op: every intermediate tensor of the reference's
    op-by-op composition (gate, up, silu, product) is rounded to `dtype`; otherwise only
    the product is.  Returns raw storage [M,N]."""
    g = np.matmul(x, wg).astype(np.float32)
    u = np.matmul(x, wu).astype(np.float32)
    if round_each_op:
        g = widen(narrow(g, dtype), dtype)
        u = widen(narrow(u, dtype), dtype)
        s = widen(narrow(silu(g), dtype), dtype)
        return narrow(s * u, dtype)
    return narrow(silu(g) * u, dtype)


def linear(x: np.ndarray, w: np.ndarray, bias: np.ndarray, dtype: int, round_each_op: bool = True) -> np.ndarray:
    """x[..., K] . w[K, N] + bias[N] for widened-f32 arrays holding values of storage dtype
    `dtype` (`Linear::forward`, crates/hodu_nn/src/modules/linear.rs:38-47: `matmul`, then `add`).
    round_each_op: the product is rounded to `dtype` before the addition, as the reference's two
    ops do; otherwise only the sum is rounded.  Returns raw storage, flat."""
    c = np.matmul(x, w).astype(np.float32)
    if round_each_op:
        c = widen(narrow(c, dtype), dtype)
    return narrow((c + bias.astype(np.float32)).astype(np.float32), dtype).reshape(-1)


def parse_einsum_md(md: Sequence[int]):
    """Splits the reference's einsum wire format
    (crates/hodu_cpu_kernels/kernels/ops_einsum.c:27-70 reads it the same way)."""
    md = [int(v) for v in md]
    n_out, n_in, n_idx, n_con, out_ndim = md[:5]
    pos = 5
    out_shape = md[pos:pos + out_ndim]; pos += out_ndim
    inputs = []
    for _ in range(n_in):
        nd = md[pos]; pos += 1
        shape = md[pos:pos + nd]; pos += nd
        strides = md[pos:pos + nd]; pos += nd
        off = md[pos]; pos += 1
        ids = md[pos:pos + nd]; pos += nd
        inputs.append((shape, strides, off, ids))
    con = md[pos:pos + n_con]; pos += n_con
    sizes = md[pos:pos + n_idx]; pos += n_idx
    out_ids = md[pos:pos + out_ndim]; pos += out_ndim
    assert pos == len(md), "einsum metadata length"
    return n_out, out_shape, inputs, con, sizes, out_ids


def einsum(inputs: Sequence[np.ndarray], md: Sequence[int], dtype: int) -> np.ndarray:
    """Oracle of the einsum op for storage dtype `dtype`: every output element is the sum over
    all contraction indices of the product of the operands' elements, accumulated in f32 and
    converted once (crates/hodu_cpu_kernels/kernels/ops_einsum.c:134-170; the CUDA kernel
    crates/hodu_cuda_kernels/kernels/ops_einsum.cu:126-175 does the same).  Integers: exact,
    wrapped to the storage width.  Returns raw storage, flat."""
    n_out, out_shape, ins, _con, _sizes, out_ids = parse_einsum_md(md)
    views, subs = [], []
    for flat, (shape, strides, off, ids) in zip(inputs, ins):
        v = _strided(flat.reshape(-1), shape, strides, off)
        if dtype in (I8, I32):
            v = widen(np.ascontiguousarray(v), dtype).astype(np.float64)
        else:
            v = widen(np.ascontiguousarray(v), dtype)
        views.append(v)
        subs.append(list(ids))
    args = []
    for v, sub in zip(views, subs):
        args += [v, sub]
    c = np.einsum(*args, list(out_ids))
    if dtype in (I8, I32):
        ci = np.rint(c).astype(np.int64)
        if dtype == I32:
            return (ci & 0xFFFFFFFF).astype(np.uint32).view(np.int32).reshape(-1)
        return narrow(ci, I8).reshape(-1)
    return narrow(np.asarray(c, dtype=np.float32), dtype).reshape(-1)


def conv2d(inp: np.ndarray, weight: np.ndarray, md: Sequence[int], dtype: int) -> np.ndarray:
    """Oracle of conv2d for storage dtype `dtype`: NCHW input and [Cout,Cin,KH,KW] weight,
    contiguous from their offsets; every output element is the f32 sum over (ic, kh, kw) of
    input x weight with zero padding, converted once
    (crates/hodu_cuda_kernels/kernels/ops_conv.cu:65-92; the CPU f32 form
    crates/hodu_cpu_kernels/kernels/ops_conv.c:172-232 is the same sum).  Computed as
    unfold + f32 matrix product per image.  Returns raw storage, flat [B, Cout, OH, OW]."""
    (_n, B, cin, cout, H, W, KH, KW, OH, OW, sh, sw, ph, pw, dh, dw, ioff, woff) = [int(v) for v in md]
    x = widen(inp.reshape(-1)[ioff:ioff + B * cin * H * W], dtype).reshape(B, cin, H, W)
    w = widen(weight.reshape(-1)[woff:woff + cout * cin * KH * KW], dtype).reshape(cout, cin * KH * KW)
    xp = np.zeros((B, cin, H + 2 * ph, W + 2 * pw), dtype=np.float32)
    xp[:, :, ph:ph + H, pw:pw + W] = x
    col = np.empty((B, cin, KH, KW, OH, OW), dtype=np.float32)
    for kh in range(KH):
        for kw in range(KW):
            col[:, :, kh, kw] = xp[:, :, kh * dh:kh * dh + (OH - 1) * sh + 1:sh, kw * dw:kw * dw + (OW - 1) * sw + 1:sw]
    col = col.reshape(B, cin * KH * KW, OH * OW)
    out = np.matmul(w[None], col).astype(np.float32)
    return narrow(out, dtype).reshape(-1)


def rel_err(got_f32: np.ndarray, want_f32: np.ndarray) -> float:
    """max|got - want| / max|want| -- the error measure of the floating-point parity bars."""
    want = np.asarray(want_f32, dtype=np.float64)
    got = np.asarray(got_f32, dtype=np.float64)
    scale = np.max(np.abs(want)) if want.size else 0.0
    if scale == 0.0:
        return float(np.max(np.abs(got))) if got.size else 0.0
    return float(np.max(np.abs(got - want)) / scale)
