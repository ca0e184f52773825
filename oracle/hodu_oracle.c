/*
 * TEST INFRASTRUCTURE -- not part of the product.  Only tests/, the smoke check and
 * the cpu_baseline / reference legs of bench.py may build, load or call this file.
 *
 * CPU restatement of the reference algorithm for the matmul / dot / cast path, in
 * plain C.  Each function names the reference code it follows (paths relative to
 * the reference project root).  What "the reference result" means per dtype:
 *
 *  f32          the reference's own f32 matmul: a k-ordered sum per output element
 *               (crates/hodu_cpu_kernels/kernels/ops_matrix.c:46-193, 399-549); with the
 *               `openblas` feature it is cblas_sgemm instead (ops_matrix_openblas.c:19-153),
 *               which differs only in summation order.
 *  bf16/f16/f8  operands widened exactly to f32 (ops_cast.c:132,170,189), the f32 matmul
 *               above, one round-to-nearest-even narrowing of the result.  The
 *               reference's per-dtype CPU kernels re-round the running sum at every k
 *               (ops_matrix.c:196-219, t_bf16.h:35-55) and are NOT the oracle.
 *  i8 -> i32    cast_i8_to_i32 (ops_cast.c:330) then the native-width integer matmul
 *               (ops_matrix.c:357,719): exact.
 *  casts        to f32: exact.  From f32: round to nearest even, f8e4m3 saturating to
 *               +-448 with NaN kept -- what the reference's CUDA casts do
 *               (crates/hodu_cuda_kernels/kernels/ops_cast.cu:115-118, math.cuh:42-54) and what the
 *               Rust-side `half` / `float8` types do.  The reference's C casts differ
 *               (bf16 truncates, t_bf16.h:35-39; its f8e4m3 tops out at 240,
 *               t_f8e4m3.h:32-38,61-63) and are not used.
 *
 * Pinned against: the reference's known-answer tests (tests/test_oracle.py) and
 * the reference's own C kernels compiled from source into oracle/_ref.
 */
#include <math.h>
#include <stddef.h>
#include <stdint.h>
#include <string.h>

/* ------------------------------------------------------------------ codecs */

/* bf16 -> f32: shift into the high half (t_bf16.h:28-33). */
float oracle_bf16_to_f32(uint16_t v) {
    uint32_t bits = (uint32_t)v << 16;
    float f;
    memcpy(&f, &bits, 4);
    return f;
}

/* f32 -> bf16, round to nearest even, NaN stays NaN (`__nv_bfloat16(x)`, math.cuh:50). */
uint16_t oracle_f32_to_bf16(float f) {
    uint32_t bits;
    memcpy(&bits, &f, 4);
    if ((bits & 0x7FFFFFFFu) > 0x7F800000u) return (uint16_t)((bits >> 16) | 0x0040u);
    uint32_t lsb = (bits >> 16) & 1u;
    bits += 0x7FFFu + lsb;
    return (uint16_t)(bits >> 16);
}

/* f16 -> f32 (t_f16.h:27-46), exact. */
float oracle_f16_to_f32(uint16_t v) {
    uint32_t sign = (uint32_t)(v >> 15) << 31, e = (v >> 10) & 0x1F, m = v & 0x3FF, bits;
    if (e == 0x1F) bits = sign | 0x7F800000u | (m << 13);
    else if (e == 0) {
        if (m == 0) bits = sign;
        else {
            int sh = 0;
            while (!(m & 0x400)) { m <<= 1; ++sh; }
            bits = sign | ((uint32_t)(127 - 15 - sh + 1) << 23) | ((m & 0x3FF) << 13);
        }
    } else bits = sign | ((e + 112) << 23) | (m << 13);
    float f;
    memcpy(&f, &bits, 4);
    return f;
}

/* f32 -> f16, round to nearest even, overflow to inf (`__half(x)`, math.cuh:46). */
uint16_t oracle_f32_to_f16(float f) {
    uint32_t bits;
    memcpy(&bits, &f, 4);
    uint16_t sign = (uint16_t)((bits >> 16) & 0x8000u);
    uint32_t abs = bits & 0x7FFFFFFFu;
    if (abs > 0x7F800000u) return (uint16_t)(sign | 0x7E00u | ((abs >> 13) & 0x1FF));
    if (abs >= 0x47800000u) return (uint16_t)(sign | 0x7C00u); /* >= 65536 (rounding below handles 65520) */
    if (abs < 0x33000000u) return sign;                         /* < 2^-25 rounds to 0 */
    int32_t e = (int32_t)(abs >> 23) - 127;
    uint32_t m = (abs & 0x7FFFFFu) | 0x800000u;
    uint32_t shift = e < -14 ? (uint32_t)(13 + (-14 - e)) : 13u;
    uint32_t half = 1u << (shift - 1), rest = m & ((1u << shift) - 1);
    uint32_t q = m >> shift;
    if (rest > half || (rest == half && (q & 1u))) ++q;
    uint32_t out = e < -14 ? q : (((uint32_t)(e + 15) << 10) + (q - 0x400u));
    return (uint16_t)(sign | out); /* a mantissa carry bumps the exponent; 0x7C00 is inf */
}

/* OCP e4m3fn -> f32: bias 7, no infinities, 0x7F / 0xFF are NaN, max finite 448
 * (what `float8::F8E4M3` and `__nv_fp8_e4m3` decode; NOT t_f8e4m3.h, whose exponent 15
 * is inf/NaN). */
float oracle_e4m3_to_f32(uint8_t v) {
    uint32_t s = v >> 7, e = (v >> 3) & 0xF, m = v & 7;
    float r;
    if (e == 0xF && m == 7) return NAN;
    if (e == 0) r = ldexpf((float)m, -9);
    else r = ldexpf(1.0f + (float)m / 8.0f, (int)e - 7);
    return s ? -r : r;
}

/* f32 -> OCP e4m3fn, round to nearest even, saturate finite to +-448, NaN -> 0x7F
 * (`__nv_fp8_e4m3(x)` = cvt.rn.satfinite, ops_cast.cu:115-118). */
uint8_t oracle_f32_to_e4m3(float f) {
    uint32_t bits;
    memcpy(&bits, &f, 4);
    uint8_t sign = (uint8_t)((bits >> 24) & 0x80u);
    uint32_t abs = bits & 0x7FFFFFFFu;
    if (abs > 0x7F800000u) return (uint8_t)(sign | 0x7F);
    float a = fabsf(f);
    if (a >= 448.0f) return (uint8_t)(sign | 0x7E);
    if (a < ldexpf(1.0f, -10)) return sign;            /* below half the smallest subnormal */
    int e;
    (void)frexpf(a, &e);                               /* a = frac * 2^e, frac in [0.5,1) */
    int exp = e - 1;                                   /* a = 1.xxx * 2^exp */
    if (exp < -6) exp = -6;                            /* subnormal range: fixed scale 2^-6 */
    float scaled = ldexpf(a, 3 - exp);                 /* in units of the last mantissa bit */
    float fl = floorf(scaled), rem = scaled - fl;
    uint32_t q = (uint32_t)fl;
    if (rem > 0.5f || (rem == 0.5f && (q & 1u))) ++q;
    /* q in [0,16]: subnormal when exp == -6 and q < 8 */
    uint32_t out;
    if (exp == -6 && q < 8) out = q;
    else {
        if (q == 16) { q = 8; ++exp; }
        out = ((uint32_t)(exp + 7) << 3) | (q - 8);
    }
    if (out > 0x7E) out = 0x7E;
    return (uint8_t)(sign | out);
}

void oracle_cast_bf16_to_f32(const uint16_t *in, float *out, size_t n) { for (size_t i = 0; i < n; i++) out[i] = oracle_bf16_to_f32(in[i]); }
void oracle_cast_f16_to_f32(const uint16_t *in, float *out, size_t n) { for (size_t i = 0; i < n; i++) out[i] = oracle_f16_to_f32(in[i]); }
void oracle_cast_e4m3_to_f32(const uint8_t *in, float *out, size_t n) { for (size_t i = 0; i < n; i++) out[i] = oracle_e4m3_to_f32(in[i]); }
void oracle_cast_f32_to_bf16(const float *in, uint16_t *out, size_t n) { for (size_t i = 0; i < n; i++) out[i] = oracle_f32_to_bf16(in[i]); }
void oracle_cast_f32_to_f16(const float *in, uint16_t *out, size_t n) { for (size_t i = 0; i < n; i++) out[i] = oracle_f32_to_f16(in[i]); }
void oracle_cast_f32_to_e4m3(const float *in, uint8_t *out, size_t n) { for (size_t i = 0; i < n; i++) out[i] = oracle_f32_to_e4m3(in[i]); }
/* i8 -> i32 (ops_cast.c:330): sign extension. */
void oracle_cast_i8_to_i32(const int8_t *in, int32_t *out, size_t n) { for (size_t i = 0; i < n; i++) out[i] = in[i]; }

/* Strided cast input gather, [num_els, ndim, shape.., strides.., offset] (ops_cast.c:34-103):
 * writes the flat source index of each of the n output elements. */
void oracle_cast_indices(const size_t *md, size_t *idx_out) {
    size_t n = md[0], nd = md[1];
    const size_t *shape = md + 2, *strides = md + 2 + nd;
    size_t off = md[2 + 2 * nd];
    for (size_t i = 0; i < n; i++) {
        size_t rem = i, s = off;
        for (size_t d = nd; d-- > 0;) { s += (rem % shape[d]) * strides[d]; rem /= shape[d]; }
        idx_out[i] = s;
    }
}

/* ------------------------------------------------------------------ matmul */

/* Batched matmul with broadcasting over the reference wire format
 * [num_els, lhs_ndim, rhs_ndim, batch_ndim, lhs_shape.., rhs_shape.., batch_shape..,
 *  lhs_strides.., rhs_strides.., lhs_off, rhs_off, M, K, N]: the general path of
 * ops_matrix.c:144-193 (decompose the flat batch index, right-align each operand's
 * batch dims, extent-1 dims stay at index 0, sum over k in order). */
#define ORACLE_MATMUL(NAME, T, ACC)                                                              \
    void NAME(const T *lhs, const T *rhs, T *out, const size_t *md) {                            \
        size_t num_els = md[0], ln = md[1], rn = md[2], bn = md[3];                              \
        const size_t *lshape = md + 4, *rshape = lshape + ln, *bshape = rshape + rn;             \
        const size_t *lstr = bshape + bn, *rstr = lstr + ln, *t = rstr + rn;                     \
        size_t loff = t[0], roff = t[1], M = t[2], K = t[3], N = t[4];                           \
        size_t lb = ln - 2, rb = rn - 2;                                                         \
        for (size_t idx = 0; idx < num_els; idx++) {                                             \
            size_t mn = idx % (M * N), b = idx / (M * N), i = mn / N, j = mn % N;                \
            size_t bi[16], tmp = b;                                                              \
            for (size_t d = bn; d-- > 0;) { bi[d] = tmp % bshape[d]; tmp /= bshape[d]; }         \
            size_t lbase = loff, rbase = roff;                                                   \
            for (size_t d = 0; d < lb; d++) lbase += (lshape[d] == 1 ? 0 : bi[bn - lb + d]) * lstr[d]; \
            for (size_t d = 0; d < rb; d++) rbase += (rshape[d] == 1 ? 0 : bi[bn - rb + d]) * rstr[d]; \
            ACC sum = 0;                                                                         \
            for (size_t k = 0; k < K; k++)                                                       \
                sum += (ACC)lhs[lbase + i * lstr[ln - 2] + k * lstr[ln - 1]] *                   \
                       (ACC)rhs[rbase + k * rstr[rn - 2] + j * rstr[rn - 1]];                    \
            out[idx] = (T)sum;                                                                   \
        }                                                                                        \
    }
ORACLE_MATMUL(oracle_matmul_f32, float, float)      /* MATMUL_OP(f32_t, f32_fallback), ops_matrix.c:342 */
ORACLE_MATMUL(oracle_matmul_i32, int32_t, uint32_t) /* MATMUL_OP(int32_t, i32), ops_matrix.c:357; wraps */
ORACLE_MATMUL(oracle_matmul_i8, int8_t, uint8_t)    /* MATMUL_OP(int8_t, i8), ops_matrix.c:355; wraps to 8 bits */

/* 2-D dot over [M, K, N, lhs_sm, lhs_sk, rhs_sk, rhs_sn, lhs_off, rhs_off]
 * (ops_matrix.c:423-549): C[i,j] = sum_k A[i,k] * B[k,j]. */
#define ORACLE_DOT(NAME, T, ACC)                                                                 \
    void NAME(const T *lhs, const T *rhs, T *out, const size_t *md) {                            \
        size_t M = md[0], K = md[1], N = md[2];                                                  \
        for (size_t i = 0; i < M; i++)                                                           \
            for (size_t j = 0; j < N; j++) {                                                     \
                ACC sum = 0;                                                                     \
                for (size_t k = 0; k < K; k++)                                                   \
                    sum += (ACC)lhs[md[7] + i * md[3] + k * md[4]] * (ACC)rhs[md[8] + k * md[5] + j * md[6]]; \
                out[i * N + j] = (T)sum;                                                         \
            }                                                                                    \
    }
ORACLE_DOT(oracle_dot_f32, float, float)
ORACLE_DOT(oracle_dot_i32, int32_t, uint32_t)
ORACLE_DOT(oracle_dot_i8, int8_t, uint8_t)

/* silu (math_utils.h:184; CUDA math.cuh:232-235). */
void oracle_silu_f32(const float *in, float *out, size_t n) {
    for (size_t i = 0; i < n; i++) out[i] = in[i] / (1.0f + expf(-in[i]));
}
