// f32 <-> bf16 | f16 | f8e4m3 (and i8 -> i32) as coalesced 128-bit HBM streams.
// Replaces `hodu_cuda_cast_{src}_to_{dst}`
// (crates/hodu_cuda_kernels/kernels/ops_cast.cu:7-30): one scalar load and store
// per thread with a 32-bit index there; here each thread moves 16 bytes of the
// narrow type per step, the grid is sized to the SM count, and indices are 64-bit.
// Rounding matches the reference's CUDA conversions: to bf16 / f16 round to
// nearest even (`__nv_bfloat16(x)`, `__half(x)`), to f8e4m3 round to nearest even
// and saturate to +-448, NaN kept (`__nv_fp8_e4m3(x)`; math.cuh:42-54,
// ops_cast.cu:115-118).  Widening directions are exact.
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>

#include "common.cuh"

namespace hodu_b200 {
namespace {

template <typename S, typename D> struct Conv;
template <> struct Conv<float, __nv_bfloat16> { static __device__ __nv_bfloat16 f(float x) { return __float2bfloat16_rn(x); } };
template <> struct Conv<float, __half> { static __device__ __half f(float x) { return __float2half_rn(x); } };
template <> struct Conv<float, __nv_fp8_e4m3> {
  static __device__ __nv_fp8_e4m3 f(float x) {
    __nv_fp8_e4m3 r;
    r.__x = __nv_cvt_float_to_fp8(x, __NV_SATFINITE, __NV_E4M3);
    return r;
  }
};
template <> struct Conv<__nv_bfloat16, float> { static __device__ float f(__nv_bfloat16 x) { return __bfloat162float(x); } };
template <> struct Conv<__half, float> { static __device__ float f(__half x) { return __half2float(x); } };
template <> struct Conv<__nv_fp8_e4m3, float> { static __device__ float f(__nv_fp8_e4m3 x) { return static_cast<float>(x); } };
template <> struct Conv<int8_t, int32_t> { static __device__ int32_t f(int8_t x) { return x; } };
// The remaining pairs hodu_core wires for CUDA (be_cuda/storage.rs:652-673), with the
// reference's conversions: (double)x, (float)x, (int32_t)x (toward zero), (float)i
// (ops_cast.cu:119,126,134,239).
template <> struct Conv<float, double> { static __device__ double f(float x) { return static_cast<double>(x); } };
template <> struct Conv<double, float> { static __device__ float f(double x) { return static_cast<float>(x); } };
template <> struct Conv<float, int32_t> { static __device__ int32_t f(float x) { return static_cast<int32_t>(x); } };
template <> struct Conv<int32_t, float> { static __device__ float f(int32_t x) { return static_cast<float>(x); } };
template <> struct Conv<float, uint32_t> { static __device__ uint32_t f(float x) { return static_cast<uint32_t>(x); } };
template <> struct Conv<uint32_t, float> { static __device__ float f(uint32_t x) { return static_cast<float>(x); } };
// Same-type "conversion": the strided -> contiguous copy (`contiguous`), by element width.
template <> struct Conv<uint8_t, uint8_t> { static __device__ uint8_t f(uint8_t x) { return x; } };
template <> struct Conv<uint16_t, uint16_t> { static __device__ uint16_t f(uint16_t x) { return x; } };
template <> struct Conv<uint32_t, uint32_t> { static __device__ uint32_t f(uint32_t x) { return x; } };
template <> struct Conv<uint64_t, uint64_t> { static __device__ uint64_t f(uint64_t x) { return x; } };

template <typename T, int N> struct alignas(sizeof(T) * N) Pack { T v[N]; };

// Contiguous fast path.  VEC = elements per thread per step, chosen so that the
// narrow side moves 16 bytes; the wide side then moves VEC*4 bytes as 16-byte pieces.
template <typename S, typename D, int VEC>
__global__ void __launch_bounds__(256) cast_contig_kernel(const S* __restrict__ in, D* __restrict__ out,
                                                          size_t n) {
  const size_t nvec = n / VEC;
  const size_t stride = static_cast<size_t>(gridDim.x) * blockDim.x;
  for (size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < nvec; i += stride) {
    Pack<S, VEC> src;
    constexpr int kSrcPieces = sizeof(S) * VEC / 16;
    const uint4* sp = reinterpret_cast<const uint4*>(in) + i * kSrcPieces;
#pragma unroll
    for (int j = 0; j < kSrcPieces; ++j) reinterpret_cast<uint4*>(&src)[j] = __ldcs(sp + j);
    Pack<D, VEC> dst;
#pragma unroll
    for (int j = 0; j < VEC; ++j) dst.v[j] = Conv<S, D>::f(src.v[j]);
    constexpr int kDstPieces = sizeof(D) * VEC / 16;
    uint4* dp = reinterpret_cast<uint4*>(out) + i * kDstPieces;
#pragma unroll
    for (int j = 0; j < kDstPieces; ++j) __stcs(dp + j, reinterpret_cast<uint4*>(&dst)[j]);
  }
  // ragged tail (fewer than VEC elements)
  const size_t tail0 = nvec * VEC;
  const size_t t = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (t < n - tail0) out[tail0 + t] = Conv<S, D>::f(in[tail0 + t]);
}

struct StridedMeta {
  int ndim;
  long long shape[8];
  long long strides[8];
};

// Any layout (or unaligned pointers): one element per thread per step.
template <typename S, typename D>
__global__ void __launch_bounds__(256) cast_strided_kernel(const S* __restrict__ in, D* __restrict__ out,
                                                           size_t n, const StridedMeta m) {
  const size_t stride = static_cast<size_t>(gridDim.x) * blockDim.x;
  for (size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += stride) {
    size_t rem = i;
    long long off = 0;
    for (int d = m.ndim - 1; d >= 0; --d) {
      off += static_cast<long long>(rem % m.shape[d]) * m.strides[d];
      rem /= m.shape[d];
    }
    out[i] = Conv<S, D>::f(in[off]);
  }
}

template <typename S, typename D>
int run_cast(const void* in_base, void* out, size_t n, bool contiguous, const StridedMeta& m,
             DeviceState* st, cudaStream_t stream) {
  if (n == 0) return 0;
  constexpr int kNarrow = sizeof(S) < sizeof(D) ? sizeof(S) : sizeof(D);
  constexpr int VEC = 16 / kNarrow;
  const S* in = static_cast<const S*>(in_base);
  const bool aligned = reinterpret_cast<uintptr_t>(in) % 16 == 0 && reinterpret_cast<uintptr_t>(out) % 16 == 0;
  if (contiguous && aligned) {
    const size_t nvec = n / VEC;
    size_t blocks = (nvec + 255) / 256;
    const size_t cap = static_cast<size_t>(st->sm_count) * 16;  // grid-stride beyond this
    if (blocks > cap) blocks = cap;
    if (blocks == 0) blocks = 1;
    cast_contig_kernel<S, D, VEC><<<static_cast<unsigned>(blocks), 256, 0, stream>>>(in, static_cast<D*>(out), n);
  } else {
    StridedMeta mm = m;
    if (contiguous) { mm.ndim = 1; mm.shape[0] = static_cast<long long>(n); mm.strides[0] = 1; }
    size_t blocks = (n + 255) / 256;
    const size_t cap = static_cast<size_t>(st->sm_count) * 16;
    if (blocks > cap) blocks = cap;
    cast_strided_kernel<S, D><<<static_cast<unsigned>(blocks), 256, 0, stream>>>(in, static_cast<D*>(out), n, mm);
  }
  HODU_CUDA_TRY(cudaGetLastError(), HODU_B200_ERR_LAUNCH);
  count_launch();
  return 0;
}

}  // namespace

int launch_cast(int src, int dst, const void* in, void* out, const size_t* md, size_t md_len,
                int device, cudaStream_t stream) {
  if (!md || md_len < 3) return fail(HODU_B200_ERR_INVALID_INPUT, "cast: metadata too short");
  const size_t n = md[0], ndim = md[1];
  if (ndim > 64 || md_len != 3 + 2 * ndim)   // the bound first: 2 * ndim wraps for ndim >= 2^63
    return fail(HODU_B200_ERR_INVALID_INPUT, "cast: metadata length %zu does not match ndim %zu", md_len, ndim);
  const size_t* shape = md + 2;
  const size_t* strides = md + 2 + ndim;
  const size_t offset = md[2 + 2 * ndim];
  size_t prod = 1;
  for (size_t d = 0; d < ndim; ++d) prod *= shape[d];
  if (prod != n) return fail(HODU_B200_ERR_INVALID_INPUT, "cast: num_els %zu != product of shape %zu", n, prod);
  if (n == 0) return 0;
  if (!in || !out) return fail(HODU_B200_ERR_INVALID_INPUT, "cast: null pointer");

  // Row-major contiguity, ignoring dims of extent 1 (same rule as the reference's
  // `is_contiguous`, crates/hodu_cuda_kernels/kernels/utils.cuh).
  bool contiguous = true;
  {
    size_t expect = 1;
    for (size_t d = ndim; d-- > 0;) {
      if (shape[d] != 1 && strides[d] != expect) { contiguous = false; break; }
      expect *= shape[d];
    }
  }
  StridedMeta m{};
  if (!contiguous) {
    // Drop extent-1 dims; more than 8 remaining dims is not supported.
    int k = 0;
    for (size_t d = 0; d < ndim; ++d) {
      if (shape[d] == 1) continue;
      if (k == 8) return fail(HODU_B200_ERR_INVALID_INPUT, "cast: more than 8 non-unit dims in a strided input");
      m.shape[k] = static_cast<long long>(shape[d]);
      m.strides[k] = static_cast<long long>(strides[d]);
      ++k;
    }
    m.ndim = k;
  }
  const uint8_t* base = static_cast<const uint8_t*>(in) + offset * dtype_size(src);
  const bool known = (src == HODU_DTYPE_F32 && (dst == HODU_DTYPE_BF16 || dst == HODU_DTYPE_F16 || dst == HODU_DTYPE_F8E4M3)) ||
                     (dst == HODU_DTYPE_F32 && (src == HODU_DTYPE_BF16 || src == HODU_DTYPE_F16 || src == HODU_DTYPE_F8E4M3)) ||
                     (src == HODU_DTYPE_I8 && dst == HODU_DTYPE_I32) ||
                     (src == HODU_DTYPE_F32 && (dst == HODU_DTYPE_F64 || dst == HODU_DTYPE_I32 || dst == HODU_DTYPE_U32)) ||
                     (dst == HODU_DTYPE_F32 && (src == HODU_DTYPE_F64 || src == HODU_DTYPE_I32 || src == HODU_DTYPE_U32)) ||
                     (src == dst && dtype_size(src) > 0);
  if (!known) return fail(HODU_B200_ERR_INVALID_KERNEL, "cast: unsupported pair %s -> %s", dtype_name(src), dtype_name(dst));
  // Arguments are valid: only now is the device touched.
  DeviceState* st = device_state(device);
  if (!st) return HODU_B200_ERR_NOT_INITIALISED;
  DeviceGuard guard(device);
  if (!guard.ok) return fail(HODU_B200_ERR_LAUNCH, "cannot select CUDA device %d", device);

#define HODU_CAST(SD, DD, S, D) \
  if (src == SD && dst == DD) return run_cast<S, D>(base, out, n, contiguous, m, st, stream)
  HODU_CAST(HODU_DTYPE_F32, HODU_DTYPE_BF16, float, __nv_bfloat16);
  HODU_CAST(HODU_DTYPE_F32, HODU_DTYPE_F16, float, __half);
  HODU_CAST(HODU_DTYPE_F32, HODU_DTYPE_F8E4M3, float, __nv_fp8_e4m3);
  HODU_CAST(HODU_DTYPE_BF16, HODU_DTYPE_F32, __nv_bfloat16, float);
  HODU_CAST(HODU_DTYPE_F16, HODU_DTYPE_F32, __half, float);
  HODU_CAST(HODU_DTYPE_F8E4M3, HODU_DTYPE_F32, __nv_fp8_e4m3, float);
  HODU_CAST(HODU_DTYPE_I8, HODU_DTYPE_I32, int8_t, int32_t);
  HODU_CAST(HODU_DTYPE_F32, HODU_DTYPE_F64, float, double);
  HODU_CAST(HODU_DTYPE_F64, HODU_DTYPE_F32, double, float);
  HODU_CAST(HODU_DTYPE_F32, HODU_DTYPE_I32, float, int32_t);
  HODU_CAST(HODU_DTYPE_I32, HODU_DTYPE_F32, int32_t, float);
  HODU_CAST(HODU_DTYPE_F32, HODU_DTYPE_U32, float, uint32_t);
  HODU_CAST(HODU_DTYPE_U32, HODU_DTYPE_F32, uint32_t, float);
#undef HODU_CAST
  if (src == dst) {
    switch (dtype_size(src)) {
      case 1: return run_cast<uint8_t, uint8_t>(base, out, n, contiguous, m, st, stream);
      case 2: return run_cast<uint16_t, uint16_t>(base, out, n, contiguous, m, st, stream);
      case 4: return run_cast<uint32_t, uint32_t>(base, out, n, contiguous, m, st, stream);
      case 8: return run_cast<uint64_t, uint64_t>(base, out, n, contiguous, m, st, stream);
      default: break;
    }
  }
  return fail(HODU_B200_ERR_INVALID_KERNEL, "cast: unsupported pair %s -> %s", dtype_name(src), dtype_name(dst));
}

}  // namespace hodu_b200
