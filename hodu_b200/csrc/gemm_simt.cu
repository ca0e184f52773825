// Generic strided GEMM on the CUDA cores: any strides, offsets and batch
// broadcast the matmul / dot wire formats can express, every supported dtype
// pair.  It takes the calls the tcgen05 kernel cannot describe to TMA (unaligned
// bases or pitches, tiny shapes) and f32, and doubles as a second, independent
// GPU implementation the tests cross-check the tensor-core path against.
//
// Arithmetic follows what the reference's result means after widening: operands
// are widened to f32 (s32 for integers), products accumulate in f32 (s32), and the
// sum is converted once at the end.  The reference kernels
// (crates/hodu_cuda_kernels/kernels/ops_matrix.cu:56,76-80) re-round the running
// sum to the storage type at every k instead; that is not reproduced.
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>

#include <type_traits>

#include "common.cuh"

namespace hodu_b200 {
namespace {

constexpr int TM = 64, TN = 64, TK = 16;  // tile of one 256-thread CTA; 4x4 outputs per thread

struct SimtParams {
  const void* a;
  const void* b;
  const void* b2;
  void* out;
  long long M, N, K;
  long long a_sr, a_sc, b_sr, b_sc, b2_sr, b2_sc;  // element strides (offset already applied)
  int batch_ndim;
  long long batches;       // product of bshape[0..batch_ndim)
  long long bshape[16];
  long long a_bs[16], b_bs[16], b2_bs[16];
  float alpha;
  unsigned swiglu_flags;
  long long tiles_m, tiles_n, ldc;
  const void* bias;        // [N] of TOut (offset applied), or null
  long long bias_stride;
  unsigned bias_flags;
};

template <typename T> struct Widen;
template <> struct Widen<float> { using acc = float; static __device__ float get(float x) { return x; } };
template <> struct Widen<__nv_bfloat16> { using acc = float; static __device__ float get(__nv_bfloat16 x) { return __bfloat162float(x); } };
template <> struct Widen<__half> { using acc = float; static __device__ float get(__half x) { return __half2float(x); } };
template <> struct Widen<__nv_fp8_e4m3> { using acc = float; static __device__ float get(__nv_fp8_e4m3 x) { return static_cast<float>(x); } };
template <> struct Widen<int8_t> { using acc = int; static __device__ int get(int8_t x) { return x; } };
template <> struct Widen<int32_t> { using acc = int; static __device__ int get(int32_t x) { return x; } };

template <typename TOut, typename TAcc> struct Narrow;
template <> struct Narrow<float, float> { static __device__ float put(float x) { return x; } };
template <> struct Narrow<__nv_bfloat16, float> { static __device__ __nv_bfloat16 put(float x) { return __float2bfloat16_rn(x); } };
template <> struct Narrow<__half, float> { static __device__ __half put(float x) { return __float2half_rn(x); } };
template <> struct Narrow<__nv_fp8_e4m3, float> {
  static __device__ __nv_fp8_e4m3 put(float x) {
    __nv_fp8_e4m3 r;
    r.__x = __nv_cvt_float_to_fp8(x, __NV_SATFINITE, __NV_E4M3);
    return r;
  }
};
template <> struct Narrow<int32_t, int> { static __device__ int32_t put(int x) { return x; } };
template <> struct Narrow<int8_t, int> { static __device__ int8_t put(int x) { return static_cast<int8_t>(x & 0xFF); } };

__device__ __forceinline__ float silu_ref(float x) { return x / (1.0f + expf(-x)); }

template <typename TIn, typename TOut, bool SWIGLU>
__global__ void __launch_bounds__(256) gemm_simt_kernel(const SimtParams p) {
  using W = Widen<TIn>;
  using Acc = typename W::acc;
  __shared__ Acc As[TK][TM + 4];
  __shared__ Acc Bs[TK][TN + 4];
  __shared__ Acc B2s[SWIGLU ? TK : 1][TN + 4];

  const long long per_batch = p.tiles_m * p.tiles_n;
  for (long long tile = blockIdx.x; tile < per_batch * p.batches; tile += gridDim.x) {
    const long long batch = tile / per_batch;
    const long long r = tile - batch * per_batch;
    const long long m0 = (r / p.tiles_n) * TM;
    const long long n0 = (r % p.tiles_n) * TN;

    long long a_base = 0, b_base = 0, b2_base = 0;
    {
      long long rem = batch;
      for (int d = p.batch_ndim - 1; d >= 0; --d) {
        const long long idx = rem % p.bshape[d];
        rem /= p.bshape[d];
        a_base += idx * p.a_bs[d];
        b_base += idx * p.b_bs[d];
        if (SWIGLU) b2_base += idx * p.b2_bs[d];
      }
    }
    const TIn* A = static_cast<const TIn*>(p.a) + a_base;
    const TIn* B = static_cast<const TIn*>(p.b) + b_base;
    const TIn* B2 = SWIGLU ? static_cast<const TIn*>(p.b2) + b2_base : nullptr;

    Acc acc[4][4] = {};
    Acc acc2[SWIGLU ? 4 : 1][4] = {};
    const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;

    for (long long k0 = 0; k0 < p.K; k0 += TK) {
      // 64x16 and 16x64 elements: four per thread each.  The index that is
      // contiguous in memory is walked by neighbouring threads.
      for (int e = threadIdx.x; e < TM * TK; e += 256) {
        int i, k;
        if (p.a_sc == 1) { k = e % TK; i = e / TK; } else { i = e % TM; k = e / TM; }
        const long long gi = m0 + i, gk = k0 + k;
        As[k][i] = (gi < p.M && gk < p.K) ? W::get(A[gi * p.a_sr + gk * p.a_sc]) : Acc(0);
      }
      for (int e = threadIdx.x; e < TN * TK; e += 256) {
        int j, k;
        if (p.b_sc == 1) { j = e % TN; k = e / TN; } else { k = e % TK; j = e / TK; }
        const long long gj = n0 + j, gk = k0 + k;
        const bool in = gj < p.N && gk < p.K;
        Bs[k][j] = in ? W::get(B[gk * p.b_sr + gj * p.b_sc]) : Acc(0);
        if (SWIGLU) B2s[k][j] = in ? W::get(B2[gk * p.b2_sr + gj * p.b2_sc]) : Acc(0);
      }
      __syncthreads();
#pragma unroll
      for (int k = 0; k < TK; ++k) {
        Acc av[4], bv[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) av[i] = As[k][ty * 4 + i];
#pragma unroll
        for (int j = 0; j < 4; ++j) bv[j] = Bs[k][tx * 4 + j];
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
          for (int j = 0; j < 4; ++j) acc[i][j] += av[i] * bv[j];
        if (SWIGLU) {
#pragma unroll
          for (int j = 0; j < 4; ++j) bv[j] = B2s[k][tx * 4 + j];
#pragma unroll
          for (int i = 0; i < 4; ++i)
#pragma unroll
            for (int j = 0; j < 4; ++j) acc2[i][j] += av[i] * bv[j];
        }
      }
      __syncthreads();
    }

    TOut* O = static_cast<TOut*>(p.out) + batch * p.M * p.ldc;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const long long gi = m0 + ty * 4 + i;
      if (gi >= p.M) continue;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const long long gj = n0 + tx * 4 + j;
        if (gj >= p.N) continue;
        if constexpr (SWIGLU) {
          float g = static_cast<float>(acc[i][j]), u = static_cast<float>(acc2[i][j]);
          float v;
          if (p.swiglu_flags == HODU_B200_SWIGLU_ROUND_EACH_OP) {
            g = Widen<TOut>::get(Narrow<TOut, float>::put(g));
            u = Widen<TOut>::get(Narrow<TOut, float>::put(u));
            const float s = Widen<TOut>::get(Narrow<TOut, float>::put(silu_ref(g)));
            v = s * u;
          } else {
            v = silu_ref(g) * u;
          }
          O[gi * p.ldc + gj] = Narrow<TOut, float>::put(v);
        } else if constexpr (std::is_same<Acc, float>::value) {
          float v = acc[i][j] * p.alpha;
          if (p.bias) {
            if (p.bias_flags == HODU_B200_LINEAR_ROUND_EACH_OP) v = Widen<TOut>::get(Narrow<TOut, float>::put(v));
            v += Widen<TOut>::get(static_cast<const TOut*>(p.bias)[gj * p.bias_stride]);
          }
          O[gi * p.ldc + gj] = Narrow<TOut, Acc>::put(v);
        } else {
          O[gi * p.ldc + gj] = Narrow<TOut, Acc>::put(acc[i][j]);
        }
      }
    }
  }
}

template <typename TIn, typename TOut, bool SWIGLU>
int launch_one(const SimtParams& p, int grid, cudaStream_t stream) {
  gemm_simt_kernel<TIn, TOut, SWIGLU><<<grid, 256, 0, stream>>>(p);
  HODU_CUDA_TRY(cudaGetLastError(), HODU_B200_ERR_LAUNCH);
  count_launch();
  return 0;
}

}  // namespace

int launch_gemm_simt(const Problem& pb, DeviceState* st, cudaStream_t stream) {
  const int esize = dtype_size(pb.in_dtype);
  SimtParams p{};
  p.a = static_cast<const uint8_t*>(pb.a.ptr) + pb.a.offset * esize;
  p.b = static_cast<const uint8_t*>(pb.b.ptr) + pb.b.offset * esize;
  p.b2 = pb.swiglu ? static_cast<const uint8_t*>(pb.b2.ptr) + pb.b2.offset * esize : nullptr;
  p.out = pb.out;
  p.M = pb.M; p.N = pb.N; p.K = pb.K;
  p.a_sr = pb.a.stride_r; p.a_sc = pb.a.stride_c;
  p.b_sr = pb.b.stride_r; p.b_sc = pb.b.stride_c;
  p.b2_sr = pb.b2.stride_r; p.b2_sc = pb.b2.stride_c;
  if (pb.batch_ndim > 16) return fail(HODU_B200_ERR_INVALID_INPUT, "more than 16 batch dims");
  p.batch_ndim = pb.batch_ndim;
  for (int d = 0; d < pb.batch_ndim; ++d) {
    p.bshape[d] = pb.batch_shape[d];
    p.a_bs[d] = pb.a.bstride[d];
    p.b_bs[d] = pb.b.bstride[d];
    p.b2_bs[d] = pb.b2.bstride[d];
  }
  p.batches = pb.batches;
  p.alpha = pb.alpha;
  p.swiglu_flags = pb.swiglu_flags;
  p.bias = pb.bias ? static_cast<const uint8_t*>(pb.bias) + pb.bias_offset * dtype_size(pb.out_dtype) : nullptr;
  p.bias_stride = pb.bias_stride;
  p.bias_flags = pb.bias_flags;
  p.ldc = pb.ldc > 0 ? pb.ldc : pb.N;
  p.tiles_m = (pb.M + TM - 1) / TM;
  p.tiles_n = (pb.N + TN - 1) / TN;
  const long long tiles = p.tiles_m * p.tiles_n * pb.batches;
  if (tiles <= 0) return 0;  // nothing to write
  const long long cap = static_cast<long long>(st->sm_count) * 8;
  const int grid = static_cast<int>(tiles < cap ? tiles : cap);

  const int in = pb.in_dtype, out = pb.out_dtype;
#define HODU_SIMT(TI, TO) return launch_one<TI, TO, false>(p, grid, stream)
  if (pb.swiglu) {
    if (in == HODU_DTYPE_BF16 && out == HODU_DTYPE_BF16) return launch_one<__nv_bfloat16, __nv_bfloat16, true>(p, grid, stream);
    if (in == HODU_DTYPE_F16 && out == HODU_DTYPE_F16) return launch_one<__half, __half, true>(p, grid, stream);
    if (in == HODU_DTYPE_F32 && out == HODU_DTYPE_F32) return launch_one<float, float, true>(p, grid, stream);
    return fail(HODU_B200_ERR_INVALID_KERNEL, "swiglu: unsupported dtype %s -> %s", dtype_name(in), dtype_name(out));
  }
  if (in == HODU_DTYPE_F32 && out == HODU_DTYPE_F32) HODU_SIMT(float, float);
  if (in == HODU_DTYPE_BF16 && out == HODU_DTYPE_BF16) HODU_SIMT(__nv_bfloat16, __nv_bfloat16);
  if (in == HODU_DTYPE_BF16 && out == HODU_DTYPE_F32) HODU_SIMT(__nv_bfloat16, float);
  if (in == HODU_DTYPE_F16 && out == HODU_DTYPE_F16) HODU_SIMT(__half, __half);
  if (in == HODU_DTYPE_F16 && out == HODU_DTYPE_F32) HODU_SIMT(__half, float);
  if (in == HODU_DTYPE_F8E4M3 && out == HODU_DTYPE_BF16) HODU_SIMT(__nv_fp8_e4m3, __nv_bfloat16);
  if (in == HODU_DTYPE_F8E4M3 && out == HODU_DTYPE_F16) HODU_SIMT(__nv_fp8_e4m3, __half);
  if (in == HODU_DTYPE_F8E4M3 && out == HODU_DTYPE_F32) HODU_SIMT(__nv_fp8_e4m3, float);
  if (in == HODU_DTYPE_F8E4M3 && out == HODU_DTYPE_F8E4M3) HODU_SIMT(__nv_fp8_e4m3, __nv_fp8_e4m3);
  if (in == HODU_DTYPE_I8 && out == HODU_DTYPE_I32) HODU_SIMT(int8_t, int32_t);
  if (in == HODU_DTYPE_I8 && out == HODU_DTYPE_I8) HODU_SIMT(int8_t, int8_t);
  if (in == HODU_DTYPE_I32 && out == HODU_DTYPE_I32) HODU_SIMT(int32_t, int32_t);
#undef HODU_SIMT
  return fail(HODU_B200_ERR_INVALID_KERNEL, "matmul: unsupported dtype pair %s -> %s", dtype_name(in),
              dtype_name(out));
}

}  // namespace hodu_b200
