// Split over K for products whose output is too small to occupy the GPU.
//
// A product with few output tiles and a long K (config 1 of the benchmark: 512 x 768 outputs,
// 48 tiles of 128 x 64 on 148 SMs) leaves most SMs idle while each busy one walks the whole K.
// Here K is cut into S equal slices that run as the S "batches" of one launch of the tensor-core
// kernel (operand batch stride = K/S along K; f32 partial results [S][M][N] in scratch), and a
// small second kernel adds the partials in slice order, applies scale and bias and converts.
// The order of additions is fixed, so results do not depend on timing.  The reference has no
// counterpart: its kernels give every output element to one thread that walks all of K
// (crates/hodu_cuda_kernels/kernels/ops_matrix.cu:9-102).
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <stdlib.h>

#include "common.cuh"

namespace hodu_b200 {
namespace {

struct ReduceParams {
  const float* parts;   // [S][M][N]
  void* out;
  const void* bias;     // [N] of the output dtype (offset applied) or null
  long long bias_stride;
  unsigned bias_flags;
  int splits;
  long long M, N, ldc;
  float alpha;
};

template <typename T> __device__ __forceinline__ float widen_out(T x);
template <> __device__ __forceinline__ float widen_out<float>(float x) { return x; }
template <> __device__ __forceinline__ float widen_out<__nv_bfloat16>(__nv_bfloat16 x) { return __bfloat162float(x); }
template <> __device__ __forceinline__ float widen_out<__half>(__half x) { return __half2float(x); }
template <typename T> __device__ __forceinline__ T narrow_out(float x);
template <> __device__ __forceinline__ float narrow_out<float>(float x) { return x; }
template <> __device__ __forceinline__ __nv_bfloat16 narrow_out<__nv_bfloat16>(float x) { return __float2bfloat16_rn(x); }
template <> __device__ __forceinline__ __half narrow_out<__half>(float x) { return __float2half_rn(x); }

// One thread per four consecutive columns of one output row (N is a multiple of 4 here).
template <typename T>
__global__ void __launch_bounds__(256) reduce_partials_kernel(const ReduceParams p) {
  const long long quads_per_row = p.N / 4;
  const long long total = p.M * quads_per_row;
  const long long plane = p.M * p.N;
  for (long long i = blockIdx.x * 256ll + threadIdx.x; i < total; i += gridDim.x * 256ll) {
    const long long row = i / quads_per_row, col = (i - row * quads_per_row) * 4;
    const float* src = p.parts + row * p.N + col;
    float4 acc = *reinterpret_cast<const float4*>(src);
    for (int s = 1; s < p.splits; ++s) {
      const float4 v = *reinterpret_cast<const float4*>(src + s * plane);
      acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
    }
    float r[4] = {acc.x * p.alpha, acc.y * p.alpha, acc.z * p.alpha, acc.w * p.alpha};
    if (p.bias) {
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        float x = r[j];
        if (p.bias_flags == HODU_B200_LINEAR_ROUND_EACH_OP) x = widen_out<T>(narrow_out<T>(x));
        r[j] = x + widen_out<T>(static_cast<const T*>(p.bias)[(col + j) * p.bias_stride]);
      }
    }
    T* dst = static_cast<T*>(p.out) + row * p.ldc + col;
#pragma unroll
    for (int j = 0; j < 4; ++j) dst[j] = narrow_out<T>(r[j]);
  }
}

// Number of K slices, or 1 when splitting does not apply.
int pick_splits(const Problem& pb, const DeviceState* st) {
  if (pb.no_scratch || pb.swiglu || pb.batches != 1 || pb.ldc < 0) return 1;
  int esize;
  switch (pb.in_dtype) {
    case HODU_DTYPE_BF16: case HODU_DTYPE_F16: esize = 2; break;
    case HODU_DTYPE_F8E4M3: esize = 1; break;
    case HODU_DTYPE_F32: if (!pb.f32_presplit) return 1; esize = 4; break;
    default: return 1;
  }
  if (pb.out_dtype != HODU_DTYPE_F32 && pb.out_dtype != HODU_DTYPE_BF16 && pb.out_dtype != HODU_DTYPE_F16) return 1;
  if (pb.N % 4 != 0) return 1;
  // Worth it when even 128 x 256 tiles would leave half of the SMs idle; as many slices as bring
  // the count of such tiles up to the SM count (at most 8, at least eight k-blocks each).
  const long long tiles = ((pb.M + 127) / 128) * ((pb.N + 255) / 256);
  if (tiles * 2 > st->sm_count) return 1;
  const long long k_blocks = pb.K * esize / 128;
  long long s = st->sm_count / tiles;
  if (s > 8) s = 8;
  if (s > k_blocks / 8) s = k_blocks / 8;       // at least eight k-blocks per slice
  if (const char* e = getenv("HODU_B200_SPLITK")) {   // tuning aid: upper bound on the slices
    const long long cap = atoi(e);
    if (cap >= 1 && s > cap) s = cap;
  }
  // Two slices do not pay for the partial sums and the second launch (measured on 1024^3 and
  // 1536^3: 30 % and 20 % slower than the whole product); three or more do.
  for (; s >= 3; --s)
    if (pb.K % s == 0 && (pb.K / s * esize) % 128 == 0) return static_cast<int>(s);
  return 1;
}

}  // namespace

int launch_gemm_tc_splitk(const Problem& pb, DeviceState* st, cudaStream_t stream, const char** why) {
  const int splits = forced_path() == HODU_B200_PATH_AUTO || forced_path() == HODU_B200_PATH_TENSOR ? pick_splits(pb, st) : 1;
  if (splits <= 1) return launch_gemm_tc(pb, st, stream, why);
  // The tensor-core kernel can slice K itself, across the CTAs of a cluster and without scratch
  // or a second launch; where its planner would, that is the faster of the two.
  // (Measured exception: a K so long that the cluster's slices would still be 32 k-blocks or more
  // while this path has twice as many slices -- 256 x 8192 x 2048 -- stays here.)
  const int in_kernel = tc_planned_k_slices(pb, st);
  const long long k_blocks = pb.K * dtype_size(pb.in_dtype) / 128;
  if (in_kernel > 1 && !(splits >= 2 * in_kernel && k_blocks / in_kernel >= 32)) return launch_gemm_tc(pb, st, stream, why);
  Problem q = pb;
  q.K = pb.K / splits;
  q.batch_ndim = 1;
  q.batch_shape[0] = splits;
  q.batches = splits;
  q.a.bstride[0] = q.K * pb.a.stride_c;
  q.b.bstride[0] = q.K * pb.b.stride_r;
  q.out_dtype = HODU_DTYPE_F32;
  q.alpha = 1.0f;
  q.bias = nullptr;
  q.ldc = 0;
  void* parts = nullptr;
  const size_t bytes = static_cast<size_t>(splits) * pb.M * pb.N * sizeof(float);
  if (const int ra = scratch_alloc(st, &parts, bytes, stream)) return ra;
  q.out = parts;
  int r = launch_gemm_tc(q, st, stream, why);
  if (r == 0) {
    ReduceParams rp{};
    rp.parts = static_cast<const float*>(parts);
    rp.out = pb.out;
    rp.bias = pb.bias ? static_cast<const uint8_t*>(pb.bias) + pb.bias_offset * dtype_size(pb.out_dtype) : nullptr;
    rp.bias_stride = pb.bias_stride;
    rp.bias_flags = pb.bias_flags;
    rp.splits = splits;
    rp.M = pb.M; rp.N = pb.N; rp.ldc = pb.ldc > 0 ? pb.ldc : pb.N;
    rp.alpha = pb.alpha;
    const long long quads = pb.M * (pb.N / 4);
    long long blocks = (quads + 255) / 256;
    const long long cap = static_cast<long long>(st->sm_count) * 8;
    if (blocks > cap) blocks = cap;
    const unsigned g = static_cast<unsigned>(blocks < 1 ? 1 : blocks);
    if (pb.out_dtype == HODU_DTYPE_F32) reduce_partials_kernel<float><<<g, 256, 0, stream>>>(rp);
    else if (pb.out_dtype == HODU_DTYPE_BF16) reduce_partials_kernel<__nv_bfloat16><<<g, 256, 0, stream>>>(rp);
    else reduce_partials_kernel<__half><<<g, 256, 0, stream>>>(rp);
    const cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) r = fail(HODU_B200_ERR_LAUNCH, "reduce_partials launch failed: %s", cudaGetErrorString(e));
    else count_launch();
  }
  const int rf = scratch_free(parts, stream);
  if (r == 1) return launch_gemm_tc(pb, st, stream, why);  // the sliced form was refused: run it whole
  return r ? r : rf;
}

}  // namespace hodu_b200
