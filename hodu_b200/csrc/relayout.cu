// Layout front door of the tensor-core GEMM: an operand TMA cannot describe (a pitch or base
// address that is not a multiple of 16 bytes, neither matrix index contiguous) is first copied
// into stream-ordered scratch as a dense K-contiguous matrix with a 16-byte-multiple pitch, and
// the tcgen05 kernel then runs on the copy.  In the reference the same situation is met by
// `contiguous()` (crates/hodu_core/src/be_cuda/storage.rs:681-709 ->
// hodu_cuda_contiguous_*, crates/hodu_cuda_kernels/kernels/ops_memory.cu:6-27), a one-thread-per-
// element gather; here the copy goes through 32x32 shared-memory tiles so that reads follow the
// source's contiguous index and writes follow K.  Broadcast batch dims are copied once.
#include "common.cuh"

namespace hodu_b200 {
namespace {

struct CopyParams {
  const void* src;
  void* dst;
  long long mn, k;          // logical [mn, k] view of one matrix
  long long s_mn, s_k;      // source element strides
  long long nb;             // physical (non-broadcast) batches
  int nbd;
  long long bshape[3], bstride[3];
  long long pitch;          // destination pitch in elements
  long long mat_elems;
  long long tiles_mn, tiles_k;
};

template <typename T>
__global__ void __launch_bounds__(256) relayout_kernel(const CopyParams p) {
  __shared__ T tile[32][32 + 4 / sizeof(T)];
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
  const long long per = p.tiles_mn * p.tiles_k;
  const bool k_fast = (p.s_k == 1) || (p.s_mn != 1);
  for (long long t = blockIdx.x; t < per * p.nb; t += gridDim.x) {
    const long long b = t / per, r = t - b * per;
    const long long mn0 = (r / p.tiles_k) * 32, k0 = (r % p.tiles_k) * 32;
    long long boff = 0, rem = b;
    for (int d = p.nbd - 1; d >= 0; --d) { boff += (rem % p.bshape[d]) * p.bstride[d]; rem /= p.bshape[d]; }
    const T* src = static_cast<const T*>(p.src) + boff;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int i_mn = k_fast ? ty + 8 * j : tx;
      const int i_k = k_fast ? tx : ty + 8 * j;
      const long long g_mn = mn0 + i_mn, g_k = k0 + i_k;
      if (g_mn < p.mn && g_k < p.k) tile[i_mn][i_k] = src[g_mn * p.s_mn + g_k * p.s_k];
    }
    __syncthreads();
    T* dst = static_cast<T*>(p.dst) + b * p.mat_elems;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const long long g_mn = mn0 + ty + 8 * j, g_k = k0 + tx;
      if (g_mn < p.mn && g_k < p.k) dst[g_mn * p.pitch + g_k] = tile[ty + 8 * j][tx];
    }
    __syncthreads();
  }
}

struct CopyPlan {
  CopyParams cp;
  size_t bytes;
  Operand out;
};

bool plan_copy(const Problem& pb, const Operand& op, bool is_lhs, int esize, CopyPlan* plan) {
  CopyParams& cp = plan->cp;
  cp = CopyParams{};
  cp.mn = is_lhs ? pb.M : pb.N;
  cp.k = pb.K;
  cp.s_mn = is_lhs ? op.stride_r : op.stride_c;
  cp.s_k = is_lhs ? op.stride_c : op.stride_r;
  const long long unit = 16 / esize;
  cp.pitch = (cp.k + unit - 1) / unit * unit;
  cp.mat_elems = cp.pitch * cp.mn;
  cp.tiles_mn = (cp.mn + 31) / 32;
  cp.tiles_k = (cp.k + 31) / 32;
  cp.nb = 1;
  plan->out = Operand{};
  long long dense = cp.mat_elems;
  int dims[16], n = 0;
  for (int d = 0; d < pb.batch_ndim; ++d)
    if (pb.batch_shape[d] > 1 && op.bstride[d] != 0) dims[n++] = d;
  if (n > 3) return false;
  for (int j = n - 1; j >= 0; --j) {
    plan->out.bstride[dims[j]] = dense;
    dense *= pb.batch_shape[dims[j]];
  }
  for (int j = 0; j < n; ++j) {
    cp.bshape[j] = pb.batch_shape[dims[j]];
    cp.bstride[j] = op.bstride[dims[j]];
    cp.nb *= cp.bshape[j];
  }
  cp.nbd = n;
  plan->bytes = (static_cast<size_t>(dense) * esize + 255) / 256 * 256;
  plan->out.offset = 0;
  plan->out.stride_r = is_lhs ? cp.pitch : 1;   // K-contiguous either way
  plan->out.stride_c = is_lhs ? 1 : cp.pitch;
  return true;
}

int run_copy(const CopyPlan& plan, const Operand& op, int esize, void* dst, DeviceState* st, cudaStream_t stream) {
  CopyParams cp = plan.cp;
  cp.src = static_cast<const uint8_t*>(op.ptr) + op.offset * esize;
  cp.dst = dst;
  long long blocks = cp.tiles_mn * cp.tiles_k * cp.nb;
  const long long cap = static_cast<long long>(st->sm_count) * 32;
  if (blocks > cap) blocks = cap;
  if (blocks < 1) return 0;
  const unsigned g = static_cast<unsigned>(blocks);
  if (esize == 1) relayout_kernel<uint8_t><<<g, 256, 0, stream>>>(cp);
  else if (esize == 2) relayout_kernel<uint16_t><<<g, 256, 0, stream>>>(cp);
  else relayout_kernel<uint32_t><<<g, 256, 0, stream>>>(cp);
  HODU_CUDA_TRY(cudaGetLastError(), HODU_B200_ERR_LAUNCH);
  count_launch();
  return 0;
}

}  // namespace

// Returns 1 (nothing launched) when no operand needs a copy or the problem cannot be helped,
// otherwise the result of the tensor-core launch on the re-laid operands.
int launch_gemm_tc_relayout(const Problem& pb, DeviceState* st, cudaStream_t stream, const char** why) {
  const int esize = dtype_size(pb.in_dtype);
  if (pb.in_dtype == HODU_DTYPE_F32 || esize > 2) return 1;
  const bool need_a = !tc_operand_describable(pb, pb.a, true, esize);
  bool need_b = !tc_operand_describable(pb, pb.b, false, esize);
  bool need_b2 = pb.swiglu && !tc_operand_describable(pb, pb.b2, false, esize);
  if (pb.swiglu && (need_b || need_b2)) need_b = need_b2 = true;  // gate and up must end up alike
  if (!need_a && !need_b) return 1;
  CopyPlan pa, pbp, pb2;
  size_t total = 0;
  if (need_a) { if (!plan_copy(pb, pb.a, true, esize, &pa)) return 1; total += pa.bytes; }
  if (need_b) { if (!plan_copy(pb, pb.b, false, esize, &pbp)) return 1; total += pbp.bytes; }
  if (need_b2) { if (!plan_copy(pb, pb.b2, false, esize, &pb2)) return 1; total += pb2.bytes; }
  uint8_t* scratch = nullptr;
  if (const int ra = scratch_alloc(st, reinterpret_cast<void**>(&scratch), total, stream)) return ra;
  Problem q = pb;
  uint8_t* cur = scratch;
  int r = 0;
  if (need_a) { r = run_copy(pa, pb.a, esize, cur, st, stream); q.a = pa.out; q.a.ptr = cur; cur += pa.bytes; }
  if (!r && need_b) { r = run_copy(pbp, pb.b, esize, cur, st, stream); q.b = pbp.out; q.b.ptr = cur; cur += pbp.bytes; }
  if (!r && need_b2) { r = run_copy(pb2, pb.b2, esize, cur, st, stream); q.b2 = pb2.out; q.b2.ptr = cur; cur += pb2.bytes; }
  if (!r) r = launch_gemm_tc(q, st, stream, why);
  const int rf = scratch_free(scratch, stream);
  return r ? r : rf;
}

}  // namespace hodu_b200
