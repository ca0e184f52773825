// f32 matmul on the tensor cores: C = A . B computed as three TF32 products of split
// operands (A = Ahi + Alo, B = Bhi + Blo; C ~= Ahi.Bhi + Ahi.Blo + Alo.Bhi, f32 accumulate),
// which keeps ~21 bits per product -- inside the 1e-4 bar of the f32 configuration, where one
// plain TF32 product (10-bit mantissa) is not.  The reference computes f32 products on CUDA
// cores (crates/hodu_cuda_kernels/kernels/ops_matrix.cu:9-102); on B200 the same result comes
// ~10x sooner this way.
//
// Step 1 (this file): one pass over each operand writes its split form into SCRATCH memory,
//   A' = [Ahi | Ahi | Alo] (M x 3K) and B'^T = [Bhi | Blo | Bhi] (N x 3K), both K-contiguous with
//   a 16-byte-multiple pitch.  (With an M- or N-contiguous operand kind::tf32 returned zeros on
//   this hardware, so the split pass transposes through shared memory where needed; reads and
//   writes both stay coalesced.)  Any strides and offsets are accepted on the way in;
//   broadcast batch dims are split once.
// Step 2: the tcgen05 kernel (gemm_tc.cu, kind::tf32) multiplies A' [M,3K] by B' [3K,N].
// The scratch comes from the stream-ordered allocator on the caller's stream, so concurrent
// calls on different streams never share it.
#include <mutex>

#include "common.cuh"

namespace hodu_b200 {
namespace {

struct SplitParams {
  const float* src;
  float* dst;
  long long mn, k;               // logical [mn, k] view of one matrix (mn = M for lhs, N for rhs)
  long long s_mn, s_k;           // source element strides of those two indices
  long long nb;                  // physical (non-broadcast) batch count
  int nbd;                       // physical batch dims (<= 3)
  long long bshape[3], bstride[3];
  long long pitch;               // destination pitch in elements (>= 3k, multiple of 4)
  long long mat_elems;           // destination elements per matrix (pitch * mn)
  int lo_part;                   // which of the three K segments holds the low part (2 lhs, 1 rhs)
  long long tiles_mn, tiles_k;
};

__device__ __forceinline__ float tf32_round(float x) {
  uint32_t u;
  asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(u) : "f"(x));
  return __uint_as_float(u);
}

// 32 x 32 tiles, 256 threads (32 x 8).  The source is read along whichever of its two indices
// is contiguous; the destination is always written along k.
__device__ __forceinline__ void split_tf32_body(const SplitParams& p, unsigned block, unsigned blocks) {
  __shared__ float tile[32][33];
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
  const long long per = p.tiles_mn * p.tiles_k;
  const bool k_fast = (p.s_k == 1) || (p.s_mn != 1);
  for (long long t = block; t < per * p.nb; t += blocks) {
    const long long b = t / per, r = t - b * per;
    const long long mn0 = (r / p.tiles_k) * 32, k0 = (r % p.tiles_k) * 32;
    long long boff = 0, rem = b;
    for (int d = p.nbd - 1; d >= 0; --d) { boff += (rem % p.bshape[d]) * p.bstride[d]; rem /= p.bshape[d]; }
    const float* src = p.src + boff;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int i_mn = k_fast ? ty + 8 * j : tx;
      const int i_k = k_fast ? tx : ty + 8 * j;
      const long long g_mn = mn0 + i_mn, g_k = k0 + i_k;
      tile[i_mn][i_k] = (g_mn < p.mn && g_k < p.k) ? src[g_mn * p.s_mn + g_k * p.s_k] : 0.0f;
    }
    __syncthreads();
    float* dst = p.dst + b * p.mat_elems;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const long long g_mn = mn0 + ty + 8 * j, g_k = k0 + tx;
      if (g_mn < p.mn && g_k < p.k) {
        const float x = tile[ty + 8 * j][tx];
        const float hi = tf32_round(x), lo = tf32_round(x - hi);  // both rounded to nearest: no truncation bias in the MMA
        float* row = dst + g_mn * p.pitch + g_k;
        row[0] = hi;
        row[p.k] = (p.lo_part == 1) ? lo : hi;
        row[2 * p.k] = (p.lo_part == 2) ? lo : hi;
      }
    }
    __syncthreads();
  }
}

// Both operands of one product in one launch: the first `blocks_a` CTAs split the lhs, the
// rest the rhs.
__global__ void __launch_bounds__(256) split_tf32_kernel(const SplitParams pa, const SplitParams pb, unsigned blocks_a) {
  // The product kernel that follows waits for this grid before it reads the split operands
  // (griddepcontrol.wait); letting it launch now overlaps its set-up with this pass.
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  if (blockIdx.x < blocks_a) split_tf32_body(pa, blockIdx.x, blocks_a);
  else split_tf32_body(pb, blockIdx.x - blocks_a, gridDim.x - blocks_a);
}

struct SplitPlan {
  SplitParams sp;
  size_t bytes;
  Operand out;  // the split operand as the tensor-core problem sees it (ptr filled in later)
};

// Plans the split of one operand of `pb`; returns false if it has more than three
// non-broadcast batch dims.
bool plan_split(const Problem& pb, const Operand& op, bool is_lhs, SplitPlan* plan) {
  SplitParams& sp = plan->sp;
  sp = SplitParams{};
  sp.mn = is_lhs ? pb.M : pb.N;
  sp.k = pb.K;
  sp.s_mn = is_lhs ? op.stride_r : op.stride_c;
  sp.s_k = is_lhs ? op.stride_c : op.stride_r;
  sp.lo_part = is_lhs ? 2 : 1;
  sp.pitch = (3 * sp.k + 3) / 4 * 4;
  sp.mat_elems = sp.pitch * sp.mn;
  sp.tiles_mn = (sp.mn + 31) / 32;
  sp.tiles_k = (sp.k + 31) / 32;
  sp.nb = 1; sp.nbd = 0;
  plan->out = Operand{};
  long long dense = sp.mat_elems;
  // physical batch dims, innermost last; broadcast dims keep stride 0 in the new operand
  int dims[16], n = 0;
  for (int d = 0; d < pb.batch_ndim; ++d)
    if (pb.batch_shape[d] > 1 && op.bstride[d] != 0) dims[n++] = d;
  if (n > 3) return false;
  for (int j = n - 1; j >= 0; --j) {
    const int d = dims[j];
    plan->out.bstride[d] = dense;
    if (static_cast<__int128>(dense) * pb.batch_shape[d] > (static_cast<__int128>(1) << 50)) return false;  // no such scratch exists
    dense *= pb.batch_shape[d];
  }
  for (int j = 0; j < n; ++j) {
    sp.bshape[j] = pb.batch_shape[dims[j]];
    sp.bstride[j] = op.bstride[dims[j]];
    sp.nb *= sp.bshape[j];
  }
  sp.nbd = n;
  plan->bytes = static_cast<size_t>(dense) * sizeof(float);
  plan->out.offset = 0;
  // K-contiguous: lhs [M, 3K] has strides (pitch, 1); rhs [3K, N] has strides (1, pitch)
  plan->out.stride_r = is_lhs ? sp.pitch : 1;
  plan->out.stride_c = is_lhs ? 1 : sp.pitch;
  return true;
}

int run_splits(const SplitPlan& a, const Operand& opa, float* da, const SplitPlan& b, const Operand& opb, float* db,
               DeviceState* st, cudaStream_t stream) {
  SplitParams pa = a.sp, pb = b.sp;
  pa.src = static_cast<const float*>(opa.ptr) + opa.offset; pa.dst = da;
  pb.src = static_cast<const float*>(opb.ptr) + opb.offset; pb.dst = db;
  const long long cap = static_cast<long long>(st->sm_count) * 16;
  auto blocks_of = [&](const SplitParams& p) {
    long long n = p.tiles_mn * p.tiles_k * p.nb;
    return n > cap ? cap : (n < 1 ? 1 : n);
  };
  const unsigned na = static_cast<unsigned>(blocks_of(pa)), nb = static_cast<unsigned>(blocks_of(pb));
  split_tf32_kernel<<<na + nb, 256, 0, stream>>>(pa, pb, na);
  HODU_CUDA_TRY(cudaGetLastError(), HODU_B200_ERR_LAUNCH);
  count_launch();
  return 0;
}

}  // namespace

size_t gemm_f32_scratch_bytes(const Problem& pb) {
  SplitPlan a, b;
  if (!plan_split(pb, pb.a, true, &a) || !plan_split(pb, pb.b, false, &b)) return 0;
  return ((a.bytes + 255) / 256 * 256) + b.bytes;
}

int launch_gemm_f32_split(const Problem& pb, DeviceState* st, cudaStream_t stream, void* scratch,
                          size_t scratch_bytes, const char** why) {
  static const char* none = "";
  *why = none;
  if (pb.in_dtype != HODU_DTYPE_F32 || pb.out_dtype != HODU_DTYPE_F32 || pb.swiglu) { *why = "not an f32 product"; return 1; }
  if (st->cc_major != 10) { *why = "device is not sm_100"; return 1; }
  if (3 * pb.K > 0x7FFFFFFFll) { *why = "K too large"; return 1; }
  SplitPlan a, b;
  if (!plan_split(pb, pb.a, true, &a) || !plan_split(pb, pb.b, false, &b)) { *why = "more than three batch dims"; return 1; }
  const size_t a_bytes = (a.bytes + 255) / 256 * 256;
  if (a_bytes + b.bytes > scratch_bytes) { *why = "scratch too small"; return 1; }
  float* da = static_cast<float*>(scratch);
  float* db = reinterpret_cast<float*>(static_cast<uint8_t*>(scratch) + a_bytes);
  const int r = run_splits(a, pb.a, da, b, pb.b, db, st, stream);
  if (r) return r;
  Problem q = pb;
  q.K = 3 * pb.K;
  q.a = a.out; q.a.ptr = da;
  q.b = b.out; q.b.ptr = db;
  q.f32_presplit = true;
  return launch_gemm_tc_splitk(q, st, stream, why);
}

// Allocates the scratch on `stream` (stream-ordered pool), runs the split product, frees it.
int launch_gemm_f32(const Problem& pb, DeviceState* st, cudaStream_t stream, const char** why) {
  // Small products first try the one-kernel form (no scratch, one launch); a forced tile form
  // keeps the split-operand path, which is the one that has tile forms.
  const int forced = forced_path();
  if (forced == HODU_B200_PATH_AUTO || forced == HODU_B200_PATH_TENSOR) {
    const int rf = launch_gemm_f32_fused(pb, st, stream, why);
    if (rf != 1) return rf;
  }
  const size_t bytes = gemm_f32_scratch_bytes(pb);
  if (bytes == 0) { *why = "more than three batch dims"; return 1; }
  void* scratch = nullptr;
  if (const int ra = scratch_alloc(st, &scratch, bytes, stream)) return ra;
  const int r = launch_gemm_f32_split(pb, st, stream, scratch, bytes, why);
  const int rf = scratch_free(scratch, stream);
  return r ? r : rf;
}

}  // namespace hodu_b200

// ---------------------------------------------------------------------------------------------
// hodu_b200_dot_f32_static: the same f32 product for callers that must not allocate device
// memory at call time (see include/hodu_b200.h).  The split operands live in the fixed array
// below instead of stream-ordered scratch.  Everything else -- split pass, tcgen05 kernel -- is
// the code above, unchanged.
// ---------------------------------------------------------------------------------------------
namespace hodu_b200 {
namespace {

constexpr size_t kStaticScratchBytes = HODU_B200_STATIC_SCRATCH_BYTES;

// Held by every GPU that loads the library, from load until exit.  In host code these names
// are only handles for cudaGetSymbolAddress; kernels get the address that call returns.
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];
static __device__ uint32_t g_static_status;

struct StaticSetup {
  bool done = false;
  void* scratch = nullptr;     // device address of g_static_scratch on this device
  uint32_t* status = nullptr;  // device address of g_static_status on this device
  int sm_count = 0, cc_major = 0;
};
StaticSetup g_static_setup[kMaxDevices];
std::mutex g_static_mu;

// Once per device, with that device current: resolve the device addresses of the two symbols.
int static_setup(int device, StaticSetup** out) {
  std::lock_guard<std::mutex> lock(g_static_mu);
  StaticSetup* s = &g_static_setup[device];
  if (!s->done) {
    HODU_CUDA_TRY(cudaGetSymbolAddress(&s->scratch, g_static_scratch), HODU_B200_ERR_MEMORY);
    HODU_CUDA_TRY(cudaGetSymbolAddress(reinterpret_cast<void**>(&s->status), g_static_status), HODU_B200_ERR_MEMORY);
    HODU_CUDA_TRY(cudaDeviceGetAttribute(&s->sm_count, cudaDevAttrMultiProcessorCount, device), HODU_B200_ERR_LAUNCH);
    HODU_CUDA_TRY(cudaDeviceGetAttribute(&s->cc_major, cudaDevAttrComputeCapabilityMajor, device), HODU_B200_ERR_LAUNCH);
    if (s->scratch == nullptr || s->status == nullptr)
      return fail(HODU_B200_ERR_MEMORY, "cudaGetSymbolAddress returned a null device address");
    s->done = true;
  }
  *out = s;
  return 0;
}

}  // namespace
}  // namespace hodu_b200

extern "C" int hodu_b200_dot_f32_static(int device, void* stream, const void* lhs, const void* rhs,
                                        void* out, const size_t* metadata, size_t metadata_len) {
  using namespace hodu_b200;
  Problem pb;
  int r = parse_dot(metadata, metadata_len, &pb);
  if (r) return r;
  if (pb.M == 0 || pb.N == 0) return 0;
  if (!out) return fail(HODU_B200_ERR_INVALID_INPUT, "null operand pointer");
  if (device < 0 || device >= kMaxDevices)
    return fail(HODU_B200_ERR_INVALID_INPUT, "device %d out of range 0..%d", device, kMaxDevices - 1);
  pb.in_dtype = HODU_DTYPE_F32; pb.out_dtype = HODU_DTYPE_F32;
  pb.a.ptr = lhs; pb.b.ptr = rhs; pb.out = out;
  pb.no_scratch = true;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  DeviceGuard guard(device);
  if (!guard.ok) return fail(HODU_B200_ERR_LAUNCH, "cannot select CUDA device %d", device);
  if (pb.K == 0) {  // an empty sum is zero; a memset allocates nothing
    HODU_CUDA_TRY(cudaMemsetAsync(out, 0, static_cast<size_t>(pb.M) * pb.N * sizeof(float), s), HODU_B200_ERR_MEMORY);
    return 0;
  }
  if (!lhs || !rhs) return fail(HODU_B200_ERR_INVALID_INPUT, "null operand pointer");
  const size_t need = gemm_f32_scratch_bytes(pb);
  if (need == 0 || need > kStaticScratchBytes)
    return fail(HODU_B200_ERR_INVALID_INPUT,
                "dot_f32_static: this product needs %zu bytes of scratch, the fixed array holds %zu "
                "(12*(M+N)*K bytes must fit); use hodu_b200_dot for larger products",
                need, kStaticScratchBytes);
  StaticSetup* ss = nullptr;
  r = static_setup(device, &ss);
  if (r) return r;
  DeviceState st;  // a local view: nothing of the library's allocated per-device state is touched
  st.ready = true; st.sm_count = ss->sm_count; st.cc_major = ss->cc_major; st.status = ss->status;
  const char* why = "";
  r = launch_gemm_f32_split(pb, &st, s, ss->scratch, kStaticScratchBytes, &why);
  if (r == 1) return fail(HODU_B200_ERR_INVALID_INPUT, "dot_f32_static refused: %s", why);
  if (r == 0) set_last_path(HODU_B200_PATH_TENSOR);
  return r;
}

// Reads (and clears) the status word private to the entry point above.  Allocates nothing and
// does not touch the library's per-device state: it synchronises the device, copies four bytes
// from the address static_setup resolved, and clears the word if it was set.
extern "C" int hodu_b200_dot_f32_static_status(int device, uint32_t* device_status_word) {
  using namespace hodu_b200;
  if (device < 0 || device >= kMaxDevices)
    return fail(HODU_B200_ERR_INVALID_INPUT, "device %d out of range 0..%d", device, kMaxDevices - 1);
  DeviceGuard guard(device);
  if (!guard.ok) return fail(HODU_B200_ERR_LAUNCH, "cannot select CUDA device %d", device);
  StaticSetup* ss = nullptr;
  if (const int r = static_setup(device, &ss)) return r;
  HODU_CUDA_TRY(cudaDeviceSynchronize(), HODU_B200_ERR_LAUNCH);
  uint32_t w = 0;
  HODU_CUDA_TRY(cudaMemcpy(&w, ss->status, sizeof(w), cudaMemcpyDeviceToHost), HODU_B200_ERR_MEMORY);
  if (w != 0) HODU_CUDA_TRY(cudaMemset(ss->status, 0, sizeof(w)), HODU_B200_ERR_MEMORY);
  if (device_status_word) *device_status_word = w;
  if (w != 0)
    return fail(HODU_B200_ERR_DEVICE_STATUS, "static entry point: device status word 0x%08x (cta %u, wait %u)", w,
                (w >> 4) & 0xFFFFu, w & 0xFu);
  return 0;
}
