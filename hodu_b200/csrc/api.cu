// C ABI of libhodu_b200: metadata parsing, layout checks, path selection,
// per-device state and the pipelined host-buffer forms.  See include/hodu_b200.h
// for the contract of each entry point and the reference interface it replaces.
#include <stdarg.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include <atomic>
#include <mutex>

#include "common.cuh"

namespace hodu_b200 {

// ------------------------------------------------------------------ errors
namespace {
thread_local char g_msg[512] = "";
thread_local int g_last_path = HODU_B200_PATH_AUTO;
std::atomic<int> g_forced_path{HODU_B200_PATH_AUTO};
std::atomic<unsigned long long> g_launches{0};
std::mutex g_state_mu;
DeviceState g_state[kMaxDevices];
// Published with release order once every field of g_state[d] is written; readers that see it
// set (acquire) may use the state without taking the lock.
std::atomic<bool> g_state_ready[kMaxDevices];

// Tensor-core path only above this much work; below it one CUDA-core CTA wave
// finishes sooner than the TMA/TMEM pipeline fills.
constexpr long long kTensorMinWork = 1ll << 21;     // M*N*K*batches
constexpr long long kTensorMinWorkRelayout = 1ll << 24;  // an operand copy precedes the product
constexpr long long kTensorMinWorkF32 = 1ll << 24;  // f32 pays two operand-split launches first
constexpr long long kTensorMinWorkF32Fused = 1ll << 18;  // ... unless the one-kernel form takes the product
}  // namespace

int fail(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_msg, sizeof(g_msg), fmt, ap);
  va_end(ap);
  return code;
}

const char* dtype_name(int dt) {
  static const char* names[] = {"bool", "f8e4m3", "f8e5m2", "bf16", "f16", "f32", "f64", "u8",
                                "u16",  "u32",    "u64",    "i8",   "i16", "i32", "i64"};
  return (dt >= 0 && dt <= 14) ? names[dt] : "?";
}

void count_launch(unsigned n) { g_launches.fetch_add(n, std::memory_order_relaxed); }
void set_last_path(int path) { g_last_path = path; }
int forced_path() {
  // HODU_B200_FORCE_PATH=<n> presets the selector (same values as hodu_b200_force_path).
  static const bool env_read = [] {
    const char* e = getenv("HODU_B200_FORCE_PATH");
    if (e && e[0] >= '0' && e[0] <= '5' && e[1] == 0) g_forced_path.store(e[0] - '0');
    return true;
  }();
  (void)env_read;
  return g_forced_path.load(std::memory_order_relaxed);
}

DeviceGuard::DeviceGuard(int device) {
  if (cudaGetDevice(&prev) != cudaSuccess) { prev = -1; }
  // Always set the device, also when it already is the current one: on a thread that has made
  // no CUDA call yet this is what binds the device's primary context to the thread, and the
  // driver entry points used afterwards (tensor-map encoding) need a current context.
  ok = cudaSetDevice(device) == cudaSuccess;
  if (prev == device) prev = -1;  // nothing to restore
}
DeviceGuard::~DeviceGuard() {
  if (prev >= 0) cudaSetDevice(prev);
}

DeviceState* device_state(int device) {
  if (device < 0 || device >= kMaxDevices) {
    fail(HODU_B200_ERR_INVALID_INPUT, "device %d out of range 0..%d", device, kMaxDevices - 1);
    return nullptr;
  }
  DeviceState* st = &g_state[device];
  if (g_state_ready[device].load(std::memory_order_acquire)) return st;
  std::lock_guard<std::mutex> lock(g_state_mu);
  if (g_state_ready[device].load(std::memory_order_relaxed)) return st;
  DeviceGuard guard(device);
  if (!guard.ok) {
    fail(HODU_B200_ERR_LAUNCH, "cannot select CUDA device %d", device);
    return nullptr;
  }
  cudaDeviceProp prop;
  if (cudaGetDeviceProperties(&prop, device) != cudaSuccess) {
    fail(HODU_B200_ERR_LAUNCH, "cannot query CUDA device %d: %s", device, cudaGetErrorString(cudaGetLastError()));
    return nullptr;
  }
  st->sm_count = prop.multiProcessorCount;
  st->cc_major = prop.major;
  st->cc_minor = prop.minor;
  st->smem_optin = prop.sharedMemPerBlockOptin;
  st->device = device;
  if (cudaMalloc(&st->status, sizeof(uint32_t)) != cudaSuccess ||
      cudaMemset(st->status, 0, sizeof(uint32_t)) != cudaSuccess) {
    fail(HODU_B200_ERR_MEMORY, "cannot allocate the device status word on device %d", device);
    st->status = nullptr;
    return nullptr;
  }
  st->ready = true;
  g_state_ready[device].store(true, std::memory_order_release);
  return st;
}

int scratch_alloc(DeviceState* st, void** ptr, size_t bytes, cudaStream_t stream) {
  cudaMemPool_t pool_now = nullptr;
  {
    // The pool pointer is read and created under the lock (an allocation follows anyway, so the
    // lock costs nothing that matters).
    std::lock_guard<std::mutex> lock(g_state_mu);
    if (!st->pool) {
      cudaMemPoolProps props = {};
      props.allocType = cudaMemAllocationTypePinned;
      props.handleTypes = cudaMemHandleTypeNone;
      props.location.type = cudaMemLocationTypeDevice;
      props.location.id = st->device;
      cudaMemPool_t pool = nullptr;
      HODU_CUDA_TRY(cudaMemPoolCreate(&pool, &props), HODU_B200_ERR_MEMORY);
      unsigned long long keep = ~0ull;  // never trim at synchronisation points
      HODU_CUDA_TRY(cudaMemPoolSetAttribute(pool, cudaMemPoolAttrReleaseThreshold, &keep), HODU_B200_ERR_MEMORY);
      st->pool = pool;
    }
    pool_now = st->pool;
  }
  HODU_CUDA_TRY(cudaMallocFromPoolAsync(ptr, bytes, pool_now, stream), HODU_B200_ERR_MEMORY);
  return 0;
}

int scratch_free(void* ptr, cudaStream_t stream) {
  const cudaError_t e = cudaFreeAsync(ptr, stream);
  if (e != cudaSuccess) return fail(HODU_B200_ERR_MEMORY, "cudaFreeAsync failed: %s", cudaGetErrorString(e));
  return 0;
}

// ------------------------------------------------------------------ metadata
namespace {

bool in_out_pair_ok(int in, int out) {
  switch (in) {
    case HODU_DTYPE_F8E4M3:
      return out == HODU_DTYPE_BF16 || out == HODU_DTYPE_F16 || out == HODU_DTYPE_F32 || out == HODU_DTYPE_F8E4M3;
    case HODU_DTYPE_I8: return out == HODU_DTYPE_I32 || out == HODU_DTYPE_I8;
    case HODU_DTYPE_BF16: return out == HODU_DTYPE_BF16 || out == HODU_DTYPE_F32;
    case HODU_DTYPE_F16: return out == HODU_DTYPE_F16 || out == HODU_DTYPE_F32;
    case HODU_DTYPE_F32: return out == HODU_DTYPE_F32;
    case HODU_DTYPE_I32: return out == HODU_DTYPE_I32;
    default: return false;
  }
}
bool is_int_dtype(int dt) { return dt == HODU_DTYPE_I8 || dt == HODU_DTYPE_I32; }
}  // namespace

namespace {
constexpr unsigned long long kMaxExtent = 1ull << 32;
constexpr unsigned long long kMaxSpan = 1ull << 48;

// Elements between the first and the last element an operand view touches, or ~0 if any of its
// numbers is out of range.  128-bit arithmetic: the inputs are arbitrary 64-bit words.
unsigned long long operand_span(const Operand& op, int64_t rows, int64_t cols, const Problem& pb) {
  unsigned __int128 span = 0;
  auto add = [&](int64_t extent, int64_t stride) {
    if (extent < 0 || static_cast<unsigned long long>(extent) > kMaxExtent || stride < 0 ||
        static_cast<unsigned long long>(stride) > kMaxSpan)
      return false;
    if (extent > 1) span += static_cast<unsigned __int128>(extent - 1) * static_cast<unsigned long long>(stride);
    return span <= kMaxSpan;
  };
  if (op.offset < 0 || static_cast<unsigned long long>(op.offset) > kMaxSpan) return ~0ull;
  span = static_cast<unsigned long long>(op.offset);
  if (!add(rows, op.stride_r) || !add(cols, op.stride_c)) return ~0ull;
  for (int d = 0; d < pb.batch_ndim; ++d)
    if (!add(pb.batch_shape[d], op.bstride[d])) return ~0ull;
  return static_cast<unsigned long long>(span);
}
}  // namespace

int check_extents(const Problem& pb) {
  const char* what = nullptr;
  if (pb.batch_ndim < 0 || pb.batch_ndim > 16) what = "batch rank";
  unsigned __int128 out_elems = 1, batches = 1;
  for (int d = 0; !what && d < pb.batch_ndim; ++d) {
    if (pb.batch_shape[d] < 0 || static_cast<unsigned long long>(pb.batch_shape[d]) > kMaxExtent) what = "batch extent";
    else batches *= static_cast<unsigned long long>(pb.batch_shape[d]);
    if (batches > kMaxSpan) what = "batch count";
  }
  if (!what && (pb.M < 0 || pb.N < 0 || pb.K < 0 || static_cast<unsigned long long>(pb.M) > kMaxExtent ||
                static_cast<unsigned long long>(pb.N) > kMaxExtent || static_cast<unsigned long long>(pb.K) > kMaxExtent))
    what = "M, N or K";
  if (!what) {
    out_elems = batches * static_cast<unsigned long long>(pb.M) * static_cast<unsigned long long>(pb.N);
    const unsigned __int128 a_elems = static_cast<unsigned __int128>(pb.M) * static_cast<unsigned long long>(pb.K);
    const unsigned __int128 b_elems = static_cast<unsigned __int128>(pb.K) * static_cast<unsigned long long>(pb.N);
    if (out_elems > kMaxSpan || a_elems > kMaxSpan || b_elems > kMaxSpan) what = "element count";
  }
  if (!what && operand_span(pb.a, pb.M, pb.K, pb) == ~0ull) what = "lhs strides or offset";
  if (!what && operand_span(pb.b, pb.K, pb.N, pb) == ~0ull) what = "rhs strides or offset";
  if (!what && pb.swiglu && operand_span(pb.b2, pb.K, pb.N, pb) == ~0ull) what = "second rhs strides or offset";
  if (what)
    return fail(HODU_B200_ERR_INVALID_INPUT, "%s out of range (extents up to 2^32, strides, offsets and element counts up to 2^48)", what);
  return 0;
}

// [num_els, lhs_ndim, rhs_ndim, batch_ndim, lhs_shape.., rhs_shape.., batch_shape..,
//  lhs_strides.., rhs_strides.., lhs_off, rhs_off, M, K, N]
// (crates/hodu_core/src/op_metadatas.rs:192-290). Batch dims align to the right
// and an operand dim of extent 1 broadcasts
// (crates/hodu_cuda_kernels/kernels/ops_matrix.cu:27-55).
int parse_matmul(const size_t* md, size_t len, Problem* pb) {
  if (!md || len < 4) return fail(HODU_B200_ERR_INVALID_INPUT, "matmul: metadata too short (%zu)", len);
  const size_t num_els = md[0], ln = md[1], rn = md[2], bn = md[3];
  if (ln < 2 || rn < 2 || ln > 18 || rn > 18 || bn > 16)
    return fail(HODU_B200_ERR_INVALID_INPUT, "matmul: bad ranks lhs=%zu rhs=%zu batch=%zu", ln, rn, bn);
  if (len != 9 + 2 * (ln + rn) + bn)
    return fail(HODU_B200_ERR_INVALID_INPUT, "matmul: metadata length %zu, expected %zu", len, 9 + 2 * (ln + rn) + bn);
  const size_t* lshape = md + 4;
  const size_t* rshape = lshape + ln;
  const size_t* bshape = rshape + rn;
  const size_t* lstr = bshape + bn;
  const size_t* rstr = lstr + ln;
  const size_t* t = rstr + rn;
  const size_t loff = t[0], roff = t[1], M = t[2], K = t[3], N = t[4];
  if (lshape[ln - 2] != M || lshape[ln - 1] != K || rshape[rn - 2] != K || rshape[rn - 1] != N)
    return fail(HODU_B200_ERR_INVALID_INPUT, "matmul: M,K,N = %zu,%zu,%zu disagree with operand shapes", M, K, N);
  if (ln - 2 > bn || rn - 2 > bn)
    return fail(HODU_B200_ERR_INVALID_INPUT, "matmul: operand has more batch dims than the output");
  pb->M = M; pb->K = K; pb->N = N;
  pb->batch_ndim = static_cast<int>(bn);
  pb->batches = 1;
  for (size_t d = 0; d < bn; ++d) {
    if (bshape[d] > kMaxExtent || static_cast<unsigned __int128>(pb->batches) * bshape[d] > kMaxSpan)
      return fail(HODU_B200_ERR_INVALID_INPUT, "matmul: batch extents out of range");
    pb->batch_shape[d] = static_cast<int64_t>(bshape[d]);
    pb->batches *= static_cast<int64_t>(bshape[d]);
    pb->a.bstride[d] = 0;
    pb->b.bstride[d] = 0;
  }
  if (M > kMaxExtent || N > kMaxExtent || K > kMaxExtent)
    return fail(HODU_B200_ERR_INVALID_INPUT, "matmul: M, N or K out of range");
  for (size_t d = 0; d + 2 < ln; ++d) {
    const size_t od = bn - (ln - 2) + d;
    if (lshape[d] != 1 && lshape[d] != bshape[od])
      return fail(HODU_B200_ERR_INVALID_INPUT, "matmul: lhs batch dim %zu (%zu) does not broadcast to %zu", d, lshape[d], bshape[od]);
    pb->a.bstride[od] = lshape[d] == 1 ? 0 : static_cast<int64_t>(lstr[d]);
  }
  for (size_t d = 0; d + 2 < rn; ++d) {
    const size_t od = bn - (rn - 2) + d;
    if (rshape[d] != 1 && rshape[d] != bshape[od])
      return fail(HODU_B200_ERR_INVALID_INPUT, "matmul: rhs batch dim %zu (%zu) does not broadcast to %zu", d, rshape[d], bshape[od]);
    pb->b.bstride[od] = rshape[d] == 1 ? 0 : static_cast<int64_t>(rstr[d]);
  }
  if (static_cast<unsigned __int128>(num_els) != static_cast<unsigned __int128>(pb->batches) * M * N)
    return fail(HODU_B200_ERR_INVALID_INPUT, "matmul: num_els %zu != batches*M*N", num_els);
  pb->a.offset = static_cast<int64_t>(loff);
  pb->b.offset = static_cast<int64_t>(roff);
  pb->a.stride_r = static_cast<int64_t>(lstr[ln - 2]);
  pb->a.stride_c = static_cast<int64_t>(lstr[ln - 1]);
  pb->b.stride_r = static_cast<int64_t>(rstr[rn - 2]);
  pb->b.stride_c = static_cast<int64_t>(rstr[rn - 1]);
  return check_extents(*pb);
}

// [M, K, N, lhs_stride_m, lhs_stride_k, rhs_stride_k, rhs_stride_n, lhs_off, rhs_off]
// (crates/hodu_core/src/op_metadatas.rs:464-506)
int parse_dot(const size_t* md, size_t len, Problem* pb) {
  if (!md || len != 9) return fail(HODU_B200_ERR_INVALID_INPUT, "dot: metadata length %zu, expected 9", len);
  pb->M = md[0]; pb->K = md[1]; pb->N = md[2];
  pb->a.stride_r = md[3]; pb->a.stride_c = md[4];
  pb->b.stride_r = md[5]; pb->b.stride_c = md[6];
  pb->a.offset = md[7]; pb->b.offset = md[8];
  pb->batch_ndim = 0;
  pb->batches = 1;
  return check_extents(*pb);
}

namespace {
// Clears the output of a K == 0 product (an empty sum is zero).
int zero_output(const Problem& pb, cudaStream_t stream) {
  const size_t bytes = static_cast<size_t>(pb.batches) * pb.M * pb.N * dtype_size(pb.out_dtype);
  if (bytes == 0) return 0;
  HODU_CUDA_TRY(cudaMemsetAsync(pb.out, 0, bytes, stream), HODU_B200_ERR_MEMORY);
  return 0;
}

}  // namespace

// Chooses the kernel family for a validated problem and launches it.
int run_problem(const Problem& pb, DeviceState* st, cudaStream_t stream) {
  if (pb.M == 0 || pb.N == 0 || pb.batches == 0) { set_last_path(HODU_B200_PATH_AUTO); return 0; }
  if (pb.K == 0) { set_last_path(HODU_B200_PATH_AUTO); return zero_output(pb, stream); }
  const int forced = forced_path();
  const long long work = static_cast<long long>(pb.M) * pb.N * pb.K * pb.batches;
  const bool forced_tc = forced >= HODU_B200_PATH_TENSOR && forced <= HODU_B200_PATH_TENSOR_2CTA_512;
  const long long min_work = pb.in_dtype == HODU_DTYPE_F32 ? kTensorMinWorkF32 : kTensorMinWork;
  const bool want_tc = forced_tc || (forced == HODU_B200_PATH_AUTO && work >= min_work);
  if (want_tc) {
    const char* why = "";
    const int r = pb.in_dtype == HODU_DTYPE_F32 ? launch_gemm_f32(pb, st, stream, &why)
                                                : launch_gemm_tc_splitk(pb, st, stream, &why);
    if (r == 0) { set_last_path(HODU_B200_PATH_TENSOR); return 0; }
    if (r < 0) return r;
    // A layout TMA cannot take: with enough work to pay for it, copy the operand(s) first.
    if (work >= kTensorMinWorkRelayout || forced_tc) {
      const char* why2 = "";
      const int r2 = launch_gemm_tc_relayout(pb, st, stream, &why2);
      if (r2 == 0) { set_last_path(HODU_B200_PATH_TENSOR); return 0; }
      if (r2 < 0) return r2;
    }
    if (forced_tc) return fail(HODU_B200_ERR_INVALID_INPUT, "tensor-core path refused: %s", why);
  }
  if (!want_tc && forced == HODU_B200_PATH_AUTO && pb.in_dtype == HODU_DTYPE_F32 && work >= kTensorMinWorkF32Fused) {
    // too small for the split-operand path, but the one-kernel f32 form costs a single launch
    const char* why = "";
    const int r = launch_gemm_f32_fused(pb, st, stream, &why);
    if (r == 0) { set_last_path(HODU_B200_PATH_TENSOR); return 0; }
    if (r < 0) return r;
  }
  set_last_path(HODU_B200_PATH_SIMT);
  return launch_gemm_simt(pb, st, stream);
}

int check_operands(int in_dtype, int out_dtype, const void* lhs, const void* rhs, void* out,
                   float scale_lhs, float scale_rhs, uint32_t epilogue) {
  if (!in_out_pair_ok(in_dtype, out_dtype))
    return fail(HODU_B200_ERR_INVALID_KERNEL, "matmul: unsupported dtype pair %s -> %s", dtype_name(in_dtype), dtype_name(out_dtype));
  if (epilogue != HODU_B200_EPI_NONE) return fail(HODU_B200_ERR_INVALID_KERNEL, "unknown epilogue %u", epilogue);
  if (is_int_dtype(in_dtype) && (scale_lhs != 1.0f || scale_rhs != 1.0f))
    return fail(HODU_B200_ERR_INVALID_INPUT, "integer matmul takes no scales");
  if (!lhs || !rhs || !out) return fail(HODU_B200_ERR_INVALID_INPUT, "null operand pointer");
  return 0;
}

namespace {
int matmul_impl(bool is_dot, int device, void* stream, int in_dtype, int out_dtype, const void* lhs,
                const void* rhs, void* out, const size_t* md, size_t len, float sl, float sr,
                uint32_t epilogue) {
  Problem pb;
  int r = is_dot ? parse_dot(md, len, &pb) : parse_matmul(md, len, &pb);
  if (r) return r;
  const bool empty = pb.M == 0 || pb.N == 0 || pb.batches == 0;
  if (!in_out_pair_ok(in_dtype, out_dtype))
    return fail(HODU_B200_ERR_INVALID_KERNEL, "matmul: unsupported dtype pair %s -> %s", dtype_name(in_dtype), dtype_name(out_dtype));
  if (empty) return 0;
  r = check_operands(in_dtype, out_dtype, pb.K == 0 ? out : lhs, pb.K == 0 ? out : rhs, out, sl, sr, epilogue);
  if (r) return r;
  DeviceState* st = device_state(device);
  if (!st) return HODU_B200_ERR_NOT_INITIALISED;
  DeviceGuard guard(device);
  if (!guard.ok) return fail(HODU_B200_ERR_LAUNCH, "cannot select CUDA device %d", device);
  pb.in_dtype = in_dtype; pb.out_dtype = out_dtype;
  pb.a.ptr = lhs; pb.b.ptr = rhs; pb.out = out;
  pb.alpha = sl * sr;
  return run_problem(pb, st, static_cast<cudaStream_t>(stream));
}

}  // namespace
}  // namespace hodu_b200

using namespace hodu_b200;

extern "C" {

int hodu_b200_init(int device) { return device_state(device) ? 0 : HODU_B200_ERR_NOT_INITIALISED; }

void hodu_b200_shutdown(int device) {
  if (device < 0 || device >= kMaxDevices) return;
  std::lock_guard<std::mutex> lock(g_state_mu);
  DeviceState* st = &g_state[device];
  if (!g_state_ready[device].load(std::memory_order_relaxed)) return;
  g_state_ready[device].store(false, std::memory_order_release);
  DeviceGuard guard(device);
  if (guard.ok) {
    cudaDeviceSynchronize();
    release_host_pipeline(device);
    cudaFree(st->status);
    if (st->pool) cudaMemPoolDestroy(st->pool);
  }
  *st = DeviceState();
}

int hodu_b200_matmul(int device, void* stream, uint8_t dtype, const void* lhs, const void* rhs,
                     void* out, const size_t* md, size_t len) {
  return matmul_impl(false, device, stream, dtype, dtype, lhs, rhs, out, md, len, 1.0f, 1.0f, 0);
}
int hodu_b200_dot(int device, void* stream, uint8_t dtype, const void* lhs, const void* rhs,
                  void* out, const size_t* md, size_t len) {
  return matmul_impl(true, device, stream, dtype, dtype, lhs, rhs, out, md, len, 1.0f, 1.0f, 0);
}
int hodu_b200_matmul_ex(int device, void* stream, uint8_t in_dtype, uint8_t out_dtype,
                        const void* lhs, const void* rhs, void* out, const size_t* md, size_t len,
                        float sl, float sr, uint32_t epilogue) {
  return matmul_impl(false, device, stream, in_dtype, out_dtype, lhs, rhs, out, md, len, sl, sr, epilogue);
}
int hodu_b200_dot_ex(int device, void* stream, uint8_t in_dtype, uint8_t out_dtype, const void* lhs,
                     const void* rhs, void* out, const size_t* md, size_t len, float sl, float sr,
                     uint32_t epilogue) {
  return matmul_impl(true, device, stream, in_dtype, out_dtype, lhs, rhs, out, md, len, sl, sr, epilogue);
}

int hodu_b200_cast(int device, void* stream, uint8_t src, uint8_t dst, const void* in, void* out,
                   const size_t* md, size_t len) {
  return launch_cast(src, dst, in, out, md, len, device, static_cast<cudaStream_t>(stream));
}

int hodu_b200_contiguous(int device, void* stream, uint8_t dtype, const void* in, void* out,
                         const size_t* md, size_t len) {
  if (dtype_size(dtype) == 0) return fail(HODU_B200_ERR_INVALID_KERNEL, "contiguous: unknown dtype %d", dtype);
  return launch_cast(dtype, dtype, in, out, md, len, device, static_cast<cudaStream_t>(stream));
}

int hodu_b200_swiglu(int device, void* stream, uint8_t dtype, const void* x, const void* w_gate,
                     const void* w_up, void* out, const size_t* md, size_t len, uint32_t flags) {
  if (!md || len != 12) return fail(HODU_B200_ERR_INVALID_INPUT, "swiglu: metadata length %zu, expected 12", len);
  if (dtype != HODU_DTYPE_BF16 && dtype != HODU_DTYPE_F16 && dtype != HODU_DTYPE_F32)
    return fail(HODU_B200_ERR_INVALID_KERNEL, "swiglu: unsupported dtype %s", dtype_name(dtype));
  if (flags != HODU_B200_SWIGLU_ROUND_EACH_OP && flags != HODU_B200_SWIGLU_ROUND_ONCE)
    return fail(HODU_B200_ERR_INVALID_INPUT, "swiglu: unknown flags %u", flags);
  Problem pb;
  pb.M = md[0]; pb.K = md[1]; pb.N = md[2];
  pb.a.stride_r = md[3]; pb.a.stride_c = md[4];
  pb.b.stride_r = md[5]; pb.b.stride_c = md[6];
  pb.b2.stride_r = md[7]; pb.b2.stride_c = md[8];
  pb.a.offset = md[9]; pb.b.offset = md[10]; pb.b2.offset = md[11];
  pb.batch_ndim = 0; pb.batches = 1;
  pb.swiglu = true;
  if (const int rc = check_extents(pb)) return rc;
  if (pb.M == 0 || pb.N == 0) return 0;
  if (!out) return fail(HODU_B200_ERR_INVALID_INPUT, "null operand pointer");
  DeviceState* st = device_state(device);
  if (!st) return HODU_B200_ERR_NOT_INITIALISED;
  DeviceGuard guard(device);
  if (!guard.ok) return fail(HODU_B200_ERR_LAUNCH, "cannot select CUDA device %d", device);
  pb.in_dtype = dtype; pb.out_dtype = dtype;
  pb.a.ptr = x; pb.b.ptr = w_gate; pb.b2.ptr = w_up; pb.out = out;
  pb.swiglu = true; pb.swiglu_flags = flags;
  if (pb.K == 0) return zero_output(pb, static_cast<cudaStream_t>(stream));  // silu(0)*0 == 0
  if (!x || !w_gate || !w_up) return fail(HODU_B200_ERR_INVALID_INPUT, "null operand pointer");
  return run_problem(pb, st, static_cast<cudaStream_t>(stream));
}

int hodu_b200_linear(int device, void* stream, uint8_t dtype, const void* x, const void* w,
                     const void* bias, void* out, const size_t* md, size_t len, uint32_t flags) {
  if (dtype != HODU_DTYPE_BF16 && dtype != HODU_DTYPE_F16 && dtype != HODU_DTYPE_F32)
    return fail(HODU_B200_ERR_INVALID_KERNEL, "linear: unsupported dtype %s", dtype_name(dtype));
  if (flags != HODU_B200_LINEAR_ROUND_EACH_OP && flags != HODU_B200_LINEAR_ROUND_ONCE)
    return fail(HODU_B200_ERR_INVALID_INPUT, "linear: unknown flags %u", flags);
  if (!md || len < 2) return fail(HODU_B200_ERR_INVALID_INPUT, "linear: metadata too short (%zu)", len);
  Problem pb;
  int r = parse_matmul(md, len - 2, &pb);
  if (r) return r;
  if (pb.M == 0 || pb.N == 0 || pb.batches == 0) return 0;
  if (!x || !w || !out) return fail(HODU_B200_ERR_INVALID_INPUT, "null operand pointer");
  DeviceState* st = device_state(device);
  if (!st) return HODU_B200_ERR_NOT_INITIALISED;
  DeviceGuard guard(device);
  if (!guard.ok) return fail(HODU_B200_ERR_LAUNCH, "cannot select CUDA device %d", device);
  pb.in_dtype = dtype; pb.out_dtype = dtype;
  pb.a.ptr = x; pb.b.ptr = w; pb.out = out;
  pb.bias = bias;
  if (md[len - 2] > kMaxSpan || md[len - 1] > kMaxSpan)
    return fail(HODU_B200_ERR_INVALID_INPUT, "linear: bias stride or offset out of range");
  pb.bias_stride = static_cast<int64_t>(md[len - 2]);
  pb.bias_offset = static_cast<int64_t>(md[len - 1]);
  pb.bias_flags = flags;
  if (pb.K == 0 && bias)
    return fail(HODU_B200_ERR_INVALID_INPUT, "linear: in_features == 0 with a bias is not supported");
  return run_problem(pb, st, static_cast<cudaStream_t>(stream));
}

int hodu_b200_einsum(int device, void* stream, uint8_t dtype, const void* const* inputs,
                     size_t num_inputs, void* out, const size_t* md, size_t len) {
  if (!in_out_pair_ok(dtype, dtype))
    return fail(HODU_B200_ERR_INVALID_KERNEL, "einsum: unsupported dtype %s", dtype_name(dtype));
  Problem pb;
  bool swapped = false;
  const int r = parse_einsum(md, len, num_inputs, &pb, &swapped);
  if (r) return r;
  if (pb.M == 0 || pb.N == 0 || pb.batches == 0) return 0;
  if (!inputs || !inputs[0] || !inputs[1] || !out) return fail(HODU_B200_ERR_INVALID_INPUT, "null operand pointer");
  DeviceState* st = device_state(device);
  if (!st) return HODU_B200_ERR_NOT_INITIALISED;
  DeviceGuard guard(device);
  if (!guard.ok) return fail(HODU_B200_ERR_LAUNCH, "cannot select CUDA device %d", device);
  pb.in_dtype = dtype; pb.out_dtype = dtype;
  pb.a.ptr = inputs[swapped ? 1 : 0];
  pb.b.ptr = inputs[swapped ? 0 : 1];
  pb.out = out;
  return run_problem(pb, st, static_cast<cudaStream_t>(stream));
}

int hodu_b200_conv2d(int device, void* stream, uint8_t dtype, const void* input, const void* weight,
                     void* out, const size_t* md, size_t len) {
  if (dtype != HODU_DTYPE_BF16 && dtype != HODU_DTYPE_F16 && dtype != HODU_DTYPE_F32)
    return fail(HODU_B200_ERR_INVALID_KERNEL, "conv2d: unsupported dtype %s", dtype_name(dtype));
  if (!md || len != 18) return fail(HODU_B200_ERR_INVALID_INPUT, "conv2d: metadata length %zu, expected 18", len);
  const size_t B = md[1], cin = md[2], cout = md[3], H = md[4], W = md[5], KH = md[6], KW = md[7];
  const size_t OH = md[8], OW = md[9], sh = md[10], sw = md[11], ph = md[12], pw = md[13], dh = md[14], dw = md[15];
  if (sh == 0 || sw == 0 || dh == 0 || dw == 0 || KH == 0 || KW == 0)
    return fail(HODU_B200_ERR_INVALID_INPUT, "conv2d: zero stride, dilation or kernel extent");
  const size_t span_h = dh * (KH - 1) + 1, span_w = dw * (KW - 1) + 1;
  if (H + 2 * ph < span_h || W + 2 * pw < span_w)
    return fail(HODU_B200_ERR_INVALID_INPUT, "conv2d: kernel larger than the padded input");
  if (OH != (H + 2 * ph - span_h) / sh + 1 || OW != (W + 2 * pw - span_w) / sw + 1)
    return fail(HODU_B200_ERR_INVALID_INPUT, "conv2d: output extent %zux%zu disagrees with input, kernel, stride, padding and dilation", OH, OW);
  if (md[0] != B * cout * OH * OW)
    return fail(HODU_B200_ERR_INVALID_INPUT, "conv2d: num_els %zu != batch*out_channels*out_h*out_w", md[0]);
  if (md[0] == 0) return 0;
  if (cin == 0) return fail(HODU_B200_ERR_INVALID_INPUT, "conv2d: in_channels == 0");
  if (!input || !weight || !out) return fail(HODU_B200_ERR_INVALID_INPUT, "null operand pointer");
  DeviceState* st = device_state(device);
  if (!st) return HODU_B200_ERR_NOT_INITIALISED;
  DeviceGuard guard(device);
  if (!guard.ok) return fail(HODU_B200_ERR_LAUNCH, "cannot select CUDA device %d", device);
  return run_conv2d(dtype, input, weight, out, md, len, st, static_cast<cudaStream_t>(stream));
}

const char* hodu_b200_strerror(int code) {
  switch (code) {
    case HODU_B200_OK: return "ok";
    case HODU_B200_ERR_INVALID_KERNEL: return "invalid kernel";
    case HODU_B200_ERR_INVALID_INPUT: return "invalid input";
    case HODU_B200_ERR_LAUNCH: return "launch error";
    case HODU_B200_ERR_MEMORY: return "memory error";
    case HODU_B200_ERR_DEVICE_STATUS: return "device status: a bounded wait ran out";
    case HODU_B200_ERR_NOT_INITIALISED: return "device not initialised";
    default: return "unknown error";
  }
}
const char* hodu_b200_last_error_message(void) { return g_msg; }

int hodu_b200_last_status(int device, uint32_t* word) {
  DeviceState* st = device_state(device);
  if (!st) return HODU_B200_ERR_NOT_INITIALISED;
  DeviceGuard guard(device);
  if (!guard.ok) return fail(HODU_B200_ERR_LAUNCH, "cannot select CUDA device %d", device);
  HODU_CUDA_TRY(cudaDeviceSynchronize(), HODU_B200_ERR_LAUNCH);
  uint32_t w = 0;
  HODU_CUDA_TRY(cudaMemcpy(&w, st->status, sizeof(w), cudaMemcpyDeviceToHost), HODU_B200_ERR_MEMORY);
  if (w != 0) HODU_CUDA_TRY(cudaMemset(st->status, 0, sizeof(w)), HODU_B200_ERR_MEMORY);
  if (word) *word = w;
  if (w != 0) return fail(HODU_B200_ERR_DEVICE_STATUS, "device status word 0x%08x (cta %u, wait %u)", w, (w >> 4) & 0xFFFFu, w & 0xFu);
  return 0;
}

int hodu_b200_debug_wait_timeout(int device, void* stream, uint32_t limit_ms) {
  if (limit_ms == 0 || limit_ms > 2000) return fail(HODU_B200_ERR_INVALID_INPUT, "limit_ms must be 1..2000");
  DeviceState* st = device_state(device);
  if (!st) return HODU_B200_ERR_NOT_INITIALISED;
  DeviceGuard guard(device);
  if (!guard.ok) return fail(HODU_B200_ERR_LAUNCH, "cannot select CUDA device %d", device);
  return launch_wait_timeout_probe(st, static_cast<cudaStream_t>(stream), limit_ms);
}

int hodu_b200_force_path(int path) {
  if (path < HODU_B200_PATH_AUTO || path > HODU_B200_PATH_TENSOR_2CTA_512) return HODU_B200_ERR_INVALID_INPUT;
  return g_forced_path.exchange(path);
}
int hodu_b200_last_path(void) { return g_last_path; }
uint64_t hodu_b200_launch_count(void) { return g_launches.load(); }
int hodu_b200_version(void) { return 100; }

}  // extern "C"

