// Shared host/device declarations of libhodu_b200: dtype table, per-device state,
// error reporting, and the internal launch interfaces of the kernel families.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stddef.h>
#include <stdint.h>

#include "../../include/hodu_b200.h"

namespace hodu_b200 {

constexpr int kMaxDevices = 16;   // Device::CUDA ids 0..15 (hodu_core tensor/creation.rs:33-37)
constexpr int kMaxBatchDims = 3;  // collapsed batch dims a tensor-core launch can address

// ------------------------------------------------------------------ dtypes
__host__ __device__ inline int dtype_size(int dt) {
  switch (dt) {
    case HODU_DTYPE_F8E4M3: case HODU_DTYPE_I8: case HODU_DTYPE_U8: case HODU_DTYPE_BOOL:
    case HODU_DTYPE_F8E5M2: return 1;
    case HODU_DTYPE_BF16: case HODU_DTYPE_F16: case HODU_DTYPE_I16: case HODU_DTYPE_U16: return 2;
    case HODU_DTYPE_F32: case HODU_DTYPE_I32: case HODU_DTYPE_U32: return 4;
    case HODU_DTYPE_F64: case HODU_DTYPE_I64: case HODU_DTYPE_U64: return 8;
    default: return 0;
  }
}
const char* dtype_name(int dt);

// ------------------------------------------------------------------ errors
// Records a formatted message for hodu_b200_last_error_message() and returns `code`.
int fail(int code, const char* fmt, ...);

#define HODU_CUDA_TRY(expr, code)                                                       \
  do {                                                                                  \
    cudaError_t _e = (expr);                                                            \
    if (_e != cudaSuccess)                                                              \
      return ::hodu_b200::fail((code), "%s failed: %s", #expr, cudaGetErrorString(_e)); \
  } while (0)

// ------------------------------------------------------------------ device state
struct DeviceState {
  bool ready = false;
  int sm_count = 0;
  int cc_major = 0, cc_minor = 0;
  size_t smem_optin = 0;
  uint32_t* status = nullptr;  // one device word: first bounded wait that gave up
  int device = -1;
  cudaMemPool_t pool = nullptr;  // scratch pool of this library (created on first use)
};
// Stream-ordered scratch from a memory pool that belongs to this library (the caller's default
// pool is left alone).  The pool keeps what it has handed out for reuse until
// hodu_b200_shutdown, so repeated calls do not go back to the driver for memory.
int scratch_alloc(DeviceState* st, void** ptr, size_t bytes, cudaStream_t stream);
int scratch_free(void* ptr, cudaStream_t stream);
// Returns the state for `device`, initialising it on first use (thread-safe);
// nullptr + recorded error on failure.
DeviceState* device_state(int device);
// Makes `device` current for the scope, restoring the previous device after.
struct DeviceGuard {
  int prev = -1;
  bool ok = false;
  explicit DeviceGuard(int device);
  ~DeviceGuard();
};

// cuTensorMapEncodeTiled, fetched from the driver once (null if the driver has none).
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn tensor_map_encoder();
// HODU_B200_DEBUG=1 (see gemm_tc.cu).
bool debug_enabled();
// Whether kernels are launched with programmatic stream serialisation (HODU_B200_PDL=0: no).
bool dependent_launch_enabled();

void count_launch(unsigned n = 1);
void set_last_path(int path);
int forced_path();

// ------------------------------------------------------------------ problem description
// One matrix operand of a (batched) product, strides in elements.
struct Operand {
  const void* ptr = nullptr;  // base pointer WITHOUT the offset applied
  int64_t offset = 0;         // elements
  int64_t stride_r = 0;       // stride of the row index    (M for lhs, K for rhs)
  int64_t stride_c = 0;       // stride of the column index (K for lhs, N for rhs)
  int64_t bstride[16] = {0};  // stride per OUTPUT batch dim (0 where broadcast)
};
struct Problem {
  int in_dtype = 0, out_dtype = 0;
  int64_t M = 0, N = 0, K = 0;
  int batch_ndim = 0;
  int64_t batch_shape[16] = {0};
  int64_t batches = 1;
  Operand a, b;
  Operand b2;            // second right-hand operand (SwiGLU up projection)
  bool swiglu = false;
  uint32_t swiglu_flags = 0;
  void* out = nullptr;   // [batches, M, N]; rows `ldc` elements apart, batches M*ldc apart
  int64_t ldc = 0;       // 0: N (a contiguous output, what every entry point of the C ABI passes)
  float alpha = 1.0f;    // scale_lhs * scale_rhs
  // Bias of a Linear layer: [N] values of the OUTPUT dtype added to every output row
  // (hodu_nn/src/modules/linear.rs:38-47).  `bias_flags` says whether the product is rounded
  // to the output dtype before the addition (what the reference's two ops do) or only after.
  const void* bias = nullptr;
  int64_t bias_offset = 0, bias_stride = 1;
  uint32_t bias_flags = 0;
  bool no_scratch = false;    // the caller forbids stream-ordered scratch (hodu_b200_dot_f32_static)
  bool f32_presplit = false;  // f32 operands already in the three-segment TF32 split form (gemm_f32.cu)
};

// Generic strided CUDA-core kernel: any layout, every supported dtype pair.
int launch_gemm_simt(const Problem& pb, DeviceState* st, cudaStream_t stream);
// tcgen05 kernel. Returns 1 if the layout cannot be described to TMA (nothing
// launched, `why` says which rule failed), 0 when launched, <0 on error.
int launch_gemm_tc(const Problem& pb, DeviceState* st, cudaStream_t stream, const char** why);
// The same, with K cut into slices that run as one batched launch plus a reduction when the
// output alone cannot occupy the GPU (splitk.cu); otherwise exactly launch_gemm_tc.
int launch_gemm_tc_splitk(const Problem& pb, DeviceState* st, cudaStream_t stream, const char** why);
// K slices launch_gemm_tc would give `pb` inside ONE launch (clusters of CTAs sharing a tile); 1 = none.
int tc_planned_k_slices(const Problem& pb, DeviceState* st);
// Layout front door (relayout.cu): copies the operands TMA cannot describe into scratch as
// K-contiguous matrices, then runs the tensor-core kernel.  1 = nothing to fix / not applicable.
bool tc_operand_describable(const Problem& pb, const Operand& op, bool is_lhs, int esize);
int launch_gemm_tc_relayout(const Problem& pb, DeviceState* st, cudaStream_t stream, const char** why);
// f32 on the tensor cores through split TF32 operands held in scratch memory (gemm_f32.cu).
// Return convention as launch_gemm_tc.  `launch_gemm_f32` takes the scratch from the
// stream-ordered allocator; `launch_gemm_f32_split` uses the scratch it is given.
size_t gemm_f32_scratch_bytes(const Problem& pb);
int launch_gemm_f32(const Problem& pb, DeviceState* st, cudaStream_t stream, const char** why);
// One-kernel form for small f32 products (gemm_f32_fused.cu): raw f32 tiles arrive by TMA, are
// split into TF32 high and low parts in shared memory, multiplied on the tensor cores, and the K
// slices of a tile are added across a thread-block cluster.  No scratch memory, one launch.
// Return convention as launch_gemm_tc (1 = not applicable, nothing launched).
int launch_gemm_f32_fused(const Problem& pb, DeviceState* st, cudaStream_t stream, const char** why);
int launch_gemm_f32_split(const Problem& pb, DeviceState* st, cudaStream_t stream, void* scratch,
                          size_t scratch_bytes, const char** why);
// One tiny kernel whose only wait can never be satisfied; it gives up after limit_ms.
int launch_wait_timeout_probe(DeviceState* st, cudaStream_t stream, uint32_t limit_ms);
// Refuses problems whose extents, strides or offsets are beyond anything a real buffer can hold
// (extent > 2^32, stride or offset > 2^48, an operand that spans more than 2^48 elements, more
// than 2^48 output elements), so that the host arithmetic further down -- products of extents,
// strides times extents, byte sizes -- cannot overflow.  Every parser ends with it.
int check_extents(const Problem& pb);
// Parsers of the reference's wire formats and the path chooser (api.cu).
int parse_matmul(const size_t* md, size_t len, Problem* pb);
int parse_dot(const size_t* md, size_t len, Problem* pb);
// Two-operand einsum wire format -> matrix product over views (einsum.cu).  `swapped`: the
// second einsum operand is the product's left-hand side.
int parse_einsum(const size_t* md, size_t len, size_t num_inputs, Problem* pb, bool* swapped);
int check_operands(int in_dtype, int out_dtype, const void* lhs, const void* rhs, void* out,
                   float scale_lhs, float scale_rhs, uint32_t epilogue);
int run_problem(const Problem& pb, DeviceState* st, cudaStream_t stream);
// conv2d wire format (validated by the caller) -> im2col + one batched product (conv.cu).
int run_conv2d(int dtype, const void* input, const void* weight, void* out, const size_t* md, size_t len,
               DeviceState* st, cudaStream_t stream);
// The same convolution without the unfolded copy (conv_implicit.cu): 0 launched, 1 not a case
// that form takes (nothing launched), < 0 error.
int run_conv2d_implicit(int dtype, const void* input, const void* weight, void* out, const size_t* md, DeviceState* st,
                        cudaStream_t stream, const char** why);
// Frees the staging memory and streams of the host-buffer forms (host_pipeline.cu).
void release_host_pipeline(int device);
// Casts.
int launch_cast(int src, int dst, const void* in, void* out, const size_t* md, size_t md_len,
                int device, cudaStream_t stream);

}  // namespace hodu_b200
