/*
 * hodu_b200.h -- C ABI of the B200 (sm_100a) matmul / dot / cast path for Hodu.
 *
 * This library stands where the reference's `hodu_cuda_kernels` crate stands for
 * three of its entry points.  Every function below names the reference interface
 * it replaces (paths are relative to the reference project root).
 *
 * Conventions shared by all entry points
 *  - Return value: 0 on success, otherwise one of the negative HODU_B200_ERR_*
 *    codes.  Nothing aborts or throws.  The codes mirror the variants of the
 *    reference's `CudaKernelError` (crates/hodu_cuda_kernels/src/error.rs:7-18).
 *  - `device` is the CUDA ordinal of `Device::CUDA(n)`
 *    (crates/hodu_core/src/types/device.rs:4-11).
 *  - `stream` is a `CUstream`/`cudaStream_t` passed as `void*`; NULL means the
 *    context's default stream, which is what the reference launches on
 *    (crates/hodu_cuda_kernels/src/kernels/ops_matrix.rs:572-582).  Work is only
 *    enqueued: the call returns before the kernel has finished, as in the
 *    reference.  No implicit synchronisation.
 *  - dtypes are the `#[repr(u8)]` discriminants of `DType`
 *    (crates/hodu_core/src/types/dtype.rs:6-30).
 *  - `metadata` is a HOST array of `size_t` in the wire format built by
 *    `crates/hodu_core/src/op_metadatas.rs`; strides and offsets are in elements.
 *    It is read during the call only (no device copy of it is made).
 *  - The caller owns every buffer.  Inputs may alias each other; `out` must not
 *    alias an input.  `out` is contiguous, offset 0, and may be uninitialised.
 *  - Thread-safe: any thread may call for any device.
 *  - There is no CPU fallback and no cuBLAS: an unsupported dtype or layout is an
 *    error code.
 */
#ifndef HODU_B200_H
#define HODU_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* DType discriminants (crates/hodu_core/src/types/dtype.rs:6-30). */
enum {
  HODU_DTYPE_BOOL = 0,
  HODU_DTYPE_F8E4M3 = 1,
  HODU_DTYPE_F8E5M2 = 2,
  HODU_DTYPE_BF16 = 3,
  HODU_DTYPE_F16 = 4,
  HODU_DTYPE_F32 = 5,
  HODU_DTYPE_F64 = 6,
  HODU_DTYPE_U8 = 7,
  HODU_DTYPE_U16 = 8,
  HODU_DTYPE_U32 = 9,
  HODU_DTYPE_U64 = 10,
  HODU_DTYPE_I8 = 11,
  HODU_DTYPE_I16 = 12,
  HODU_DTYPE_I32 = 13,
  HODU_DTYPE_I64 = 14
};

/* Error codes; one per CudaKernelError variant plus a device-status code. */
enum {
  HODU_B200_OK = 0,
  HODU_B200_ERR_INVALID_KERNEL = -1, /* unsupported dtype pair / op          */
  HODU_B200_ERR_INVALID_INPUT = -2,  /* bad metadata, null pointer, layout   */
  HODU_B200_ERR_LAUNCH = -3,         /* CUDA launch failed                   */
  HODU_B200_ERR_MEMORY = -4,         /* allocation or copy failed            */
  HODU_B200_ERR_DEVICE_STATUS = -5,  /* a kernel reported a bounded wait ran out */
  HODU_B200_ERR_NOT_INITIALISED = -6
};

/* Epilogue selector of the *_ex entry points. */
enum {
  HODU_B200_EPI_NONE = 0
};

/* Path selector for hodu_b200_force_path (testing aid). */
enum {
  HODU_B200_PATH_AUTO = 0,
  HODU_B200_PATH_SIMT = 1,   /* generic strided CUDA-core kernel          */
  HODU_B200_PATH_TENSOR = 2, /* tcgen05 kernel; error if layout unfit     */
  HODU_B200_PATH_TENSOR_1CTA = 3, /* tcgen05, one CTA per tile, whatever the size  */
  HODU_B200_PATH_TENSOR_2CTA = 4, /* tcgen05, CTA pair per 256x256 tile, whatever the size */
  HODU_B200_PATH_TENSOR_2CTA_512 = 5 /* tcgen05, CTA pair per 512x256 tile, whatever the size */
};

/* Flags of hodu_b200_swiglu. */
enum {
  /* Round gate/up projections, silu and product to the storage dtype one by one,
   * as the reference's op-by-op composition does
   * (Linear::forward -> Tensor::silu -> Tensor::mul, each producing a tensor). */
  HODU_B200_SWIGLU_ROUND_EACH_OP = 0,
  /* Keep gate/up/silu in f32 and round the product once. */
  HODU_B200_SWIGLU_ROUND_ONCE = 1
};

/* Flags of hodu_b200_linear. */
enum {
  /* Round the product to the storage dtype, then add the bias and round again: what the
   * reference's two ops (`matmul`, then `add`) produce. */
  HODU_B200_LINEAR_ROUND_EACH_OP = 0,
  /* Add the bias to the f32 accumulator and round once. */
  HODU_B200_LINEAR_ROUND_ONCE = 1
};

/*
 * Per-device set-up: creates the status word and caches device properties.
 * Replaces the lazily built per-device state of the reference
 * (`Kernels::new`, crates/hodu_cuda_kernels/src/kernel.rs:102-126, and the
 * context pool in crates/hodu_core/src/be_cuda/device.rs:20-65).
 * Called implicitly by the first compute call on a device.
 */
int hodu_b200_init(int device);
void hodu_b200_shutdown(int device);

/*
 * Batched matmul with broadcasting, output dtype == input dtype.
 * Replaces `call_ops_matmul`
 * (crates/hodu_cuda_kernels/src/kernels/ops_matrix.rs:415-429) and the kernels
 * `hodu_cuda_matmul_{dtype}` (crates/hodu_cuda_kernels/kernels/ops_matrix.cu:9-102).
 * metadata = [num_els, lhs_ndim, rhs_ndim, batch_ndim, lhs_shape.., rhs_shape..,
 *             batch_shape.., lhs_strides.., rhs_strides.., lhs_off, rhs_off, M, K, N]
 * (crates/hodu_core/src/op_metadatas.rs:192-290).
 * dtypes: f8e4m3, bf16, f16, f32, i8 (i8 keeps the reference CPU semantics: the
 * exact sum wrapped to 8 bits), i32.
 */
int hodu_b200_matmul(int device, void* stream, uint8_t dtype,
                     const void* lhs, const void* rhs, void* out,
                     const size_t* metadata, size_t metadata_len);

/*
 * 2-D matmul.  Replaces `call_ops_dot`
 * (crates/hodu_cuda_kernels/src/kernels/ops_matrix.rs:611-625) and
 * `hodu_cuda_dot_{dtype}` (crates/hodu_cuda_kernels/kernels/ops_matrix.cu:104-165).
 * metadata = [M, K, N, lhs_stride_m, lhs_stride_k, rhs_stride_k, rhs_stride_n,
 *             lhs_off, rhs_off]  (crates/hodu_core/src/op_metadatas.rs:464-506).
 */
int hodu_b200_dot(int device, void* stream, uint8_t dtype,
                  const void* lhs, const void* rhs, void* out,
                  const size_t* metadata, size_t metadata_len);

/*
 * Mixed-dtype forms of the two calls above.  The reference has no such op: its
 * CUDA dispatch fixes output dtype == input dtype and rejects f8e4m3 / i8
 * (crates/hodu_core/src/be_cuda/storage/ops_matrix.rs:66-92,142-167).  These carry
 * what that signature cannot: out = cast_out(scale_lhs * scale_rhs * (lhs . rhs)).
 * Supported (in -> out): f8e4m3 -> bf16 | f16 | f32 | f8e4m3;  i8 -> i32 | i8;
 * bf16 -> bf16 | f32;  f16 -> f16 | f32;  f32 -> f32;  i32 -> i32.
 * Scales apply to floating inputs only and must be 1 for integer inputs.
 * Float outputs are rounded to nearest even; f8e4m3 output saturates to +-448.
 */
int hodu_b200_matmul_ex(int device, void* stream, uint8_t in_dtype, uint8_t out_dtype,
                        const void* lhs, const void* rhs, void* out,
                        const size_t* metadata, size_t metadata_len,
                        float scale_lhs, float scale_rhs, uint32_t epilogue);
int hodu_b200_dot_ex(int device, void* stream, uint8_t in_dtype, uint8_t out_dtype,
                     const void* lhs, const void* rhs, void* out,
                     const size_t* metadata, size_t metadata_len,
                     float scale_lhs, float scale_rhs, uint32_t epilogue);

/*
 * Element-wise dtype conversion.  Replaces `call_ops_cast`
 * (crates/hodu_cuda_kernels/src/kernels/ops_cast.rs:27-64) and
 * `hodu_cuda_cast_{src}_to_{dst}` (crates/hodu_cuda_kernels/kernels/ops_cast.cu:7-30)
 * for f32 <-> bf16 | f16 | f8e4m3, i8 -> i32, and the pairs hodu_core wires for CUDA today:
 * f32 <-> f64, f32 <-> i32 (crates/hodu_core/src/be_cuda/storage.rs:652-673), plus f32 <-> u32,
 * the remaining pair of the reference's cast tests (crates/hodu_cuda_kernels/tests/ops_cast.rs:48-89).
 * metadata = [num_els, ndim, shape.., strides.., offset]
 * (crates/hodu_core/src/op_metadatas.rs:1615-1640).
 */
int hodu_b200_cast(int device, void* stream, uint8_t src_dtype, uint8_t dst_dtype,
                   const void* in, void* out,
                   const size_t* metadata, size_t metadata_len);

/*
 * Strided -> contiguous copy of any dtype.  Replaces `call_ops_contiguous` and
 * `hodu_cuda_contiguous_{dtype}` (crates/hodu_cuda_kernels/kernels/ops_memory.cu:6-27; call
 * site crates/hodu_core/src/be_cuda/storage.rs:681-709).  metadata as for hodu_b200_cast.
 */
int hodu_b200_contiguous(int device, void* stream, uint8_t dtype, const void* in, void* out,
                         const size_t* metadata, size_t metadata_len);

/*
 * Fused gate/up half of a SwiGLU MLP:  out[M,N] = silu(x . w_gate) * (x . w_up).
 * In the reference this is three launches and two [M,N] temporaries:
 * `Linear::forward` twice (crates/hodu_nn/src/modules/linear.rs:38-47), `silu`
 * (crates/hodu_cuda_kernels/kernels/ops_unary.cu:178, math.cuh:232-235) and `mul`
 * (crates/hodu_cuda_kernels/kernels/ops_binary.cu).
 * metadata = [M, K, N, x_stride_m, x_stride_k, wg_stride_k, wg_stride_n,
 *             wu_stride_k, wu_stride_n, x_off, wg_off, wu_off]
 * i.e. the dot wire format with a second right-hand operand.  dtype: bf16 | f16.
 * `flags`: HODU_B200_SWIGLU_ROUND_EACH_OP or HODU_B200_SWIGLU_ROUND_ONCE.
 */
int hodu_b200_swiglu(int device, void* stream, uint8_t dtype,
                     const void* x, const void* w_gate, const void* w_up, void* out,
                     const size_t* metadata, size_t metadata_len, uint32_t flags);

/*
 * Linear layer with its bias fused into the product's epilogue:
 *   out[..., N] = x[..., K] . w[K, N] + bias[N]
 * In the reference `Linear::forward` (crates/hodu_nn/src/modules/linear.rs:38-47) is
 * `input.matmul(weight.transpose(-2,-1))` followed by `output.add(bias)`, a separate broadcast
 * kernel over the whole output (crates/hodu_cuda_kernels/kernels/ops_binary.cu).
 * metadata = the matmul wire format of hodu_b200_matmul (any batch dims on x; `w` is normally the
 * 2-D transposed view of the [N,K] weight, strides (1,K)) followed by two more words:
 * [bias_stride, bias_offset] in elements.  `bias` has the dtype of the output and may be null
 * (no bias: same as hodu_b200_matmul).  dtype: bf16 | f16 | f32.
 * `flags`: HODU_B200_LINEAR_ROUND_EACH_OP or HODU_B200_LINEAR_ROUND_ONCE.
 */
int hodu_b200_linear(int device, void* stream, uint8_t dtype,
                     const void* x, const void* w, const void* bias, void* out,
                     const size_t* metadata, size_t metadata_len, uint32_t flags);

/*
 * Two-operand einsum contractions routed to the GEMM.  Replaces, for the forms below,
 * `call_ops_einsum` (crates/hodu_cuda_kernels/src/kernels/ops_einsum.rs:24-70) and its
 * one-thread-per-output kernel (crates/hodu_cuda_kernels/kernels/ops_einsum.cu:76-...).
 * metadata = the reference's einsum wire format (`einsum_metadata`,
 * crates/hodu_core/src/op_metadatas.rs:1502-1567; restated in crates/hodu_cpu_kernels/tests/ops_einsum.rs:18-84):
 *   [num_output_els, num_inputs, num_total_indices, num_contraction_indices, output_ndim,
 *    output_shape.., then per input: ndim, shape.., strides.., offset, dim_to_index_id..,
 *    contraction_index_ids.., index_sizes.., output_index_ids..]
 * Accepted: num_inputs == 2, no index repeated within one operand, and every index of exactly
 * one of four kinds -- batch (in both operands and the output), M (first operand and output),
 * N (second operand and output), K (both operands, not the output) -- with the output ordered
 * [batch.., M.., N..] or [batch.., N.., M..] (the operands are then swapped) and the indices
 * of a kind mergeable into one stride in each operand.  That covers "ij,jk->ik", "bij,bjk->bik",
 * "ik,jk->ij", "bhqd,bhkd->bhqk", "i,i->", "i,j->ij" and the like.  Anything else
 * (trace, transposition, sums over one operand) returns HODU_B200_ERR_INVALID_KERNEL so the
 * caller keeps its own kernel for it.  `inputs` is an array of `num_inputs` device pointers.
 */
int hodu_b200_einsum(int device, void* stream, uint8_t dtype, const void* const* inputs,
                     size_t num_inputs, void* out, const size_t* metadata, size_t metadata_len);

/*
 * conv2d (NCHW input, [Cout,Cin,KH,KW] weight, NCHW output) as im2col + one batched product on
 * the same GEMM kernels.  Replaces `call_ops_conv` with `hodu_cuda_conv2d_{dtype}`
 * (crates/hodu_cuda_kernels/src/kernels/ops_conv.rs; direct kernel
 * crates/hodu_cuda_kernels/kernels/ops_conv.cu:45-93), in the form the reference's CPU OpenBLAS
 * build uses (crates/hodu_cpu_kernels/kernels/ops_conv_openblas.c:84-133).
 * metadata = `conv2d_metadata` (crates/hodu_core/src/op_metadatas.rs:1076-1123), 18 words:
 *   [num_els, batch, in_channels, out_channels, in_h, in_w, kernel_h, kernel_w, out_h, out_w,
 *    stride_h, stride_w, padding_h, padding_w, dilation_h, dilation_w, input_offset, weight_offset]
 * Input and weight are contiguous from their offsets.  dtype: bf16 | f16 | f32; f32 accumulate,
 * one rounding.  The unfolded input lives in stream-ordered scratch for the duration of the call
 * (at most 2 GiB at a time; larger batches run in several passes); a 1x1 kernel with unit stride
 * and no padding needs none.
 */
int hodu_b200_conv2d(int device, void* stream, uint8_t dtype, const void* input, const void* weight,
                     void* out, const size_t* metadata, size_t metadata_len);

/*
 * Host-buffer forms: the whole of "create tensors on the device, multiply, read
 * the result back", i.e. `BackendDevice` upload (crates/hodu_core/src/be/device.rs:35-55),
 * `call_ops_matmul` / `call_ops_dot`, then `to_cpu_storage`
 * (crates/hodu_core/src/be_cuda/storage.rs:165-173), as one pipelined call.
 * lhs/rhs/out are HOST pointers (pinned memory gives full copy speed); metadata
 * describes the host operands exactly as in the device forms.  The call copies
 * operands to device staging memory in slices, runs the same kernels as the
 * device forms, copies results back, and returns after the output is complete.
 * Only contiguous operands with offset 0 are accepted (what a freshly created
 * tensor has).  Staging memory is allocated on first use and kept per device.
 */
int hodu_b200_matmul_host(int device, uint8_t in_dtype, uint8_t out_dtype,
                          const void* lhs_host, const void* rhs_host, void* out_host,
                          const size_t* metadata, size_t metadata_len,
                          float scale_lhs, float scale_rhs);
int hodu_b200_dot_host(int device, uint8_t in_dtype, uint8_t out_dtype,
                       const void* lhs_host, const void* rhs_host, void* out_host,
                       const size_t* metadata, size_t metadata_len,
                       float scale_lhs, float scale_rhs);

/*
 * SwiGLU MLP forward over HOST activations with DEVICE-resident weights:
 *   y_host[tokens, d_out] = (silu(x . W_gate) * (x . W_up)) . W_down
 * i.e. "tensor from host data -> three `Linear::forward` calls, silu, mul
 * (crates/hodu_nn/src/modules/linear.rs:38-47) -> to_cpu_storage" as one pipelined call: tokens
 * travel in row blocks whose upload, two products and download overlap; the hidden activations
 * never leave the device.  x_host and y_host are contiguous host arrays (pinned memory gives full
 * copy speed); w_gate, w_up, w_down are device pointers to the layers' weights.
 * metadata (13 words) = [tokens, d_in, d_hidden, d_out,
 *                        wg_stride_k, wg_stride_n, wu_stride_k, wu_stride_n, wd_stride_k, wd_stride_n,
 *                        wg_off, wu_off, wd_off]   (strides and offsets in elements; a `Linear`
 * weight stored [out, in] is passed as its transposed view: stride_k = 1, stride_n = in).
 * dtype: bf16 | f16.  flags as hodu_b200_swiglu.  Returns after y_host is complete.
 */
int hodu_b200_swiglu_mlp_host(int device, uint8_t dtype, const void* x_host, const void* w_gate,
                              const void* w_up, const void* w_down, void* y_host,
                              const size_t* metadata, size_t metadata_len, uint32_t flags);

/*
 * 2-D f32 product that allocates NOTHING.  It has no counterpart in the reference (whose
 * wrappers allocate on every call: the metadata copy in
 * crates/hodu_cuda_kernels/src/kernels/ops_matrix.rs:572-582).
 *
 * Who needs it: code that may not reach the device allocator while it runs -- a real-time
 * loop that must not take the allocator's lock or risk the implicit device synchronisation an
 * allocation can bring, a process that runs inside a fixed memory reservation where a late
 * allocation can fail, a plug-in called from a host that forbids allocation in its compute
 * callbacks.  hodu_b200_dot computes
 * an f32 product through split TF32 operands that it keeps in scratch memory taken from the
 * stream-ordered allocator; this entry point runs the same kernels with that scratch in a
 * fixed array compiled into the library instead.  It calls no cudaMalloc / cudaFree /
 * cudaMallocAsync and does not touch the library's per-device state (hodu_b200_init is not
 * needed and is not called).
 *
 *  - metadata: the dot wire format, as hodu_b200_dot; any strides and offsets.
 *  - Limit: the split operands take 12*(M+N)*K bytes (rows padded to 16 bytes) and must fit
 *    HODU_B200_STATIC_SCRATCH_BYTES; larger products are rejected with
 *    HODU_B200_ERR_INVALID_INPUT and a message naming both sizes.  Every GPU that loads the
 *    library holds the array (that many bytes) from load to exit, used or not.
 *  - The first call on a device resolves the array's device address (cudaGetSymbolAddress,
 *    with that device current) and sets kernel attributes.  Make that first call before any
 *    stream capture begins.
 *  - All calls on a device share the one array, and it keeps the previous call's contents.
 *    Nothing in it has to start at zero: each call overwrites every element it later reads.
 *    Two calls whose kernels can overlap on the GPU (different streams without an ordering
 *    between them) race on it; order them.
 *  - A bounded wait that runs out is recorded in a device word private to this entry point,
 *    not in the word hodu_b200_last_status reads; hodu_b200_dot_f32_static_status reads it.
 */
#define HODU_B200_STATIC_SCRATCH_BYTES (32u << 20)
int hodu_b200_dot_f32_static(int device, void* stream, const void* lhs, const void* rhs, void* out,
                             const size_t* metadata, size_t metadata_len);
/*
 * Synchronises `device`, then reads (and clears) the status word of hodu_b200_dot_f32_static.
 * Zero: every kernel that entry point launched finished its waits.  Non-zero: a bounded wait
 * gave up and the output of that call is incomplete; the function then returns
 * HODU_B200_ERR_DEVICE_STATUS.  Like the entry point it belongs to, it allocates nothing and
 * needs no hodu_b200_init.  No counterpart in the reference.
 */
int hodu_b200_dot_f32_static_status(int device, uint32_t* device_status_word);

/* Text for an error code (static storage).  Mirrors `Display for CudaKernelError`
 * (crates/hodu_cuda_kernels/src/error.rs:20-32). */
const char* hodu_b200_strerror(int code);
/* Longer message for the last failing call on the calling thread (thread-local). */
const char* hodu_b200_last_error_message(void);

/*
 * Reads (and clears) the device status word of `device` after synchronising the
 * device.  Zero means every kernel finished its waits; non-zero encodes which
 * bounded wait gave up.  Returns HODU_B200_ERR_DEVICE_STATUS if the word was
 * non-zero.  The reference has no counterpart: its kernels have no waits.
 */
int hodu_b200_last_status(int device, uint32_t* device_status_word);

/* Testing aids (no reference counterpart). */
int hodu_b200_force_path(int path);      /* process-wide; returns previous value  */
int hodu_b200_last_path(void);           /* path taken by the last matmul/dot/swiglu
                                            call on the calling thread            */
/* Launches one tiny kernel whose only wait can never be satisfied and whose limit is
 * `limit_ms` (1..2000): the wait gives up, the kernel records a code in the status word
 * and returns normally.  hodu_b200_last_status then reports it.  Exercises the
 * bounded-wait mechanism of the GEMM kernels without faulting or hanging anything. */
int hodu_b200_debug_wait_timeout(int device, void* stream, uint32_t limit_ms);
uint64_t hodu_b200_launch_count(void);   /* kernels launched by this library so far */
int hodu_b200_version(void);

#ifdef __cplusplus
}
#endif
#endif /* HODU_B200_H */
