// conv2d as im2col + GEMM.
//
// The reference's CUDA conv2d is a direct kernel, one thread per output element walking
// in_channels x kernel_h x kernel_w (crates/hodu_cuda_kernels/kernels/ops_conv.cu:45-93; f32
// running sum, one conversion); its CPU OpenBLAS build already does im2col + sgemm per image
// (crates/hodu_cpu_kernels/kernels/ops_conv_openblas.c:44-133).  Here the same split runs on the
// GPU: one HBM-bound kernel unfolds every image into col[b][K][N] (K = Cin*KH*KW rows,
// N = OH*OW columns, N contiguous, pitch padded to 16 bytes), then ONE batched product
//   out[b][Cout][N] = weight[Cout][K] . col[b][K][N]
// goes through the same kernels as every other matmul (weight broadcast over the batch, col as
// an N-contiguous right-hand operand), which writes the NCHW output directly.  A 1x1 kernel
// with unit stride and no padding needs no unfolding: the input already is col.
//
// Wire format (crates/hodu_core/src/op_metadatas.rs:1076-1123):
// [num_els, batch, in_channels, out_channels, in_h, in_w, kernel_h, kernel_w, out_h, out_w,
//  stride_h, stride_w, padding_h, padding_w, dilation_h, dilation_w, input_offset, weight_offset]
// Input [B, Cin, H, W] and weight [Cout, Cin, KH, KW] are contiguous from their offsets.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "common.cuh"

namespace hodu_b200 {
namespace {

struct Im2colParams {
  const void* in;   // first element of image 0
  void* col;
  int images, cin, h, w, kh, kw, oh, ow;
  int sh, sw, ph, pw, dh, dw;
  int K, N, npitch;            // col is [images][K][npitch]
};

// Block = 32 column vectors x 8 col rows; grid = (column chunks, row groups, images).  One thread
// writes VEC consecutive columns of one col row with a single 16-byte store.  All index
// arithmetic inside an image is 32-bit, and a warp shares its row, so the row's (ic, kh, kw)
// split costs one instruction stream per 32 vectors.
template <typename T, int VEC>
__global__ void __launch_bounds__(256) im2col_kernel(const Im2colParams p) {
  const int n0 = (blockIdx.x * 32 + threadIdx.x) * VEC;
  if (n0 >= p.npitch) return;
  const int oh0 = n0 / p.ow, ow0 = n0 - oh0 * p.ow;
  const bool one_row = p.sw == 1 && ow0 + VEC <= p.ow && n0 + VEC <= p.N;  // VEC neighbours in one input row
  for (int img = blockIdx.z; img < p.images; img += gridDim.z) {
    for (int k = blockIdx.y * 8 + threadIdx.y; k < p.K; k += gridDim.y * 8) {
      const int kw = k % p.kw;
      const int kh = (k / p.kw) % p.kh;
      const int ic = k / (p.kw * p.kh);
      const T* src = static_cast<const T*>(p.in) + (static_cast<size_t>(img) * p.cin + ic) * p.h * p.w;
      const int ih_off = kh * p.dh - p.ph, iw_off = kw * p.dw - p.pw;
      alignas(16) T v[VEC];
      const int ih0 = oh0 * p.sh + ih_off, iw0 = ow0 + iw_off;
      if (one_row && iw0 >= 0 && iw0 + VEC <= p.w) {
        if (static_cast<unsigned>(ih0) < static_cast<unsigned>(p.h)) {
          const T* row = src + ih0 * p.w + iw0;
#pragma unroll
          for (int j = 0; j < VEC; ++j) v[j] = row[j];
        } else {
#pragma unroll
          for (int j = 0; j < VEC; ++j) v[j] = T(0.0f);
        }
      } else {
        int oh = oh0, ow = ow0;
#pragma unroll
        for (int j = 0; j < VEC; ++j) {
          T x = T(0.0f);
          const int ih = oh * p.sh + ih_off, iw = ow * p.sw + iw_off;
          if (n0 + j < p.N && static_cast<unsigned>(ih) < static_cast<unsigned>(p.h) &&
              static_cast<unsigned>(iw) < static_cast<unsigned>(p.w))
            x = src[ih * p.w + iw];
          v[j] = x;
          if (++ow == p.ow) { ow = 0; ++oh; }
        }
      }
      T* dst = static_cast<T*>(p.col) + (static_cast<size_t>(img) * p.K + k) * p.npitch + n0;
      *reinterpret_cast<uint4*>(dst) = *reinterpret_cast<const uint4*>(v);
    }
  }
}

// Unit stride and dilation along the width: the KW col rows of one (ic, kh) read overlapping
// windows of the same input row, so one thread loads VEC + KW - 1 neighbours once and writes KW
// vectors from them.  The 256 threads of a CTA are blockDim.x along the columns times blockDim.y
// (ic, kh) pairs: as many threads along a row as it has vectors (up to all 256), so that long
// rows are written in long contiguous runs (4 KB per pass) and short rows still fill the CTA.
template <typename T, int VEC, int KW>
__global__ void __launch_bounds__(256) im2col_unit_kernel(const Im2colParams p) {
  const int pairs = p.cin * p.kh;
  for (int img = blockIdx.y; img < p.images; img += gridDim.y) {
    for (int r = blockIdx.x * blockDim.y + threadIdx.y; r < pairs; r += gridDim.x * blockDim.y) {
      const int kh = r % p.kh, ic = r / p.kh;
      const T* src = static_cast<const T*>(p.in) + (static_cast<size_t>(img) * p.cin + ic) * p.h * p.w;
      const int ih_off = kh * p.dh - p.ph;
      T* dst_row = static_cast<T*>(p.col) + (static_cast<size_t>(img) * p.K + static_cast<size_t>(r) * KW) * p.npitch;
      for (int n0 = threadIdx.x * VEC; n0 < p.npitch; n0 += blockDim.x * VEC) {
        const int oh0 = n0 / p.ow, ow0 = n0 - oh0 * p.ow;
        T* dst = dst_row + n0;
        if (ow0 + VEC <= p.ow && n0 + VEC <= p.N) {   // VEC neighbours in one input row
          const int ih = oh0 * p.sh + ih_off, iw_base = ow0 - p.pw;
          const bool row_ok = static_cast<unsigned>(ih) < static_cast<unsigned>(p.h);
          const T* row = src + (row_ok ? ih : 0) * p.w;
          T win[VEC + KW - 1];
#pragma unroll
          for (int i = 0; i < VEC + KW - 1; ++i) {
            const int iw = iw_base + i;
            win[i] = (row_ok && static_cast<unsigned>(iw) < static_cast<unsigned>(p.w)) ? row[iw] : T(0.0f);
          }
#pragma unroll
          for (int kw = 0; kw < KW; ++kw) {
            alignas(16) T v[VEC];
#pragma unroll
            for (int j = 0; j < VEC; ++j) v[j] = win[kw + j];
            *reinterpret_cast<uint4*>(dst + static_cast<size_t>(kw) * p.npitch) = *reinterpret_cast<const uint4*>(v);
          }
        } else {
#pragma unroll
          for (int kw = 0; kw < KW; ++kw) {
            int oh = oh0, ow = ow0;
            alignas(16) T v[VEC];
#pragma unroll
            for (int j = 0; j < VEC; ++j) {
              T x = T(0.0f);
              const int ih = oh * p.sh + ih_off, iw = ow + kw - p.pw;
              if (n0 + j < p.N && static_cast<unsigned>(ih) < static_cast<unsigned>(p.h) &&
                  static_cast<unsigned>(iw) < static_cast<unsigned>(p.w))
                x = src[ih * p.w + iw];
              v[j] = x;
              if (++ow == p.ow) { ow = 0; ++oh; }
            }
            *reinterpret_cast<uint4*>(dst + static_cast<size_t>(kw) * p.npitch) = *reinterpret_cast<const uint4*>(v);
          }
        }
      }
    }
  }
}

template <typename T, int VEC>
int launch_im2col(const Im2colParams& p, cudaStream_t stream) {
  if (p.images <= 0 || p.K <= 0 || p.npitch <= 0) return 0;
  const bool unit = p.sw == 1 && p.dw == 1 && (p.kw == 3 || p.kw == 5 || p.kw == 7);
  if (unit) {
    const int pairs = p.cin * p.kh, vectors = (p.npitch + VEC - 1) / VEC;
    int tx = 32;
    while (tx < 256 && tx < vectors) tx *= 2;
    const dim3 block(tx, 256 / tx, 1);
    const int groups = (pairs + static_cast<int>(block.y) - 1) / static_cast<int>(block.y);
    dim3 grid(static_cast<unsigned>(groups < 65535 ? groups : 65535), static_cast<unsigned>(p.images < 65535 ? p.images : 65535), 1);
    if (p.kw == 3) im2col_unit_kernel<T, VEC, 3><<<grid, block, 0, stream>>>(p);
    else if (p.kw == 5) im2col_unit_kernel<T, VEC, 5><<<grid, block, 0, stream>>>(p);
    else im2col_unit_kernel<T, VEC, 7><<<grid, block, 0, stream>>>(p);
  } else {
    const int row_groups = (p.K + 7) / 8;
    dim3 grid(static_cast<unsigned>((p.npitch + VEC * 32 - 1) / (VEC * 32)),
              static_cast<unsigned>(row_groups < 65535 ? row_groups : 65535),
              static_cast<unsigned>(p.images < 65535 ? p.images : 65535));
    im2col_kernel<T, VEC><<<grid, dim3(32, 8, 1), 0, stream>>>(p);
  }
  HODU_CUDA_TRY(cudaGetLastError(), HODU_B200_ERR_LAUNCH);
  count_launch();
  return 0;
}

constexpr size_t kMaxColBytes = size_t(2) << 30;  // scratch per pass; more images run in several passes

}  // namespace

int run_conv2d(int dtype, const void* input, const void* weight, void* out, const size_t* md, size_t len,
               DeviceState* st, cudaStream_t stream) {
  const long long B = md[1], cin = md[2], cout = md[3], H = md[4], W = md[5], KH = md[6], KW = md[7];
  const long long OH = md[8], OW = md[9], sh = md[10], sw = md[11], ph = md[12], pw = md[13];
  const long long dh = md[14], dw = md[15], in_off = md[16], w_off = md[17];
  (void)len;
  const int esize = dtype_size(dtype);
  const long long K = cin * KH * KW, N = OH * OW;
  // The unfolding kernel indexes inside one image with 32-bit integers.
  if (cin * H * W >= (1ll << 31) || K * ((N + 15) / 16 * 16) >= (1ll << 31) || (H + 2 * ph) * sh >= (1ll << 30) ||
      (W + 2 * pw) * sw >= (1ll << 30))
    return fail(HODU_B200_ERR_INVALID_INPUT, "conv2d: one image (or its unfolded form) exceeds 2^31 elements");
  const bool pointwise = KH == 1 && KW == 1 && sh == 1 && sw == 1 && ph == 0 && pw == 0 && OH == H && OW == W;
  if (!pointwise && (forced_path() == HODU_B200_PATH_AUTO || forced_path() == HODU_B200_PATH_TENSOR)) {
    // the implicit form first: no unfolded copy; it declines what it does not take
    const char* why = "";
    const int ri = run_conv2d_implicit(dtype, input, weight, out, md, st, stream, &why);
    if (ri == 0) { set_last_path(HODU_B200_PATH_TENSOR); return 0; }
    if (ri < 0) return ri;
  }
  const long long vec = 16 / esize;
  const long long npitch = pointwise ? N : (N + vec - 1) / vec * vec;

  Problem pb;
  pb.in_dtype = dtype; pb.out_dtype = dtype;
  pb.M = cout; pb.K = K; pb.N = N;
  pb.batch_ndim = 1;
  pb.a.ptr = weight; pb.a.offset = w_off; pb.a.stride_r = K; pb.a.stride_c = 1; pb.a.bstride[0] = 0;
  pb.b.stride_r = npitch; pb.b.stride_c = 1; pb.b.bstride[0] = K * npitch;

  if (pointwise) {
    pb.batch_shape[0] = B; pb.batches = B;
    pb.b.ptr = input; pb.b.offset = in_off;
    pb.out = out;
    return run_problem(pb, st, stream);
  }

  const size_t per_image = static_cast<size_t>(K) * npitch * esize;
  long long per_pass = static_cast<long long>(kMaxColBytes / (per_image ? per_image : 1));
  if (per_pass < 1) per_pass = 1;
  if (per_pass > B) per_pass = B;
  void* col = nullptr;
  if (const int ra = scratch_alloc(st, &col, per_image * per_pass, stream)) return ra;
  int r = 0;
  for (long long b0 = 0; b0 < B && r == 0; b0 += per_pass) {
    const long long nb = b0 + per_pass <= B ? per_pass : B - b0;
    Im2colParams ip{};
    ip.in = static_cast<const uint8_t*>(input) + (in_off + b0 * cin * H * W) * esize;
    ip.col = col;
    ip.images = static_cast<int>(nb); ip.cin = static_cast<int>(cin); ip.h = static_cast<int>(H); ip.w = static_cast<int>(W);
    ip.kh = static_cast<int>(KH); ip.kw = static_cast<int>(KW); ip.oh = static_cast<int>(OH); ip.ow = static_cast<int>(OW);
    ip.sh = static_cast<int>(sh); ip.sw = static_cast<int>(sw); ip.ph = static_cast<int>(ph); ip.pw = static_cast<int>(pw);
    ip.dh = static_cast<int>(dh); ip.dw = static_cast<int>(dw);
    ip.K = static_cast<int>(K); ip.N = static_cast<int>(N); ip.npitch = static_cast<int>(npitch);
    if (dtype == HODU_DTYPE_BF16) r = launch_im2col<__nv_bfloat16, 8>(ip, stream);
    else if (dtype == HODU_DTYPE_F16) r = launch_im2col<__half, 8>(ip, stream);
    else r = launch_im2col<float, 4>(ip, stream);
    if (r) break;
    Problem q = pb;
    q.batch_shape[0] = nb; q.batches = nb;
    q.b.ptr = col; q.b.offset = 0;
    q.out = static_cast<uint8_t*>(out) + static_cast<size_t>(b0) * cout * N * esize;
    r = run_problem(q, st, stream);
  }
  const int rf = scratch_free(col, stream);
  return r ? r : rf;
}

}  // namespace hodu_b200
