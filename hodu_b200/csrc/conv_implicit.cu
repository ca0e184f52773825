// conv2d as an implicit GEMM: the unfolded matrix is never written.
//
// out[b][co][oh][ow] = sum over (kh, kw, ci) of in[b][ci][oh*sh + kh*dh - ph][ow*sw + kw*dw - pw] * w[co][ci][kh][kw]
// (the reference's direct kernel, crates/hodu_cuda_kernels/kernels/ops_conv.cu:45-93, and the
// im2col + sgemm of its CPU OpenBLAS build, crates/hodu_cpu_kernels/kernels/ops_conv_openblas.c:84-133).
// As a matrix product: D[pixel][co] = A[pixel][k] . B[k][co] with pixel = (b, oh, ow) and
// k = (kh, kw, ci).  The explicit form (conv.cu) writes A -- KH*KW times the input -- to memory and
// reads it back, which bounds it by HBM.  Here:
//   1. one pass re-lays the input from NCHW to NHWC and the weights from [co][ci][kh][kw] to
//      [co][kh][kw][ci] in scratch (once the size of the input, instead of KH*KW times);
//   2. the GEMM kernel's producer fetches each A tile -- 128 output pixels x 64 channels of one
//      filter tap -- with ONE TMA load in im2col mode: the TMA unit walks the output pixels
//      (stride, padding and image boundaries included, out-of-image taps zero-filled) and writes
//      the 128-byte-swizzled K-major tile the tensor core reads; weights come by ordinary tiled
//      loads; tcgen05.mma accumulates in TMEM, double buffered so that the epilogue of a tile
//      overlaps the next one;
//   3. the epilogue writes D transposed, i.e. straight into the NCHW output.
// Takes bf16 / f16 with in_channels a multiple of 64; everything else keeps the explicit form.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include <atomic>
#include <mutex>

#include "bounded_wait.cuh"
#include "common.cuh"
#include "sm100_ptx.cuh"

namespace hodu_b200 {
using namespace ptx;

namespace {

// ------------------------------------------------------------------ pass 1: re-lay input and weights
struct RelayParams {
  const uint16_t* in;    // [B][C][HW]
  uint16_t* in_nhwc;     // [B][HW][C]
  const uint16_t* w;     // [Cout][C][T]   (T = KH*KW taps)
  uint16_t* w_perm;      // [Cout][T][C]
  int B, C, HW, T, Cout;
  int blocks_in;         // CTAs that handle the input; the rest handle the weights
};

// Input: 64 channels x 64 pixels per CTA through shared memory; reads run along the pixels,
// writes along the channels (128 bytes per pixel row piece).  Weights: one thread per element.
__global__ void __launch_bounds__(256) conv_relay_kernel(const RelayParams p) {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");   // the GEMM waits for this grid before it reads
  __shared__ uint16_t tile[64][66];
  if (static_cast<int>(blockIdx.x) < p.blocks_in) {
    const int hw_tiles = (p.HW + 63) / 64, c_tiles = p.C / 64;
    int t = blockIdx.x;
    const int ht = t % hw_tiles; t /= hw_tiles;
    const int ct = t % c_tiles;
    const int b = t / c_tiles;
    const int hw0 = ht * 64, c0 = ct * 64;
    const uint16_t* src = p.in + (static_cast<size_t>(b) * p.C + c0) * p.HW + hw0;
    const int tx = threadIdx.x & 63, ty = threadIdx.x >> 6;   // 64 pixels x 4 channel rows per pass
    for (int c = ty; c < 64; c += 4) tile[c][tx] = hw0 + tx < p.HW ? src[static_cast<size_t>(c) * p.HW + tx] : 0;
    __syncthreads();
    uint16_t* dst = p.in_nhwc + (static_cast<size_t>(b) * p.HW + hw0) * p.C + c0;
    const int cx = threadIdx.x & 7, py = threadIdx.x >> 3;    // 8 threads x 16 bytes per pixel, 32 pixels per pass
    for (int px = py; px < 64; px += 32) {
      if (hw0 + px >= p.HW) break;
      uint32_t v[4];
#pragma unroll
      for (int j = 0; j < 4; ++j)
        v[j] = static_cast<uint32_t>(tile[cx * 8 + 2 * j][px]) | (static_cast<uint32_t>(tile[cx * 8 + 2 * j + 1][px]) << 16);
      *reinterpret_cast<uint4*>(dst + static_cast<size_t>(px) * p.C + cx * 8) = make_uint4(v[0], v[1], v[2], v[3]);
    }
  } else {
    const long long total = static_cast<long long>(p.Cout) * p.C * p.T;
    const long long stride = static_cast<long long>(gridDim.x - p.blocks_in) * 256;
    for (long long i = static_cast<long long>(blockIdx.x - p.blocks_in) * 256 + threadIdx.x; i < total; i += stride) {
      // i walks the destination [co][t][c]
      const int c = static_cast<int>(i % p.C);
      const long long r = i / p.C;
      const int t = static_cast<int>(r % p.T);
      const long long co = r / p.T;
      p.w_perm[i] = p.w[(co * p.C + c) * p.T + t];
    }
  }
}

// The same pass when every channel row starts on a 16-byte boundary (H*W a multiple of 8), without
// shared memory: a thread loads an 8-channel x 8-pixel block as eight 16-byte vectors (one per
// channel), transposes it in registers and stores eight 16-byte vectors (one per pixel).  The
// eight lanes that share a pixel group hold the 64 channels of the CTA's channel tile, so every
// store instruction writes whole 128-byte pixel rows; loads fetch 64-byte runs.
__global__ void __launch_bounds__(256) conv_relay_vec_kernel(const RelayParams p) {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  if (static_cast<int>(blockIdx.x) < p.blocks_in) {
    const int px_tiles = (p.HW + 255) / 256, c_tiles = p.C / 64;
    int t = blockIdx.x;
    const int pt = t % px_tiles; t /= px_tiles;
    const int ct = t % c_tiles;
    const int b = t / c_tiles;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int cg = lane & 7, pg = warp * 4 + (lane >> 3);
    const int px0 = pt * 256 + pg * 8, c0 = ct * 64 + cg * 8;
    if (px0 >= p.HW) return;
    const uint16_t* src = p.in + (static_cast<size_t>(b) * p.C + c0) * p.HW + px0;
    uint4 row[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) row[i] = *reinterpret_cast<const uint4*>(src + static_cast<size_t>(i) * p.HW);
    uint16_t* dst = p.in_nhwc + (static_cast<size_t>(b) * p.HW + px0) * p.C + c0;
#pragma unroll
    for (int j = 0; j < 8; ++j) {      // pixel j of the group: halves j of the eight channel vectors
      const uint32_t sel = (j & 1) ? 0x7632u : 0x5410u;
      uint32_t w[4];
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const uint32_t a = reinterpret_cast<const uint32_t*>(&row[2 * k])[j >> 1];
        const uint32_t c = reinterpret_cast<const uint32_t*>(&row[2 * k + 1])[j >> 1];
        w[k] = __byte_perm(a, c, sel);
      }
      *reinterpret_cast<uint4*>(dst + static_cast<size_t>(j) * p.C) = make_uint4(w[0], w[1], w[2], w[3]);
    }
  } else {
    const long long total = static_cast<long long>(p.Cout) * p.C * p.T;
    const long long stride = static_cast<long long>(gridDim.x - p.blocks_in) * 256;
    for (long long i = static_cast<long long>(blockIdx.x - p.blocks_in) * 256 + threadIdx.x; i < total; i += stride) {
      const int c = static_cast<int>(i % p.C);
      const long long r = i / p.C;
      const int t = static_cast<int>(r % p.T);
      const long long co = r / p.T;
      p.w_perm[i] = p.w[(co * p.C + c) * p.T + t];
    }
  }
}

// ------------------------------------------------------------------ pass 2: the GEMM
struct ConvParams {
  uint32_t pixels;        // B * OH * OW
  uint32_t n_img;         // OH * OW
  uint32_t ow;            // OW
  uint32_t cout, cin;
  uint32_t kh, kw;
  int32_t sh, sw, ph, pw, dh, dw;
  uint32_t tiles_m, tiles_n, num_tiles;
  uint32_t c_blocks;      // cin / 64
  uint32_t idesc;
  void* out;              // NCHW
  uint32_t* status;
};

struct ConvTail {
  uint64_t full[8];
  uint64_t empty[8];
  uint64_t tmem_full[2];
  uint64_t tmem_empty[2];
  uint32_t tmem_base;
  uint32_t abort_flag;
};

template <int BN> struct ConvCfg {
  // k-blocks (one filter tap x 64 channels) per stage: the narrow tiles take two, because the
  // handshake of a stage (a wait, a commit, a producer iteration: ~250 cycles each for the one
  // thread that runs it) costs more than the 128 or 256 MMA cycles of one of their k-blocks.
  static constexpr uint32_t kKbPerStage = BN == 64 ? 3u : (BN == 128 ? 2u : 1u);
  static constexpr uint32_t kStageA1 = 128u * 128u;   // 128 pixels x 64 channels
  static constexpr uint32_t kStageB1 = BN * 128u;     // BN output channels x 64 k
  static constexpr uint32_t kStageA = kKbPerStage * kStageA1;
  static constexpr uint32_t kStageB = kKbPerStage * kStageB1;
  static constexpr int kStages = BN == 256 ? 4 : 3;
  static constexpr size_t kSmem = kStages * (kStageA + kStageB) + 256 + 1024;
};

// TMA load in im2col mode: `pixels per column` output pixels starting at the base pixel
// (w, h, n) -- coordinates of the filter's upper-left tap in the input, i.e. output coordinate
// times stride minus padding -- each shifted by the tap offset (off_w, off_h), 64 channels from c.
__device__ __forceinline__ void tma_load_im2col_4d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int32_t c, int32_t w,
                                                   int32_t h, int32_t n, uint16_t off_w, uint16_t off_h) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.im2col.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2], {%7, %8};" ::"r"(dst),
      "l"(reinterpret_cast<uint64_t>(map)), "r"(bar), "r"(c), "r"(w), "r"(h), "r"(n), "h"(off_w), "h"(off_h)
      : "memory");
}
__device__ __forceinline__ uint64_t kmajor_desc128(uint32_t smem_addr) {
  const uint32_t hi = (1024u >> 4) | (1u << 14) | (2u << 29);
  const uint32_t lo = ((smem_addr >> 4) & 0x3FFFu) | (1u << 16);
  return (static_cast<uint64_t>(hi) << 32) | lo;
}

template <int BN, bool IS_BF16>
__global__ void __launch_bounds__(192, 1)
conv_implicit_kernel(const __grid_constant__ CUtensorMap map_in, const __grid_constant__ CUtensorMap map_w, const ConvParams p) {
  using Cfg = ConvCfg<BN>;
  constexpr int kStages = Cfg::kStages;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_u32 = smem_u32(smem_raw);
  const uint32_t base = (raw_u32 + 1023u) & ~1023u;
  ConvTail* tail = reinterpret_cast<ConvTail*>(smem_raw + (base - raw_u32) + kStages * (Cfg::kStageA + Cfg::kStageB));
  volatile uint32_t* abort_flag = &tail->abort_flag;
  const uint32_t smem_a = base, smem_b = base + kStages * Cfg::kStageA;
  const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31u;
  const uint32_t code_base = 0x80000000u | ((blockIdx.x & 0xFFFFu) << 4);

  if (threadIdx.x == 0) {
    prefetch_tensormap(&map_in);
    prefetch_tensormap(&map_w);
    for (int s = 0; s < kStages; ++s) {
      mbar_init(smem_u32(&tail->full[s]), 1);
      mbar_init(smem_u32(&tail->empty[s]), 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(smem_u32(&tail->tmem_full[i]), 1);
      mbar_init(smem_u32(&tail->tmem_empty[i]), 4);
    }
    tail->abort_flag = 0;
    fence_barrier_init();
  }
  if (warp == 1) {
    tmem_alloc<1>(smem_u32(&tail->tmem_base), 2 * BN);
    tmem_relinquish<1>();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t*>(&tail->tmem_base);
  grid_dependency_wait();     // pass 1 wrote what the loads below read
  grid_launch_dependents();

  const uint32_t taps = p.kh * p.kw;
  const uint32_t k_blocks = taps * p.c_blocks;

  if (warp == 0) {
    // ---------------------------------------------------------------- producer (a second producer
    // thread for the weights measured no gain)
    if (lane == 0) {
      uint32_t s = 0, ph = 0;
      bool ok = true;
      for (uint32_t t = blockIdx.x; ok && t < p.num_tiles; t += gridDim.x) {
        const uint32_t mt = t / p.tiles_n, nt = t % p.tiles_n;
        const uint32_t p0 = mt * 128u;                      // first output pixel of the tile
        const uint32_t img = p0 / p.n_img, r = p0 - img * p.n_img;
        const uint32_t oh0 = r / p.ow, ow0 = r - oh0 * p.ow;
        const int32_t base_w = static_cast<int32_t>(ow0) * p.sw - p.pw, base_h = static_cast<int32_t>(oh0) * p.sh - p.ph;
        // k-block kb = (tap, 64-channel block cb), taps outermost; fh, fw: the tap's row and column
        uint32_t cb = 0, fh = 0, fw = 0;
        for (uint32_t kb = 0; kb < k_blocks; kb += Cfg::kKbPerStage) {
          ok = wait_bounded(smem_u32(&tail->empty[s]), ph ^ 1u, abort_flag, p.status, code_base | 1u);
          if (!ok) break;
          const uint32_t bar = smem_u32(&tail->full[s]);
          const uint32_t n_kb = Cfg::kKbPerStage == 1u ? 1u : min(Cfg::kKbPerStage, k_blocks - kb);
          mbar_arrive_expect_tx_relaxed(bar, n_kb * (Cfg::kStageA1 + Cfg::kStageB1));
#pragma unroll
          for (uint32_t j = 0; j < Cfg::kKbPerStage; ++j) {
            if (j >= n_kb) break;
            tma_load_im2col_4d(smem_a + s * Cfg::kStageA + j * Cfg::kStageA1, &map_in, bar, static_cast<int32_t>(cb * 64u), base_w,
                               base_h, static_cast<int32_t>(img), static_cast<uint16_t>(fw * p.dw), static_cast<uint16_t>(fh * p.dh));
            tma_load_2d(smem_b + s * Cfg::kStageB + j * Cfg::kStageB1, &map_w, bar, static_cast<int32_t>((kb + j) * 64u),
                        static_cast<int32_t>(nt * BN));
            if (++cb == p.c_blocks) {
              cb = 0;
              if (++fw == p.kw) { fw = 0; ++fh; }
            }
          }
          if (++s == kStages) { s = 0; ph ^= 1u; }
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ---------------------------------------------------------------- MMA issuer
    if (lane == 0) {
      uint32_t s = 0, ph = 0, lt = 0;
      bool ok = true;
      for (uint32_t t = blockIdx.x; ok && t < p.num_tiles; t += gridDim.x, ++lt) {
        const uint32_t acc = lt & 1u, acc_ph = (lt >> 1) & 1u;
        ok = wait_bounded(smem_u32(&tail->tmem_empty[acc]), acc_ph ^ 1u, abort_flag, p.status, code_base | 2u);
        if (!ok) break;
        tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (uint32_t kb = 0; kb < k_blocks; kb += Cfg::kKbPerStage) {
          ok = wait_bounded(smem_u32(&tail->full[s]), ph, abort_flag, p.status, code_base | 3u);
          if (!ok) break;
          tc_fence_after_sync();
          const uint64_t a_desc = kmajor_desc128(smem_a + s * Cfg::kStageA), b_desc = kmajor_desc128(smem_b + s * Cfg::kStageB);
#pragma unroll
          for (uint32_t j = 0; j < Cfg::kKbPerStage; ++j) {
            if (kb + j >= k_blocks) break;
#pragma unroll
            for (uint32_t kk = 0; kk < 4; ++kk)     // 16 k per MMA = 32 bytes = 2 sixteen-byte units
              umma<KIND_F16, 1>(d_tmem, a_desc + j * (Cfg::kStageA1 >> 4) + kk * 2u, b_desc + j * (Cfg::kStageB1 >> 4) + kk * 2u, p.idesc,
                                (kb | j | kk) != 0u ? 1u : 0u);
          }
          umma_commit_1cta(smem_u32(&tail->empty[s]));
          if (++s == kStages) { s = 0; ph ^= 1u; }
        }
        if (ok) umma_commit_1cta(smem_u32(&tail->tmem_full[acc]));
      }
    }
    __syncwarp();
  } else {
    // ---------------------------------------------------------------- epilogue (warps 2..5)
    const uint32_t q = warp & 3u;
    uint32_t lt = 0;
    for (uint32_t t = blockIdx.x; t < p.num_tiles; t += gridDim.x, ++lt) {
      const uint32_t mt = t / p.tiles_n, nt = t % p.tiles_n;
      const uint32_t pix = mt * 128u + q * 32u + lane;          // this lane's output pixel
      const uint32_t img = pix / p.n_img, n = pix - img * p.n_img;
      const bool pix_ok = pix < p.pixels;
      uint16_t* out_px = static_cast<uint16_t*>(p.out) + (static_cast<size_t>(img) * p.cout + nt * BN) * p.n_img + n;
      const uint32_t acc = lt & 1u, acc_ph = (lt >> 1) & 1u;
      bool ok = wait_bounded(smem_u32(&tail->tmem_full[acc]), acc_ph, abort_flag, p.status, code_base | 4u);
      ok = __all_sync(0xFFFFFFFFu, ok);
      if (!ok) break;
      tc_fence_after_sync();
      const uint32_t t_row = tmem_base + acc * BN + ((q * 32u) << 16);
#pragma unroll 1
      for (uint32_t c = 0; c < BN / 32u; ++c) {
        const uint32_t co0 = nt * BN + c * 32u;
        if (co0 >= p.cout) break;
        uint32_t v[32];
        tmem_ld_32x32(t_row + c * 32u, v);
        tmem_wait_ld();
        if (pix_ok) {
          // transposed store: for one output channel the warp's 32 lanes are 32 consecutive pixels
#pragma unroll
          for (uint32_t j = 0; j < 32; ++j) {
            if (co0 + j < p.cout) {
              const float x = __uint_as_float(v[j]);
              uint16_t h;
              if constexpr (IS_BF16) { __nv_bfloat16 b = __float2bfloat16_rn(x); h = *reinterpret_cast<uint16_t*>(&b); }
              else { __half b = __float2half_rn(x); h = *reinterpret_cast<uint16_t*>(&b); }
              out_px[static_cast<size_t>(c * 32u + j) * p.n_img] = h;
            }
          }
        }
      }
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&tail->tmem_empty[acc]));
    }
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc<1>(tmem_base, 2 * BN);
  }
}

typedef CUresult (*EncodeIm2colFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                   const int*, const int*, cuuint32_t, cuuint32_t, const cuuint32_t*, CUtensorMapInterleave,
                                   CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeIm2colFn im2col_encoder() {
  static EncodeIm2colFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeIm2col", &p, cudaEnableDefault, &q) == cudaSuccess && q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeIm2colFn>(p);
  });
  return fn;
}

template <int BN, bool IS_BF16>
int launch_conv(const CUtensorMap& mi, const CUtensorMap& mw, const ConvParams& p, int sm_count, cudaStream_t stream) {
  using Cfg = ConvCfg<BN>;
  auto kern = conv_implicit_kernel<BN, IS_BF16>;
  static std::atomic<bool> configured[kMaxDevices];
  int device = 0;
  cudaGetDevice(&device);
  if (!configured[device].load(std::memory_order_relaxed)) {
    HODU_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(Cfg::kSmem)), HODU_B200_ERR_LAUNCH);
    configured[device].store(true, std::memory_order_relaxed);
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(p.num_tiles < static_cast<uint32_t>(sm_count) ? p.num_tiles : sm_count, 1, 1);
  cfg.blockDim = dim3(192, 1, 1);
  cfg.dynamicSmemBytes = Cfg::kSmem;
  cfg.stream = stream;
  cudaLaunchAttribute attr;
  attr.id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr.val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = &attr;
  cfg.numAttrs = dependent_launch_enabled() ? 1 : 0;
  if (debug_enabled())
    fprintf(stderr, "[hodu_b200] conv_implicit: %u tiles of 128 pixels x %d channels, %u k-blocks, grid %u, %zu B smem\n", p.num_tiles, BN,
            p.kh * p.kw * p.c_blocks, cfg.gridDim.x, static_cast<size_t>(Cfg::kSmem));
  HODU_CUDA_TRY(cudaLaunchKernelEx(&cfg, kern, mi, mw, p), HODU_B200_ERR_LAUNCH);
  count_launch();
  return 0;
}

}  // namespace

// Returns 0 when launched, 1 when the convolution is not one this form takes (nothing launched,
// `why` says which rule), < 0 on error.
int run_conv2d_implicit(int dtype, const void* input, const void* weight, void* out, const size_t* md, DeviceState* st,
                        cudaStream_t stream, const char** why) {
  static const char* none = "";
  *why = none;
  static const bool enabled = [] { const char* e = getenv("HODU_B200_CONV_IMPLICIT"); return !(e && e[0] == '0'); }();
  if (!enabled) { *why = "implicit form switched off"; return 1; }
  if (dtype != HODU_DTYPE_BF16 && dtype != HODU_DTYPE_F16) { *why = "dtype"; return 1; }
  if (st->cc_major != 10) { *why = "device is not sm_100"; return 1; }
  const long long B = md[1], cin = md[2], cout = md[3], H = md[4], W = md[5], KH = md[6], KW = md[7];
  const long long OH = md[8], OW = md[9], sh = md[10], sw = md[11], ph = md[12], pw = md[13];
  const long long dh = md[14], dw = md[15], in_off = md[16], w_off = md[17];
  if (cin % 64 != 0) { *why = "in_channels is not a multiple of 64"; return 1; }
  if (KH * KW == 1 && sh == 1 && sw == 1 && ph == 0 && pw == 0) { *why = "pointwise: the input already is the unfolded matrix"; return 1; }
  if (sh > 8 || sw > 8 || ph > 127 || pw > 127 || (KH - 1) * dh > 127 || (KW - 1) * dw > 127 || KH * KW > 4096) { *why = "stride, padding or filter extent beyond the TMA im2col ranges"; return 1; }
  const long long pixels = B * OH * OW;
  if (pixels >= (1ll << 31) || B * H * W * cin >= (1ll << 40) || cout >= (1ll << 24)) { *why = "extent"; return 1; }
  const long long work = pixels * cout * cin * KH * KW;
  if (work < (1ll << 24)) { *why = "too small to pay for the re-laying pass"; return 1; }
  EncodeIm2colFn enc_i = im2col_encoder();
  EncodeTiledFn enc_t = tensor_map_encoder();
  if (!enc_i || !enc_t) { *why = "tensor-map encoders unavailable"; return 1; }

  // scratch: NHWC input, permuted weights (256-byte aligned pieces)
  const size_t in_bytes = static_cast<size_t>(B) * H * W * cin * 2;
  const size_t in_pad = (in_bytes + 255) / 256 * 256;
  const size_t w_bytes = static_cast<size_t>(cout) * KH * KW * cin * 2;
  void* scratch = nullptr;
  if (const int ra = scratch_alloc(st, &scratch, in_pad + w_bytes, stream)) return ra;
  uint16_t* in_nhwc = static_cast<uint16_t*>(scratch);
  uint16_t* w_perm = reinterpret_cast<uint16_t*>(static_cast<uint8_t*>(scratch) + in_pad);

  int r = 0;
  {
    RelayParams rp{};
    rp.in = static_cast<const uint16_t*>(input) + in_off;
    rp.in_nhwc = in_nhwc;
    rp.w = static_cast<const uint16_t*>(weight) + w_off;
    rp.w_perm = w_perm;
    rp.B = static_cast<int>(B); rp.C = static_cast<int>(cin); rp.HW = static_cast<int>(H * W); rp.T = static_cast<int>(KH * KW);
    rp.Cout = static_cast<int>(cout);
    const bool vec = (H * W) % 8 == 0 && (reinterpret_cast<uintptr_t>(rp.in) % 16) == 0;
    const long long blocks_in = vec ? B * (cin / 64) * ((H * W + 255) / 256) : B * (cin / 64) * ((H * W + 63) / 64);
    const long long w_elems = cout * cin * KH * KW;
    long long blocks_w = (w_elems + 255) / 256;
    if (blocks_w > 4 * st->sm_count) blocks_w = 4 * st->sm_count;
    if (blocks_in + blocks_w >= (1ll << 31)) { scratch_free(scratch, stream); *why = "extent"; return 1; }
    rp.blocks_in = static_cast<int>(blocks_in);
    if (vec) conv_relay_vec_kernel<<<static_cast<unsigned>(blocks_in + blocks_w), 256, 0, stream>>>(rp);
    else conv_relay_kernel<<<static_cast<unsigned>(blocks_in + blocks_w), 256, 0, stream>>>(rp);
    const cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) r = fail(HODU_B200_ERR_LAUNCH, "conv_relay launch failed: %s", cudaGetErrorString(e));
    else count_launch();
  }
  if (r == 0) {
    // Output channels per tile: the widest tile the layer can fill, unless a narrower one puts the
    // layer's tiles on more of the SMs (a 7x7x512 layer of batch 32 is 13 pixel tiles: 26 CTAs at 256
    // channels, 104 at 64).  Estimate = waves x relative time of a k-block (1 : 1.15 : 1.5, measured).
    int bn = cout > 128 ? 256 : (cout > 64 ? 128 : 64);
    {
      const double tiles_m_d = static_cast<double>((pixels + 127) / 128);
      double best = 1e300;
      for (int c = bn; c >= 64; c /= 2) {
        const double tiles = tiles_m_d * static_cast<double>((cout + c - 1) / c);
        const double waves = tiles > st->sm_count ? tiles / st->sm_count : 1.0;
        const double cost = waves * (c == 256 ? 1.5 : (c == 128 ? 1.15 : 1.0));
        if (cost < best * 0.97) { best = cost; bn = c; }   // a narrower tile has to win by 3 %
      }
    }
    CUtensorMap mi, mw;
    {
      cuuint64_t dims[4] = {static_cast<cuuint64_t>(cin), static_cast<cuuint64_t>(W), static_cast<cuuint64_t>(H), static_cast<cuuint64_t>(B)};
      cuuint64_t strides[3] = {static_cast<cuuint64_t>(cin) * 2, static_cast<cuuint64_t>(W) * cin * 2, static_cast<cuuint64_t>(H) * W * cin * 2};
      int lower[2] = {static_cast<int>(-pw), static_cast<int>(-ph)};
      int upper[2] = {static_cast<int>(pw - (KW - 1) * dw), static_cast<int>(ph - (KH - 1) * dh)};
      cuuint32_t estr[4] = {1, static_cast<cuuint32_t>(sw), static_cast<cuuint32_t>(sh), 1};
      const CUresult cr = enc_i(&mi, CU_TENSOR_MAP_DATA_TYPE_UINT16, 4, in_nhwc, dims, strides, lower, upper, 64, 128, estr,
                                CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                                CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
      if (cr != CUDA_SUCCESS) r = fail(HODU_B200_ERR_LAUNCH, "cuTensorMapEncodeIm2col failed (%d)", static_cast<int>(cr));
    }
    if (r == 0) {
      const cuuint64_t kk = static_cast<cuuint64_t>(KH * KW * cin);
      cuuint64_t dims[2] = {kk, static_cast<cuuint64_t>(cout)};
      cuuint64_t strides[1] = {kk * 2};
      cuuint32_t box[2] = {64, static_cast<cuuint32_t>(bn)};
      cuuint32_t estr[2] = {1, 1};
      const CUresult cr = enc_t(&mw, CU_TENSOR_MAP_DATA_TYPE_UINT16, 2, w_perm, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                                CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
      if (cr != CUDA_SUCCESS) r = fail(HODU_B200_ERR_LAUNCH, "cuTensorMapEncodeTiled failed for the weights (%d)", static_cast<int>(cr));
    }
    if (r == 0) {
      ConvParams p{};
      p.pixels = static_cast<uint32_t>(pixels); p.n_img = static_cast<uint32_t>(OH * OW); p.ow = static_cast<uint32_t>(OW);
      p.cout = static_cast<uint32_t>(cout); p.cin = static_cast<uint32_t>(cin);
      p.kh = static_cast<uint32_t>(KH); p.kw = static_cast<uint32_t>(KW);
      p.sh = static_cast<int32_t>(sh); p.sw = static_cast<int32_t>(sw); p.ph = static_cast<int32_t>(ph); p.pw = static_cast<int32_t>(pw);
      p.dh = static_cast<int32_t>(dh); p.dw = static_cast<int32_t>(dw);
      p.tiles_m = static_cast<uint32_t>((pixels + 127) / 128);
      p.tiles_n = static_cast<uint32_t>((cout + bn - 1) / bn);
      p.num_tiles = p.tiles_m * p.tiles_n;
      p.c_blocks = static_cast<uint32_t>(cin / 64);
      const uint32_t fmt = dtype == HODU_DTYPE_BF16 ? 1u : 0u;
      p.idesc = (1u << 4) | (fmt << 7) | (fmt << 10) | (static_cast<uint32_t>(bn >> 3) << 17) | ((128u >> 4) << 24);
      p.out = out;
      p.status = st->status;
      const bool bf = dtype == HODU_DTYPE_BF16;
      if (bn == 256) r = bf ? launch_conv<256, true>(mi, mw, p, st->sm_count, stream) : launch_conv<256, false>(mi, mw, p, st->sm_count, stream);
      else if (bn == 128) r = bf ? launch_conv<128, true>(mi, mw, p, st->sm_count, stream) : launch_conv<128, false>(mi, mw, p, st->sm_count, stream);
      else r = bf ? launch_conv<64, true>(mi, mw, p, st->sm_count, stream) : launch_conv<64, false>(mi, mw, p, st->sm_count, stream);
    }
  }
  const int rf = scratch_free(scratch, stream);
  return r ? r : rf;
}

}  // namespace hodu_b200
