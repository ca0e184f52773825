// Small f32 products in ONE launch and without scratch memory.
//
// The split-operand path (gemm_f32.cu) writes TF32 high/low copies of both operands to scratch,
// multiplies them, and for small outputs adds K slices in a third kernel: three launches, which is
// most of the time of a product as small as A[512,1024] . B[1024,768].  Here the same arithmetic
// -- C = Ahi.Bhi + Ahi.Blo + Alo.Bhi with hi = tf32(x), lo = tf32(x - hi), f32 accumulation --
// runs in one kernel:
//   warp 0      one lane issues TMA loads of RAW f32 tiles (128 rows x 32 k of A, BN x 32 k of B)
//   warps 2..17 split each raw tile into hi and lo tiles of a two-deep operand ring, both in the
//               128-byte-swizzled K-major layout the tensor core reads; a rhs that is N-contiguous
//               in memory (B[K,N] row-major) is transposed on the way.  Raw tiles have a ring of
//               their own (three deep), so loads run ahead of the MMAs
//   warp 1      one lane issues the twelve tcgen05.mma (kind::tf32) of a k-block into TMEM
//   warps 2..17 epilogue: accumulator -> shared memory; the CTAs of a cluster hold the K slices
//               of one tile and add them through distributed shared memory in rank order (so the
//               result does not depend on timing); scale, bias, store
// It takes the place of the reference's CUDA-core f32 kernels for small products
// (crates/hodu_cuda_kernels/kernels/ops_matrix.cu:9-102,104-165); larger products keep the
// split-operand path, which is built for throughput.
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include <atomic>

#include "bounded_wait.cuh"
#include "common.cuh"
#include "sm100_ptx.cuh"

namespace hodu_b200 {
using namespace ptx;

namespace {

constexpr int kRawStages = 3;                       // raw f32 tiles in flight from TMA
constexpr int kOpStages = 2;                        // split (hi / lo) tiles between converters and MMAs
constexpr int kConvWarps = 16;                      // warps 2..17
constexpr uint32_t kConvThreads = 32u * kConvWarps;
constexpr int kThreadsF = 32 * (2 + kConvWarps);    // 576
constexpr uint32_t kTileA = 128u * 128u;            // 128 rows x 32 f32

struct FusedParams {
  uint32_t M, N, K;
  uint32_t tiles_n;
  uint32_t k_blocks;      // ceil(K / 32)
  uint32_t splits;        // CTAs per cluster = K slices per tile
  uint32_t b_n_major;     // rhs tiles arrive N-contiguous and are transposed by the converters
  uint32_t idesc;
  uint32_t out_vec_ok;    // rows of `out` allow 16-byte stores
  float alpha;
  unsigned long long ldc;
  const float* bias;      // [N] (offset applied) or null
  long long bias_stride;
  float* out;
  uint32_t* status;
};

struct FusedTail {
  uint64_t raw_full[kRawStages];  // TMA landed the raw tiles of a raw stage
  uint64_t raw_free[kRawStages];  // every converter warp has read the raw stage
  uint64_t conv_done[kOpStages];  // the converter warps have written the hi / lo tiles of an operand stage
  uint64_t mma_done[kOpStages];   // the MMAs that read the operand stage have retired
  uint64_t tmem_full;
  uint32_t tmem_base;
  uint32_t abort_flag;
};

template <int BN> struct FusedCfg {
  static constexpr uint32_t kTileB = BN * 128u;
  static constexpr uint32_t kOpStage = 2u * kTileA + 2u * kTileB;   // A hi, A lo, B hi, B lo
  static constexpr uint32_t kRawStage = kTileA + kTileB;            // A raw, B raw
  static constexpr uint32_t kRawBase = kOpStages * kOpStage;        // operand stages first, raw stages after
  static constexpr uint32_t kAccPitch = BN + 4;                     // floats; = 4 mod 32: conflict-free 16-byte rows
  static constexpr uint32_t kTmemCols = BN <= 32 ? 32 : (BN <= 64 ? 64 : 128);
  static constexpr size_t kSmem = kOpStages * kOpStage + kRawStages * kRawStage + 256 + 1024;
  static_assert(128u * kAccPitch * 4u <= kOpStage, "the accumulator dump must fit one operand stage");
  static_assert(kTileB % 1024u == 0, "rhs tiles keep the 1 KB alignment of the swizzle atoms");
};

// x rounded to the nearest TF32 value (ties away from zero, as cvt.rna.tf32.f32 does), with two
// integer instructions: the conversion instruction runs at a fraction of their rate and set the
// pace of the converter warps.
__device__ __forceinline__ float tf32_rna(float x) {
  return __uint_as_float((__float_as_uint(x) + 0x1000u) & 0xFFFFE000u);
}
__device__ __forceinline__ float4 lds128(uint32_t addr) {
  float4 v;
  asm volatile("ld.shared.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(addr) : "memory");
  return v;
}
__device__ __forceinline__ void sts128(uint32_t addr, const float4& v) {
  asm volatile("st.shared.v4.f32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "f"(v.x), "f"(v.y), "f"(v.z), "f"(v.w) : "memory");
}
__device__ __forceinline__ float lds32(uint32_t addr) {
  float v;
  asm volatile("ld.shared.f32 %0, [%1];" : "=f"(v) : "r"(addr) : "memory");
  return v;
}
// 16 bytes of another CTA's shared memory (shared::cluster address from mapa_shared).
__device__ __forceinline__ float4 ld_cluster128(uint32_t cluster_addr) {
  float4 v;
  asm volatile("ld.shared::cluster.v4.f32 {%0, %1, %2, %3}, [%4];"
               : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w)
               : "r"(cluster_addr)
               : "memory");
  return v;
}
__device__ __forceinline__ void split4(const float4& x, float4& hi, float4& lo) {
  hi.x = tf32_rna(x.x); hi.y = tf32_rna(x.y); hi.z = tf32_rna(x.z); hi.w = tf32_rna(x.w);
  lo.x = tf32_rna(x.x - hi.x); lo.y = tf32_rna(x.y - hi.y); lo.z = tf32_rna(x.z - hi.z); lo.w = tf32_rna(x.w - hi.w);
}
// Shared-memory matrix descriptor of a K-major, 128-byte-swizzled tile (rows 128 bytes apart,
// eight-row atoms 1024 bytes apart).
__device__ __forceinline__ uint64_t kmajor_desc(uint32_t smem_addr) {
  const uint32_t hi = (1024u >> 4) | (1u << 14) | (2u << 29);
  const uint32_t lo = ((smem_addr >> 4) & 0x3FFFu) | (1u << 16);
  return (static_cast<uint64_t>(hi) << 32) | lo;
}

template <int BN>
__global__ void __launch_bounds__(kThreadsF, 1)
gemm_f32_fused_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                      const FusedParams p) {
  using Cfg = FusedCfg<BN>;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_u32 = smem_u32(smem_raw);
  const uint32_t base = (raw_u32 + 1023u) & ~1023u;
  FusedTail* tail = reinterpret_cast<FusedTail*>(smem_raw + (base - raw_u32) + Cfg::kRawBase + kRawStages * Cfg::kRawStage);
  volatile uint32_t* abort_flag = &tail->abort_flag;

  const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31u;
  const uint32_t rank = cluster_ctarank();            // which K slice of the tile
  const uint32_t tile = blockIdx.x / p.splits;
  const uint32_t m0 = (tile / p.tiles_n) * 128u, n0 = (tile % p.tiles_n) * BN;
  const uint32_t kb_begin = static_cast<uint32_t>(static_cast<uint64_t>(rank) * p.k_blocks / p.splits);
  const uint32_t kb_end = static_cast<uint32_t>(static_cast<uint64_t>(rank + 1u) * p.k_blocks / p.splits);
  const uint32_t code_base = 0x80000000u | ((blockIdx.x & 0xFFFFu) << 4);

  if (threadIdx.x == 0) {
    prefetch_tensormap(&map_a);
    prefetch_tensormap(&map_b);
    for (int s = 0; s < kRawStages; ++s) {
      mbar_init(smem_u32(&tail->raw_full[s]), 1);
      mbar_init(smem_u32(&tail->raw_free[s]), kConvWarps);
    }
    for (int s = 0; s < kOpStages; ++s) {
      mbar_init(smem_u32(&tail->conv_done[s]), kConvWarps);
      mbar_init(smem_u32(&tail->mma_done[s]), 1);
    }
    mbar_init(smem_u32(&tail->tmem_full), 1);
    tail->abort_flag = 0;
    fence_barrier_init();
  }
  if (warp == 1) {
    tmem_alloc<1>(smem_u32(&tail->tmem_base), Cfg::kTmemCols);
    tmem_relinquish<1>();
  }
  tc_fence_before_sync();
  cluster_sync_all();          // a barrier over this CTA's threads too (a lone CTA is a cluster of one)
  tc_fence_after_sync();
  const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t*>(&tail->tmem_base);
  grid_dependency_wait();
  grid_launch_dependents();

  auto op_base = [&](uint32_t s) { return base + s * Cfg::kOpStage; };
  auto raw_base = [&](uint32_t s) { return base + Cfg::kRawBase + s * Cfg::kRawStage; };

  if (warp == 0) {
    // ---------------------------------------------------------------- TMA producer
    if (lane == 0) {
      uint32_t s = 0, ph = 0;
      for (uint32_t kb = kb_begin; kb < kb_end; ++kb) {
        if (!wait_bounded(smem_u32(&tail->raw_free[s]), ph ^ 1u, abort_flag, p.status, code_base | 1u)) break;
        const uint32_t bar = smem_u32(&tail->raw_full[s]);
        mbar_arrive_expect_tx_relaxed(bar, kTileA + Cfg::kTileB);
        const int32_t k0 = static_cast<int32_t>(kb * 32u);
        const uint32_t st = raw_base(s);
        tma_load_2d(st, &map_a, bar, k0, static_cast<int32_t>(m0));
        if (p.b_n_major) tma_load_2d(st + kTileA, &map_b, bar, static_cast<int32_t>(n0), k0);
        else tma_load_2d(st + kTileA, &map_b, bar, k0, static_cast<int32_t>(n0));
        if (++s == kRawStages) { s = 0; ph ^= 1u; }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ---------------------------------------------------------------- MMA issuer
    if (lane == 0) {
      uint32_t s = 0, ph = 0;
      bool ok = true;
      for (uint32_t kb = kb_begin; kb < kb_end; ++kb) {
        ok = wait_bounded(smem_u32(&tail->conv_done[s]), ph, abort_flag, p.status, code_base | 3u);
        if (!ok) break;
        tc_fence_after_sync();
        const uint32_t st = op_base(s);
        const uint64_t a_hi = kmajor_desc(st), a_lo = kmajor_desc(st + kTileA);
        const uint64_t b_hi = kmajor_desc(st + 2u * kTileA), b_lo = kmajor_desc(st + 2u * kTileA + Cfg::kTileB);
#pragma unroll
        for (uint32_t kk = 0; kk < 4; ++kk) {   // 8 k per MMA = 32 bytes = 2 sixteen-byte units
          const uint64_t adv = static_cast<uint64_t>(kk * 2u);
          umma<KIND_TF32, 1>(tmem_base, a_hi + adv, b_hi + adv, p.idesc, (kb != kb_begin || kk != 0u) ? 1u : 0u);
          umma<KIND_TF32, 1>(tmem_base, a_hi + adv, b_lo + adv, p.idesc, 1u);
          umma<KIND_TF32, 1>(tmem_base, a_lo + adv, b_hi + adv, p.idesc, 1u);
        }
        umma_commit_1cta(smem_u32(&tail->mma_done[s]));
        if (++s == kOpStages) { s = 0; ph ^= 1u; }
      }
      if (ok) umma_commit_1cta(smem_u32(&tail->tmem_full));
    }
    __syncwarp();
  } else {
    // ---------------------------------------------------------------- converters, then epilogue
    const uint32_t t = threadIdx.x - 64u;        // 0..kConvThreads-1
    uint32_t rs = 0, rph = 0, os = 0, oph = 0;
    bool ok = true;
    for (uint32_t kb = kb_begin; kb < kb_end; ++kb) {
      // the raw tiles have landed, and the MMAs that last read this operand stage have retired
      ok = wait_bounded(smem_u32(&tail->raw_full[rs]), rph, abort_flag, p.status, code_base | 2u) &&
           wait_bounded(smem_u32(&tail->mma_done[os]), oph ^ 1u, abort_flag, p.status, code_base | 5u);
      ok = __all_sync(0xFFFFFFFFu, ok);
      if (!ok) break;
      const uint32_t raw = raw_base(rs), st = op_base(os);
      // All loads of a k-block are issued before the first conversion, so that their latency is
      // paid once: with two converter warps per scheduler nothing else would hide it.
      // lhs: elementwise at equal offsets (TMA already wrote the swizzled K-major layout)
      constexpr uint32_t kItemsA = kTileA / 16u / kConvThreads;            // 16-byte pieces of the lhs tile per thread
      constexpr uint32_t kItemsB = (8u * BN + kConvThreads - 1u) / kConvThreads;
      float4 xa[kItemsA], xb[kItemsB];
#pragma unroll
      for (uint32_t i = 0; i < kItemsA; ++i) xa[i] = lds128(raw + (t + kConvThreads * i) * 16u);
      const uint32_t b_raw = raw + kTileA, b_hi = st + 2u * kTileA, b_lo = b_hi + Cfg::kTileB;
      if (!p.b_n_major) {
#pragma unroll
        for (uint32_t i = 0; i < kItemsB; ++i) {
          const uint32_t idx = t + kConvThreads * i;
          if (idx < 8u * BN) xb[i] = lds128(b_raw + idx * 16u);
        }
      } else {
        // raw tile: 32 rows of k, BN floats each.  One item = four consecutive k of one column n,
        // gathered by scalar loads (consecutive lanes, consecutive n) and written as one 16-byte
        // piece of row n of the K-major tiles (eight consecutive rows hit eight different pieces).
#pragma unroll
        for (uint32_t i = 0; i < kItemsB; ++i) {
          const uint32_t idx = t + kConvThreads * i;
          if (idx < 8u * BN) {
            const uint32_t n = idx % BN, kq = idx / BN;
            const uint32_t src = b_raw + (kq * 4u * BN + n) * 4u;
            xb[i].x = lds32(src); xb[i].y = lds32(src + BN * 4u); xb[i].z = lds32(src + 2u * BN * 4u); xb[i].w = lds32(src + 3u * BN * 4u);
          }
        }
      }
#pragma unroll
      for (uint32_t i = 0; i < kItemsA; ++i) {
        const uint32_t off = (t + kConvThreads * i) * 16u;
        float4 hi, lo;
        split4(xa[i], hi, lo);
        sts128(st + off, hi);
        sts128(st + kTileA + off, lo);
      }
#pragma unroll
      for (uint32_t i = 0; i < kItemsB; ++i) {
        const uint32_t idx = t + kConvThreads * i;
        if (idx < 8u * BN) {
          const uint32_t n = idx % BN, kq = idx / BN;
          const uint32_t dst = p.b_n_major ? n * 128u + ((kq ^ (n & 7u)) << 4) : idx * 16u;
          float4 hi, lo;
          split4(xb[i], hi, lo);
          sts128(b_hi + dst, hi);
          sts128(b_lo + dst, lo);
        }
      }
      fence_proxy_async_smem();     // the tensor core reads these tiles through the async proxy
      __syncwarp();
      if (lane == 0) {
        mbar_arrive(smem_u32(&tail->raw_free[rs]));    // TMA may refill the raw stage
        mbar_arrive(smem_u32(&tail->conv_done[os]));   // the MMAs of this k-block may go
      }
      if (++rs == kRawStages) { rs = 0; rph ^= 1u; }
      if (++os == kOpStages) { os = 0; oph ^= 1u; }
    }
    // accumulator -> shared memory (operand stage 0 is idle once every MMA has retired); the four warps
    // whose index mod 4 differs cover the four TMEM lane quadrants
    if (ok && warp < 6u) {
      ok = wait_bounded(smem_u32(&tail->tmem_full), 0u, abort_flag, p.status, code_base | 4u);
      ok = __all_sync(0xFFFFFFFFu, ok);
      if (ok) {
        tc_fence_after_sync();
        const uint32_t q = warp & 3u, row = q * 32u + lane;
        const uint32_t acc_row = base + row * Cfg::kAccPitch * 4u;
#pragma unroll
        for (uint32_t c = 0; c < BN / 32u; ++c) {
          uint32_t v[32];
          tmem_ld_32x32(tmem_base + ((q * 32u) << 16) + c * 32u, v);
          tmem_wait_ld();
#pragma unroll
          for (uint32_t j = 0; j < 8; ++j)
            sts128(acc_row + c * 128u + j * 16u,
                   make_float4(__uint_as_float(v[4 * j]), __uint_as_float(v[4 * j + 1]), __uint_as_float(v[4 * j + 2]),
                               __uint_as_float(v[4 * j + 3])));
        }
      }
    }
  }

  // Every CTA of the cluster has its partial sums in shared memory (or has given up).
  tc_fence_before_sync();
  cluster_sync_all();
  if (warp >= 2u && *abort_flag == 0u) {
    // Rank r adds and stores rows [r * 128 / splits, (r + 1) * 128 / splits) of the tile, reading
    // the partial sums of ranks 0, 1, .. in that order through distributed shared memory.
    const uint32_t t = threadIdx.x - 64u;
    const uint32_t rows = 128u / p.splits, r_first = rank * rows;
    constexpr uint32_t kQuads = BN / 4u;
    for (uint32_t idx = t; idx < rows * kQuads; idx += kConvThreads) {
      const uint32_t r = r_first + idx / kQuads, c = (idx % kQuads) * 4u;
      const uint32_t grow = m0 + r, gcol = n0 + c;
      if (grow >= p.M || gcol >= p.N) continue;
      const uint32_t addr = base + (r * Cfg::kAccPitch + c) * 4u;
      // the (up to four) remote loads go out together; the additions keep rank order
      float4 part[4];
#pragma unroll
      for (uint32_t peer = 0; peer < 4; ++peer)
        if (peer < p.splits) part[peer] = ld_cluster128(mapa_shared(addr, peer));
      float4 sum = part[0];
#pragma unroll
      for (uint32_t peer = 1; peer < 4; ++peer) {
        if (peer < p.splits) { sum.x += part[peer].x; sum.y += part[peer].y; sum.z += part[peer].z; sum.w += part[peer].w; }
      }
      float o[4] = {sum.x * p.alpha, sum.y * p.alpha, sum.z * p.alpha, sum.w * p.alpha};
      const uint32_t ncols = p.N - gcol < 4u ? p.N - gcol : 4u;
      if (p.bias != nullptr) {
        for (uint32_t j = 0; j < ncols; ++j) o[j] += p.bias[static_cast<long long>(gcol + j) * p.bias_stride];
      }
      float* dst = p.out + static_cast<unsigned long long>(grow) * p.ldc + gcol;
      if (p.out_vec_ok && ncols == 4u) *reinterpret_cast<float4*>(dst) = make_float4(o[0], o[1], o[2], o[3]);
      else
        for (uint32_t j = 0; j < ncols; ++j) dst[j] = o[j];
    }
  }
  // No CTA may leave while a peer can still read its shared memory.  (A rendezvous only: every
  // remote read above has delivered its value before its thread arrives, and nothing is published
  // here, so the arrive carries no release fence -- which would wait for the global stores.)
  cluster_sync_all_relaxed();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc<1>(tmem_base, Cfg::kTmemCols);
  }
}

// Tensor map of a [rows, cols] f32 matrix whose `cols` index is contiguous: dims {cols, rows}.
bool encode_f32_map(const float* base, uint64_t cols, uint64_t rows, uint64_t pitch_elems, uint32_t box_cols,
                    uint32_t box_rows, bool swizzle, CUtensorMap* out) {
  EncodeTiledFn enc = tensor_map_encoder();
  if (!enc) return false;
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {pitch_elems * 4ull};
  cuuint32_t box[2] = {box_cols, box_rows};
  cuuint32_t estr[2] = {1, 1};
  return enc(out, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<float*>(base), dims, strides, box, estr,
             CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE,
             CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// How many clusters of `splits` CTAs of the BN-wide kernel the device holds at once (clusters do
// not straddle GPCs, so this is less than SMs / splits); 0 if the query fails.  Cached per device.
template <int BN>
int resident_clusters(int splits, int device) {
  static std::atomic<int> cached[kMaxDevices][5];
  int v = cached[device][splits].load(std::memory_order_relaxed);
  if (v != 0) return v > 0 ? v : 0;
  using Cfg = FusedCfg<BN>;
  auto kern = gemm_f32_fused_kernel<BN>;
  int q = 0;
  if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(Cfg::kSmem)) == cudaSuccess) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(splits, 1, 1);
    cfg.blockDim = dim3(kThreadsF, 1, 1);
    cfg.dynamicSmemBytes = Cfg::kSmem;
    cudaLaunchAttribute attr;
    attr.id = cudaLaunchAttributeClusterDimension;
    attr.val.clusterDim.x = splits; attr.val.clusterDim.y = 1; attr.val.clusterDim.z = 1;
    cfg.attrs = &attr;
    cfg.numAttrs = 1;
    if (cudaOccupancyMaxActiveClusters(&q, kern, &cfg) != cudaSuccess) { q = 0; cudaGetLastError(); }
  } else {
    cudaGetLastError();
  }
  cached[device][splits].store(q > 0 ? q : -1, std::memory_order_relaxed);
  return q;
}
int resident_clusters_of(int bn, int splits, int device) {
  switch (bn) {
    case 96: return resident_clusters<96>(splits, device);
    case 64: return resident_clusters<64>(splits, device);
    default: return resident_clusters<32>(splits, device);
  }
}

template <int BN>
int launch_fused(const CUtensorMap& ma, const CUtensorMap& mb, const FusedParams& p, uint32_t tiles, cudaStream_t stream) {
  using Cfg = FusedCfg<BN>;
  auto kern = gemm_f32_fused_kernel<BN>;
  // (the shared-memory attribute of the kernel was set by resident_clusters, which every launch passes)
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(tiles * p.splits, 1, 1);
  cfg.blockDim = dim3(kThreadsF, 1, 1);
  cfg.dynamicSmemBytes = Cfg::kSmem;
  cfg.stream = stream;
  cudaLaunchAttribute attrs[2];
  int n = 0;
  attrs[n].id = cudaLaunchAttributeClusterDimension;
  attrs[n].val.clusterDim.x = p.splits; attrs[n].val.clusterDim.y = 1; attrs[n].val.clusterDim.z = 1;
  ++n;
  if (dependent_launch_enabled()) {
    attrs[n].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attrs[n].val.programmaticStreamSerializationAllowed = 1;
    ++n;
  }
  cfg.attrs = attrs;
  cfg.numAttrs = n;
  if (debug_enabled())
    fprintf(stderr, "[hodu_b200] gemm_f32_fused: %u tiles of 128x%d, %u K slices per tile (cluster), grid %u, %zu B smem, B %s\n",
            tiles, BN, p.splits, cfg.gridDim.x, static_cast<size_t>(Cfg::kSmem), p.b_n_major ? "N-major (transposed in shared memory)" : "K-major");
  HODU_CUDA_TRY(cudaLaunchKernelEx(&cfg, kern, ma, mb, p), HODU_B200_ERR_LAUNCH);
  count_launch();
  if (debug_enabled()) {   // wait for the kernel and read what its bounded waits recorded
    HODU_CUDA_TRY(cudaStreamSynchronize(stream), HODU_B200_ERR_LAUNCH);
    uint32_t w = 0;
    HODU_CUDA_TRY(cudaMemcpy(&w, p.status, sizeof(w), cudaMemcpyDeviceToHost), HODU_B200_ERR_MEMORY);
    if (w != 0)
      return fail(HODU_B200_ERR_DEVICE_STATUS, "debug check after launch: device status word 0x%08x (cta %u, wait %u)", w,
                  (w >> 4) & 0xFFFFu, w & 0xFu);
  }
  return 0;
}

}  // namespace

int launch_gemm_f32_fused(const Problem& pb, DeviceState* st, cudaStream_t stream, const char** why) {
  static const char* none = "";
  *why = none;
  static const bool enabled = [] { const char* e = getenv("HODU_B200_F32_FUSED"); return !(e && e[0] == '0'); }();
  if (!enabled) { *why = "one-kernel f32 form switched off"; return 1; }
  if (pb.in_dtype != HODU_DTYPE_F32 || pb.out_dtype != HODU_DTYPE_F32 || pb.swiglu) { *why = "not an f32 product"; return 1; }
  if (st->cc_major != 10) { *why = "device is not sm_100"; return 1; }
  if (pb.batches != 1) { *why = "batched"; return 1; }
  if (pb.M < 1 || pb.N < 1 || pb.K < 1 || pb.M > 0x7FFFFFFFll || pb.N > 0x7FFFFFFFll || pb.K > 0x7FFFFFFFll) { *why = "extent"; return 1; }
  // Layouts TMA can describe: lhs K-contiguous; rhs K- or N-contiguous; 16-byte-multiple pitches and bases.
  auto ok16 = [](const void* ptr, int64_t off) { return (reinterpret_cast<uintptr_t>(ptr) + static_cast<uintptr_t>(off) * 4u) % 16u == 0; };
  auto pitch_ok = [](int64_t s) { return s > 0 && s % 4 == 0 && s < (1ll << 38); };
  if (!(pb.a.stride_c == 1 || pb.K == 1) || !(pb.M == 1 || pitch_ok(pb.a.stride_r)) || !ok16(pb.a.ptr, pb.a.offset)) { *why = "lhs layout"; return 1; }
  const bool b_k_major = (pb.b.stride_r == 1 || pb.K == 1) && (pb.N == 1 || pitch_ok(pb.b.stride_c));
  const bool b_n_major = !b_k_major && (pb.b.stride_c == 1 || pb.N == 1) && (pb.K == 1 || pitch_ok(pb.b.stride_r));
  if ((!b_k_major && !b_n_major) || !ok16(pb.b.ptr, pb.b.offset)) { *why = "rhs layout"; return 1; }

  // Tile width and K slices: as many CTAs as fit ONE wave, preferring wide tiles (less re-reading
  // of the lhs) and at least four k-blocks per slice.  More than a wave, or a long K per slice,
  // belongs to the split-operand path.
  const int64_t k_blocks = (pb.K + 31) / 32, tiles_m = (pb.M + 127) / 128;
  int device = 0;
  cudaGetDevice(&device);
  int best_bn = 0, best_s = 0;
  int64_t best_ctas = 0;
  for (int bn : {96, 64, 32}) {
    const int64_t tiles = tiles_m * ((pb.N + bn - 1) / bn);
    for (int s : {1, 2, 4}) {
      if (s > 1 && k_blocks / s < 4) continue;
      const int64_t ctas = tiles * s;
      if (ctas > st->sm_count || ctas <= best_ctas) continue;
      if (tiles > resident_clusters_of(bn, s, device)) continue;   // every cluster resident at once: one wave
      best_ctas = ctas; best_bn = bn; best_s = s;
    }
  }
  if (best_bn == 0) { *why = "more than one wave of tiles"; return 1; }
  if (k_blocks / best_s > 64) { *why = "K per slice too long for the one-kernel form"; return 1; }

  const float* a_base = static_cast<const float*>(pb.a.ptr) + pb.a.offset;
  const float* b_base = static_cast<const float*>(pb.b.ptr) + pb.b.offset;
  CUtensorMap ma, mb;
  const uint64_t a_pitch = pb.M == 1 ? static_cast<uint64_t>((pb.K + 3) / 4 * 4) : static_cast<uint64_t>(pb.a.stride_r);
  if (!encode_f32_map(a_base, pb.K, pb.M, a_pitch, 32, 128, true, &ma)) { *why = "lhs tensor map"; return 1; }
  if (b_k_major) {
    const uint64_t b_pitch = pb.N == 1 ? static_cast<uint64_t>((pb.K + 3) / 4 * 4) : static_cast<uint64_t>(pb.b.stride_c);
    if (!encode_f32_map(b_base, pb.K, pb.N, b_pitch, 32, best_bn, true, &mb)) { *why = "rhs tensor map"; return 1; }
  } else {
    const uint64_t b_pitch = pb.K == 1 ? static_cast<uint64_t>((pb.N + 3) / 4 * 4) : static_cast<uint64_t>(pb.b.stride_r);
    if (!encode_f32_map(b_base, pb.N, pb.K, b_pitch, best_bn, 32, false, &mb)) { *why = "rhs tensor map"; return 1; }
  }

  FusedParams p{};
  p.M = static_cast<uint32_t>(pb.M); p.N = static_cast<uint32_t>(pb.N); p.K = static_cast<uint32_t>(pb.K);
  p.tiles_n = static_cast<uint32_t>((pb.N + best_bn - 1) / best_bn);
  p.k_blocks = static_cast<uint32_t>(k_blocks);
  p.splits = static_cast<uint32_t>(best_s);
  p.b_n_major = b_n_major ? 1u : 0u;
  // f32 accumulate, tf32 operands, both K-major, N = tile width, M = 128
  p.idesc = (1u << 4) | (2u << 7) | (2u << 10) | (static_cast<uint32_t>(best_bn >> 3) << 17) | ((128u >> 4) << 24);
  p.alpha = pb.alpha;
  p.ldc = static_cast<unsigned long long>(pb.ldc > 0 ? pb.ldc : pb.N);
  p.out_vec_ok = (reinterpret_cast<uintptr_t>(pb.out) % 16 == 0 && (p.ldc * 4u) % 16 == 0) ? 1u : 0u;
  p.bias = pb.bias ? static_cast<const float*>(pb.bias) + pb.bias_offset : nullptr;
  p.bias_stride = pb.bias_stride;
  p.out = static_cast<float*>(pb.out);
  p.status = st->status;
  const uint32_t tiles = static_cast<uint32_t>(tiles_m) * p.tiles_n;
  switch (best_bn) {
    case 96: return launch_fused<96>(ma, mb, p, tiles, stream);
    case 64: return launch_fused<64>(ma, mb, p, tiles, stream);
    default: return launch_fused<32>(ma, mb, p, tiles, stream);
  }
}

}  // namespace hodu_b200
