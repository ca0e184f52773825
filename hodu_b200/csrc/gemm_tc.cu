// tcgen05 GEMM for sm_100a: C[b] = A[b] . B[b] with the output cast fused into
// the epilogue.  Replaces the reference's 16x16 shared-memory SIMT kernels
// `hodu_cuda_matmul_*` / `hodu_cuda_dot_*`
// (crates/hodu_cuda_kernels/kernels/ops_matrix.cu:9-102,104-165).
//
// Shape of one CTA (one CTA per SM, persistent over output tiles; 224 threads, or 608 in
// the 512 x 256 pair form):
//   warp 0      TMA producer of A: 128-byte-swizzled operand tiles into a ring of stages
//   warp 6      TMA producer of B (its own barrier arrive, so neither operand waits on the other)
//   warp 1      allocates TMEM; one elected lane issues tcgen05.mma, four per asm block
//   warps 2..5  epilogue: tcgen05.ld of the accumulator, scale/convert, stores staged through
//   (+ 7..18)   swizzled shared memory so that each store instruction writes whole row pieces
// Three tile forms: one CTA per 128 x BN tile with a double-buffered accumulator in TMEM (the
// epilogue of tile i overlaps the main loop of tile i+1); a CTA pair (cta_group::2) per
// 256 x 256 tile, also double buffered; a CTA pair per 512 x 256 tile, whose two accumulators
// fill TMEM and whose sixteen epilogue warps hand them back before their global stores.
//
// Operand layouts: each of A and B may be K-major (K contiguous) or MN-major
// (M resp. N contiguous); both are described to the tensor core through the
// shared-memory matrix descriptor, so `B[K,N]` row-major, and the transposed
// weight view `hodu_nn::Linear` passes, both run without a transposing pre-pass.
//
// Every wait on an mbarrier is bounded: when a wait runs out the CTA records a
// code in the device status word, stops issuing work, drains what it started,
// frees its TMEM and returns.
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>

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

// HODU_B200_PDL=0 launches the tensor-core kernels without programmatic dependent launch.
bool dependent_launch_enabled() {
  static const bool on = [] { const char* e = getenv("HODU_B200_PDL"); return !(e && e[0] == '0'); }();
  return on;
}

// HODU_B200_DEBUG=1: every tensor-core launch prints its configuration to stderr, has its tile
// arithmetic, stage sizes, TMEM columns and TMA coordinate ranges checked on the host before it
// runs, and is followed by a stream synchronisation and a read of the device status word, so a
// fault or a wait that gave up is reported by the call that caused it.  For debugging only: it
// serialises the stream and must not be used inside a stream capture.
bool debug_enabled() {
  static const bool on = [] { const char* e = getenv("HODU_B200_DEBUG"); return e && e[0] == '1'; }();
  return on;
}

EncodeTiledFn tensor_map_encoder() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  });
  return fn;
}

namespace {

constexpr int BM = 128;                 // rows of A one CTA stages == TMEM lanes
constexpr int kHalfA = BM * 128;        // bytes: 128 rows (or M elements) x 128 B of K
// Threads = 3 warps (two producers, the MMA issuer) + the epilogue warps: four per 128-row
// accumulator, and in the 512 x 256 form, which cannot hide its epilogue behind the next tile,
// two such groups per accumulator, each draining half of the columns (16 epilogue warps).
constexpr int epi_col_groups(int mh) { return mh == 2 ? 2 : 1; }
constexpr int threads_for(int mh) { return 96 + 128 * mh * epi_col_groups(mh); }

enum : int { OUT_F32 = 0, OUT_BF16 = 1, OUT_F16 = 2, OUT_E4M3 = 3, OUT_I32 = 4, OUT_I8 = 5 };

// Stage ring per CTA.  PAIR: each CTA of the pair stages 128 columns of B.  MH = M-halves
// (128-row accumulators) per CTA: 1, or 2 for the 512 x 256 pair tile.
template <int BN, bool PAIR, int MH> struct TileCfg {
  // k-blocks (128 bytes of K) per stage.  One wait on `full`, one commit to `empty` and one
  // producer iteration cost the issuing threads ~250 cycles each whatever the stage holds (an
  // mbarrier probe answers after ~200 cycles even when the phase is long complete), which is more
  // than the 128 or 256 MMA cycles of a k-block of the narrow one-CTA tiles: those stage two
  // k-blocks at a time and pay the handshake once for both.
  static constexpr int kKbPerStage = ((!PAIR && BN <= 128) || (PAIR && MH == 1)) ? 2 : 1;
  static constexpr int kStageA1 = MH * kHalfA;                    // one k-block
  static constexpr int kStageB1 = PAIR ? 128 * 128 : BN * 128;
  static constexpr int kStageA = kKbPerStage * kStageA1;
  static constexpr int kStageB = kKbPerStage * kStageB1;
  static constexpr int kStages = PAIR ? (MH == 2 ? 4 : 3) : (BN == 256 ? 4 : (BN == 128 ? 3 : 4));
  static constexpr int kEpiWarps = 4 * MH * (MH == 2 ? 2 : 1);
  static constexpr int kEpiStage = 2048;  // per epilogue warp: a 32-row x 64-byte block
  static constexpr int kTmemCols = 2 * BN;  // two accumulators: double buffer (MH 1) or the two halves (MH 2)
};

struct SmemTail {
  uint64_t full[8];
  uint64_t empty[8];
  uint64_t tmem_full[2];
  uint64_t tmem_empty[2];
  uint64_t drain;
  uint32_t tmem_base;
  uint32_t abort_flag;
};

// How one operand is staged and described to the tensor core.
struct OperandLoad {
  uint32_t mn_major;   // 0: K contiguous, 1: M/N contiguous
  uint32_t slab_dim;   // MN-major only: the 128-byte slabs are a tensor-map dimension (one box per stage)
  uint32_t boxes;      // TMA boxes per stage (per CTA)
  uint32_t box_bytes;
  uint32_t box_mn;     // M/N elements covered by one box
  uint32_t inner;      // elements per 128 bytes
  uint32_t bmul[3];    // 0 where the operand broadcasts that (collapsed) batch dim
  uint32_t desc_hi;    // smem matrix descriptor bits 32..63
  uint32_t desc_lo;    // bits 14..31 (leading byte offset field)
  uint32_t kstep16;    // start-address advance per MMA, in 16-byte units
};

struct TcParams {
  uint32_t M, N, K;
  uint32_t tiles_m, tiles_n, num_tiles, k_blocks, group_m;
  uint32_t k_gen;         // k-blocks per accumulator generation (== k_blocks: one generation per tile)
  uint32_t k_gen_limit;   // generations of k_gen blocks up to here, then ONE generation for the rest
  uint32_t bdim1, bdim2;  // batch = (b0 * bdim1 + b1) * bdim2 + b2
  uint32_t bk;            // K elements per stage (128 bytes worth)
  uint32_t k_splits;      // CTAs of a cluster that share one tile, each taking a slice of K (1: no cluster)
  uint32_t kb_per_split;  // k-blocks per slice (the last slice takes what is left)
  OperandLoad a, b;
  uint32_t idesc;
  uint32_t out_vec_ok;    // rows of `out` allow 16-byte stores
  uint32_t out_tma;       // map_out describes `out`: a CTA's last tile leaves through TMA stores
  uint32_t swiglu_flags;
  uint32_t bias_flags;
  float alpha;
  unsigned long long ldc, out_batch_stride;  // elements
  const void* bias;       // [N] values of the output dtype added per column, or null
  long long bias_stride;  // elements
  void* out;
  uint32_t* status;
};

struct TileCoord {
  uint32_t batch, mt, nt;
};
__device__ __forceinline__ TileCoord decode_tile(const TcParams& p, uint32_t t) {
  const uint32_t per_batch = p.tiles_m * p.tiles_n;
  TileCoord c;
  c.batch = t / per_batch;
  const uint32_t r = t - c.batch * per_batch;
  const uint32_t group_sz = p.group_m * p.tiles_n;
  const uint32_t g = r / group_sz;
  const uint32_t first_m = g * p.group_m;
  const uint32_t gm = min(p.tiles_m - first_m, p.group_m);
  const uint32_t rr = r - g * group_sz;
  c.mt = first_m + rr % gm;
  c.nt = rr / gm;
  return c;
}

// End (exclusive) of the accumulator generation that starts at k-block kb0.
__device__ __forceinline__ uint32_t generation_end(const TcParams& p, uint32_t kb0) {
  if (kb0 >= p.k_gen_limit) return p.k_blocks;
  const uint32_t e = kb0 + p.k_gen;
  return e < p.k_gen_limit ? e : p.k_gen_limit;
}

// -------------------------------------------------------------- epilogue helpers
__device__ __forceinline__ float silu_f32(float x) { return x / (1.0f + expf(-x)); }

template <int OUT> __device__ __forceinline__ float round_to_storage(float x) {
  if constexpr (OUT == OUT_BF16) return __bfloat162float(__float2bfloat16_rn(x));
  else if constexpr (OUT == OUT_F16) return __half2float(__float2half_rn(x));
  else return x;
}

template <int OUT> __device__ __forceinline__ float load_bias(const void* bias, long long i) {
  if constexpr (OUT == OUT_BF16) return __bfloat162float(static_cast<const __nv_bfloat16*>(bias)[i]);
  else if constexpr (OUT == OUT_F16) return __half2float(static_cast<const __half*>(bias)[i]);
  else return static_cast<const float*>(bias)[i];
}

template <int OUT> struct OutBytes {
  static constexpr int value = (OUT == OUT_F32 || OUT == OUT_I32) ? 4
                               : (OUT == OUT_BF16 || OUT == OUT_F16) ? 2 : 1;
};

// Converts 32 values of one output row and stores the first `ncols` of them.
// `f` holds floats (float accumulators, already scaled) or raw s32 bit patterns.
template <int OUT>
__device__ __forceinline__ void store_row_chunk(uint8_t* dst, const uint32_t (&v)[32], int ncols,
                                                bool vec_ok) {
  if constexpr (OUT == OUT_F32 || OUT == OUT_I32) {
    if (vec_ok && ncols == 32) {
      uint4* d4 = reinterpret_cast<uint4*>(dst);
#pragma unroll
      for (int j = 0; j < 8; ++j) d4[j] = make_uint4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
    } else {
      uint32_t* d = reinterpret_cast<uint32_t*>(dst);
#pragma unroll
      for (int j = 0; j < 32; ++j)
        if (j < ncols) d[j] = v[j];
    }
  } else if constexpr (OUT == OUT_BF16 || OUT == OUT_F16) {
    uint32_t pk[16];
#pragma unroll
    for (int j = 0; j < 16; ++j) {
      const float a = __uint_as_float(v[2 * j]), b = __uint_as_float(v[2 * j + 1]);
      if constexpr (OUT == OUT_BF16) {
        __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
        pk[j] = *reinterpret_cast<uint32_t*>(&h);
      } else {
        __half2 h = __floats2half2_rn(a, b);
        pk[j] = *reinterpret_cast<uint32_t*>(&h);
      }
    }
    if (vec_ok && ncols == 32) {
      uint4* d4 = reinterpret_cast<uint4*>(dst);
#pragma unroll
      for (int j = 0; j < 4; ++j) d4[j] = make_uint4(pk[4 * j], pk[4 * j + 1], pk[4 * j + 2], pk[4 * j + 3]);
    } else {
      uint16_t* d = reinterpret_cast<uint16_t*>(dst);
#pragma unroll
      for (int j = 0; j < 32; ++j)
        if (j < ncols) d[j] = static_cast<uint16_t>(pk[j >> 1] >> ((j & 1) * 16));
    }
  } else {  // one byte per element
    uint32_t pk[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      if constexpr (OUT == OUT_E4M3) {
        const uint32_t lo = __nv_cvt_float2_to_fp8x2(
            make_float2(__uint_as_float(v[4 * j]), __uint_as_float(v[4 * j + 1])), __NV_SATFINITE,
            __NV_E4M3);
        const uint32_t hi = __nv_cvt_float2_to_fp8x2(
            make_float2(__uint_as_float(v[4 * j + 2]), __uint_as_float(v[4 * j + 3])),
            __NV_SATFINITE, __NV_E4M3);
        pk[j] = lo | (hi << 16);
      } else {  // OUT_I8: low 8 bits of the exact s32 sum
        pk[j] = (v[4 * j] & 0xFFu) | ((v[4 * j + 1] & 0xFFu) << 8) | ((v[4 * j + 2] & 0xFFu) << 16) |
                ((v[4 * j + 3] & 0xFFu) << 24);
      }
    }
    if (vec_ok && ncols == 32) {
      uint4* d4 = reinterpret_cast<uint4*>(dst);
      d4[0] = make_uint4(pk[0], pk[1], pk[2], pk[3]);
      d4[1] = make_uint4(pk[4], pk[5], pk[6], pk[7]);
    } else {
#pragma unroll
      for (int j = 0; j < 32; ++j)
        if (j < ncols) dst[j] = static_cast<uint8_t>(pk[j >> 2] >> ((j & 3) * 8));
    }
  }
}

// Coalesced form of the above for 2- and 4-byte outputs whose rows allow 16-byte stores.
// After tcgen05.ld a lane holds 32 columns of ONE row, so a direct store instruction scatters
// 32 lanes over 32 rows, 16 bytes each: 32 partial-sector requests per instruction, and the
// request rate (not the bytes) made the epilogue the slowest part of a tile.  Here the warp
// passes its 32 x 64-byte block through a 2 KB shared-memory buffer (16-byte chunks XOR-swizzled
// by row so that both directions are bank-conflict-free) and stores it back with four lanes per
// row: every instruction writes eight full 64-byte runs.
//   pack_chunk turns the lane's 32 values (floats already scaled, or raw s32) into output
//   words; store_packed_staged writes them: row0 = first row of this warp's 32-row block,
//   col_byte0 = byte offset of the chunk in an output row.
template <int OUT> struct ChunkWords {  // 32-bit words one lane holds for a 32-column chunk
  static constexpr int value = OutBytes<OUT>::value == 4 ? 32 : 16;
};
// Two values of a 16-bit output dtype in one word, and back (exact).
template <int OUT> __device__ __forceinline__ uint32_t pack_pair(float a, float b) {
  if constexpr (OUT == OUT_BF16) {
    __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&h);
  } else {
    __half2 h = __floats2half2_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&h);
  }
}
template <int OUT> __device__ __forceinline__ void unpack_pair(uint32_t w, float& a, float& b) {
  if constexpr (OUT == OUT_BF16) {
    a = __uint_as_float(w << 16);
    b = __uint_as_float(w & 0xFFFF0000u);
  } else {
    const __half2 h = *reinterpret_cast<const __half2*>(&w);
    a = __low2float(h);
    b = __high2float(h);
  }
}
template <int OUT>
__device__ __forceinline__ void pack_chunk(const uint32_t (&v)[32], uint32_t (&pk)[ChunkWords<OUT>::value]) {
  if constexpr (OUT == OUT_F32 || OUT == OUT_I32) {
#pragma unroll
    for (int j = 0; j < 32; ++j) pk[j] = v[j];
  } else {
#pragma unroll
    for (int j = 0; j < 16; ++j) {
      const float a = __uint_as_float(v[2 * j]), b = __uint_as_float(v[2 * j + 1]);
      if constexpr (OUT == OUT_BF16) {
        __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
        pk[j] = *reinterpret_cast<uint32_t*>(&h);
      } else {
        __half2 h = __floats2half2_rn(a, b);
        pk[j] = *reinterpret_cast<uint32_t*>(&h);
      }
    }
  }
}
// Lane l writes the 64 bytes `w` of row l of a 32-row x 64-byte block at `stage` (512-byte
// aligned): 16-byte pieces XOR-swizzled by (row / 2) % 4, which is both bank-conflict-free and
// exactly the layout a tensor map with 64-byte swizzle reads.
__device__ __forceinline__ void stage_write_row64(uint32_t stage, uint32_t lane, const uint32_t* w) {
  const uint32_t wsw = (lane >> 1) & 3u;
#pragma unroll
  for (uint32_t j = 0; j < 4; ++j) {
    const uint32_t addr = stage + lane * 64u + ((j ^ wsw) << 4);
    asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(w[4 * j]), "r"(w[4 * j + 1]),
                 "r"(w[4 * j + 2]), "r"(w[4 * j + 3])
                 : "memory");
  }
}

template <int KWORDS>
__device__ __forceinline__ void store_packed_staged(uint8_t* out_tile, unsigned long long pitch_bytes,
                                                    uint32_t row0, uint32_t rows_total, uint32_t col_byte0,
                                                    uint32_t row_bytes_total, const uint32_t (&pk)[KWORDS],
                                                    uint32_t stage, uint32_t lane, bool add_f32 = false) {
  const uint32_t wsw = (lane >> 1) & 3u;  // swizzle of the row this lane writes
#pragma unroll
  for (int g = 0; g < KWORDS / 16; ++g) {  // groups of 64 bytes per row
#pragma unroll
    for (uint32_t j = 0; j < 4; ++j) {
      const uint32_t addr = stage + lane * 64u + ((j ^ wsw) << 4);
      asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(pk[g * 16 + 4 * j]),
                   "r"(pk[g * 16 + 4 * j + 1]), "r"(pk[g * 16 + 4 * j + 2]), "r"(pk[g * 16 + 4 * j + 3])
                   : "memory");
    }
    __syncwarp();
#pragma unroll
    for (uint32_t i = 0; i < 4; ++i) {
      const uint32_t r = i * 8u + (lane >> 2), seg = lane & 3u;
      uint32_t x0, x1, x2, x3;
      const uint32_t addr = stage + r * 64u + ((seg ^ ((r >> 1) & 3u)) << 4);
      asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];" : "=r"(x0), "=r"(x1), "=r"(x2), "=r"(x3) : "r"(addr) : "memory");
      const uint32_t cb = col_byte0 + static_cast<uint32_t>(g) * 64u + seg * 16u;
      if (row0 + r < rows_total && cb < row_bytes_total) {
        uint4* dst = reinterpret_cast<uint4*>(out_tile + static_cast<unsigned long long>(row0 + r) * pitch_bytes + cb);
        if (add_f32) {  // a later generation of an f32 tile: add to what the earlier ones stored
          const uint4 old = *dst;
          x0 = __float_as_uint(__uint_as_float(old.x) + __uint_as_float(x0));
          x1 = __float_as_uint(__uint_as_float(old.y) + __uint_as_float(x1));
          x2 = __float_as_uint(__uint_as_float(old.z) + __uint_as_float(x2));
          x3 = __float_as_uint(__uint_as_float(old.w) + __uint_as_float(x3));
        }
        *dst = make_uint4(x0, x1, x2, x3);
      }
    }
    __syncwarp();
  }
}

// -------------------------------------------------------------- producer
// One thread streams ONE operand (A or B) of every tile of this CTA into the stage ring.
// The two operands have a producer warp each, so the per-stage issue cost (barrier wait,
// expect-tx arrive, TMA issue) of one never delays the other.
//   PAIR: both CTAs of the pair signal CTA 0's `full` barriers; only CTA 0's producers
//   arrive on them (with the byte count of both CTAs), CTA 1's just issue their loads.
template <int BN, bool SWIGLU, bool PAIR, int MH, bool IS_A>
__device__ __forceinline__ void producer_role(const TcParams& p, const OperandLoad& o,
                                              const CUtensorMap* map0, const CUtensorMap* map1,
                                              SmemTail* tail, uint32_t smem_operand, uint32_t rank,
                                              uint32_t kb_lo, uint32_t kb_hi,
                                              uint32_t first_tile, uint32_t tile_step,
                                              const TileCoord& first_tc, uint32_t code) {
  using Cfg = TileCfg<BN, PAIR, MH>;
  constexpr int kStages = Cfg::kStages;
  constexpr uint32_t kStageBytes = IS_A ? Cfg::kStageA : Cfg::kStageB;
  constexpr uint32_t kKbBytes = IS_A ? Cfg::kStageA1 : Cfg::kStageB1;    // one k-block of this operand
  constexpr uint32_t kKbPerStage = Cfg::kKbPerStage;
  constexpr uint32_t kOutCols = SWIGLU ? BN / 2 : BN;
  volatile uint32_t* abort_flag = &tail->abort_flag;
  const uint32_t my_bytes = o.boxes * o.box_bytes;
  const uint32_t full0 = PAIR ? mapa_shared(smem_u32(&tail->full[0]), 0u) : smem_u32(&tail->full[0]);
  uint32_t s = 0, ph = 0, issued = 0;
  bool ok = true;
  for (uint32_t t = first_tile; ok && t < p.num_tiles; t += tile_step) {
    const TileCoord tc = t == first_tile ? first_tc : decode_tile(p, t);
    const uint32_t b2 = tc.batch % p.bdim2;
    const uint32_t tmp = tc.batch / p.bdim2;
    const uint32_t b1 = tmp % p.bdim1;
    const uint32_t b0 = tmp / p.bdim1;
    const int32_t c_b2 = static_cast<int32_t>(b2 * o.bmul[2]);
    const int32_t c_b1 = static_cast<int32_t>(b1 * o.bmul[1]);
    const int32_t c_b0 = static_cast<int32_t>(b0 * o.bmul[0]);
    int32_t mn0;
    if (IS_A) mn0 = static_cast<int32_t>(tc.mt * (PAIR ? 256u * MH : 128u) + rank * 128u * MH);
    else if (PAIR) mn0 = static_cast<int32_t>(SWIGLU ? tc.nt * 128u : tc.nt * 256u + rank * 128u);
    else mn0 = static_cast<int32_t>(tc.nt * kOutCols);
    for (uint32_t kb = kb_lo; kb < kb_hi; kb += kKbPerStage) {
      ok = wait_bounded(smem_u32(&tail->empty[s]), ph ^ 1u, abort_flag, p.status, code);
      if (!ok) break;
      const uint32_t bar = full0 + s * 8u;
      const uint32_t n_kb = kKbPerStage == 1u ? 1u : min(kKbPerStage, kb_hi - kb);   // k-blocks this stage holds
      if (!PAIR) mbar_arrive_expect_tx_relaxed(bar, my_bytes * n_kb);
      else if (rank == 0) mbar_arrive_expect_tx_relaxed(smem_u32(&tail->full[s]), 2u * my_bytes * n_kb);
#pragma unroll
      for (uint32_t h = 0; h < kKbPerStage; ++h) {   // the k-blocks of this stage
      if (h >= n_kb) break;
      const int32_t k0 = static_cast<int32_t>((kb + h) * p.bk);
      uint32_t dst = smem_operand + s * kStageBytes + h * kKbBytes;
      for (uint32_t i = 0; i < o.boxes; ++i, dst += o.box_bytes) {
        const CUtensorMap* mp = map0;
        uint32_t j = i;
        if (!IS_A && SWIGLU && !PAIR && i >= o.boxes / 2) { mp = map1; j = i - o.boxes / 2; }
        const int32_t mn = mn0 + static_cast<int32_t>(j * o.box_mn);
        int32_t c0, c1, c2, c3, c4;
        if (!o.mn_major) { c0 = k0; c1 = mn; c2 = c_b2; c3 = c_b1; c4 = c_b0; }
        else if (!o.slab_dim) { c0 = mn; c1 = k0; c2 = c_b2; c3 = c_b1; c4 = c_b0; }
        else { c0 = 0; c1 = k0; c2 = mn / static_cast<int32_t>(o.inner); c3 = c_b2; c4 = c_b1; }
        if (PAIR) tma_load_5d_pair(dst, mp, bar, c0, c1, c2, c3, c4);
        else tma_load_5d(dst, mp, bar, c0, c1, c2, c3, c4);
      }
      }
      ++issued;
      if (++s == kStages) { s = 0; ph ^= 1u; }
    }
  }
  if (*abort_flag && IS_A && rank == 0) {
    // Let copies already issued land before this CTA's shared memory goes away.  CTA 0's
    // `full` barriers count the bytes of both operands (and of both CTAs of a pair).
    const uint32_t first = issued > static_cast<uint32_t>(kStages) ? issued - kStages : 0u;
    for (uint32_t j = first; j < issued; ++j)
      wait_drain(smem_u32(&tail->full[j % kStages]), (j / kStages) & 1u);
  }
}

// -------------------------------------------------------------- the kernel
// PAIR = false: one CTA per 128 x BN tile.
// PAIR = true : two CTAs on neighbouring SMs share a 256 x 256 tile through `cta_group::2`
//   MMAs.  Each CTA stages its own 128 rows of A and its own 128 columns of B (two thirds of
//   the L2->SM traffic of two 1-CTA tiles, and 32 KB stages so six fit), CTA 0 issues
//   the MMAs, each CTA's TMEM receives its 128 rows x 256 columns of the accumulator and each
//   CTA runs its own epilogue.  Loads are plain per-CTA TMA loads; CTA 0's commits signal
//   `empty` / `tmem_full` in both CTAs.  With SWIGLU, CTA 0 stages the gate weights and CTA 1
//   the up weights of the same 128 output columns.
// p.k_splits > 1 (the one-CTA form without SwiGLU; one tile per cluster): a problem with too few
//   tiles to occupy the SMs runs as clusters of k_splits CTAs per tile, each taking a
//   slice of K into its own accumulator.  The slices then share the epilogue: each owns
//   1/k_splits of the tile's 32-column chunks, writes the chunks it does not own as f32 into its
//   idle operand ring, and after a cluster barrier adds to its own chunks what the other slices
//   hold for them, read through distributed shared memory in a fixed order (so the sum does not
//   depend on timing), and stores them.
template <int KIND, int BN, int OUT, bool SWIGLU, bool PAIR, int MH>
__global__ void __launch_bounds__(threads_for(MH), 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
               const __grid_constant__ CUtensorMap map_b2, const __grid_constant__ CUtensorMap map_out,
               const TcParams p) {
  static_assert(MH == 1 || (PAIR && BN == 256), "two M-halves per CTA exist for the pair form only");
  using Cfg = TileCfg<BN, PAIR, MH>;
  constexpr int kStages = Cfg::kStages;
  constexpr int kStageA = Cfg::kStageA;
  constexpr int kStageB = Cfg::kStageB;
  constexpr int CG = PAIR ? 2 : 1;
  constexpr bool kIntAcc = (KIND == KIND_I8);
  // Only the f32 path (split TF32 operands) cuts a tile's K into accumulator generations; for
  // every other kind the generation loops below run once and fold away at compile time.
  constexpr bool kGenerations = (KIND == KIND_TF32);
  constexpr int kOutCols = SWIGLU ? BN / 2 : BN;  // output columns per tile
  constexpr uint32_t kTileM = PAIR ? 256u * MH : 128u;
  constexpr bool kSplitCapable = (!PAIR && !SWIGLU && !kGenerations);   // may run with p.k_splits > 1

  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_u32 = smem_u32(smem_raw);
  const uint32_t base_u32 = (raw_u32 + 1023u) & ~1023u;
  uint8_t* smem = smem_raw + (base_u32 - raw_u32);
  // [operand ring][epilogue staging: 2 KB per epilogue warp, 1 KB aligned][barriers and flags]
  SmemTail* tail = reinterpret_cast<SmemTail*>(smem + kStages * (kStageA + kStageB) + Cfg::kEpiWarps * Cfg::kEpiStage);
  const uint32_t smem_a = base_u32;
  const uint32_t smem_b = base_u32 + kStages * kStageA;

  const uint32_t warp = threadIdx.x >> 5;
  const uint32_t lane = threadIdx.x & 31u;
  // (Forms that never run with K slices keep all of this at its compile-time value.)
  const uint32_t k_splits = kSplitCapable ? p.k_splits : 1u;
  const uint32_t crank = (PAIR || kSplitCapable) ? cluster_ctarank() : 0u;   // 0 when launched without clusters
  const uint32_t rank = PAIR ? crank : 0u;                                   // CTA of the pair
  const uint32_t slice = kSplitCapable ? crank : 0u;                         // K slice (0 unless k_splits > 1)
  const uint32_t first_tile = PAIR ? (blockIdx.x >> 1) : (kSplitCapable ? blockIdx.x / k_splits : blockIdx.x);
  // K slices: exactly one tile per cluster (the slices meet at one cluster barrier).
  const uint32_t tile_step = PAIR ? (gridDim.x >> 1) : (k_splits > 1u ? p.num_tiles : gridDim.x);
  uint32_t kb_lo = 0, kb_hi = p.k_blocks;
  if (k_splits > 1u) {
    kb_lo = slice * p.kb_per_split;
    kb_hi = min(kb_lo + p.kb_per_split, p.k_blocks);
  }
  volatile uint32_t* abort_flag = &tail->abort_flag;

  if (threadIdx.x == 0) {
    prefetch_tensormap(&map_a);   // first: the descriptor fetch runs under the rest of the set-up
    prefetch_tensormap(&map_b);
    if constexpr (SWIGLU) prefetch_tensormap(&map_b2);
    prefetch_tensormap(&map_out);
    for (int s = 0; s < kStages; ++s) {
      mbar_init(smem_u32(&tail->full[s]), 2);   // one arrive(+tx) per operand producer
      mbar_init(smem_u32(&tail->empty[s]), 1);  // one commit arrive (delivered to both CTAs of a pair)
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(smem_u32(&tail->tmem_full[i]), 1);
      mbar_init(smem_u32(&tail->tmem_empty[i]), 4 * CG * epi_col_groups(MH));  // one arrive per epilogue warp
    }
    mbar_init(smem_u32(&tail->drain), 1);
    tail->abort_flag = 0;
    fence_barrier_init();
  }
  if (warp == 1) {
    tmem_alloc<CG>(smem_u32(&tail->tmem_base), Cfg::kTmemCols);
    tmem_relinquish<CG>();
  }
  tc_fence_before_sync();
  // One barrier for both purposes: the CTA's own barriers and TMEM address are visible to all
  // its threads, and (pair forms) the peer's barriers exist before anything signals them.  The
  // first tile's coordinates, which need nothing from anybody, are worked out between the
  // arrive and the wait.
  if constexpr (PAIR) cluster_arrive();
  const TileCoord first_tc = decode_tile(p, first_tile < p.num_tiles ? first_tile : 0u);
  if constexpr (PAIR) cluster_wait();
  else __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t*>(&tail->tmem_base);
  const uint32_t code_base = 0x80000000u | ((blockIdx.x & 0xFFFFu) << 4);
  // Everything above touched only this CTA's shared memory and TMEM, so under a programmatic
  // dependent launch it ran while the previous kernel of the stream was finishing.  From here
  // on global memory is read and written: wait for that kernel, then let the next one start
  // its own set-up as soon as SMs free up.
  grid_dependency_wait();
  grid_launch_dependents();

  if (warp == 0) {
    // ------------------------------------------------------------ producer of A
    if (lane == 0)
      producer_role<BN, SWIGLU, PAIR, MH, true>(p, p.a, &map_a, &map_a, tail, smem_a, rank, kb_lo, kb_hi,
                                                first_tile, tile_step, first_tc, code_base | 1u);
    __syncwarp();
  } else if (warp == 6) {
    // ------------------------------------------------------------ producer of B
    if (lane == 0) {
      const CUtensorMap* m0 = (PAIR && SWIGLU && rank == 1) ? &map_b2 : &map_b;
      producer_role<BN, SWIGLU, PAIR, MH, false>(p, p.b, m0, &map_b2, tail, smem_b, rank, kb_lo, kb_hi,
                                                 first_tile, tile_step, first_tc, code_base | 5u);
    }
    __syncwarp();
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer (CTA 0 of a pair)
    if (lane == 0 && rank == 0) {
      uint32_t s = 0, ph = 0, lt = 0;
      bool ok = true;
      // This one thread's instruction stream bounds the main loop (with loads switched off the
      // kernel takes the same number of cycles), so the loop is kept to: one barrier wait, one
      // fence, one asm block of four MMAs per accumulator, one commit.  Everything else -- the
      // descriptor bases per stage, the constant high words -- lives in registers.  (A second
      // issuing warp for the second accumulator of the 512x256 form measured no further gain.)
      const uint32_t a_hi = p.a.desc_hi, b_hi = p.b.desc_hi;
      const uint32_t a_step = p.a.kstep16, b_step = p.b.kstep16;
      // (A CTA of a cluster other than rank 0 sees its own shared memory at addresses that carry
      // the rank above bit 24; the descriptor's address field takes the offset within the CTA.)
      const uint32_t a_lo0 = ((smem_a & 0x3FFFFu) >> 4) | p.a.desc_lo, b_lo0 = ((smem_b & 0x3FFFFu) >> 4) | p.b.desc_lo;
      const uint32_t idesc = p.idesc, k_blocks = kb_hi;
      uint32_t a_lo = a_lo0, b_lo = b_lo0;  // descriptor low words of the current stage
      uint32_t full_bar = smem_u32(&tail->full[0]), empty_bar = smem_u32(&tail->empty[0]);
      for (uint32_t t = first_tile; ok && t < p.num_tiles; t += tile_step) {
      uint32_t kb0 = kb_lo;
      do {
        // One accumulator generation: the whole tile, or (long f32 products) a run of k_gen
        // k-blocks whose sum the epilogue adds to the output before the next run starts afresh.
        // MH == 1: the two accumulators alternate between generations (double buffer).
        // MH == 2: one generation fills both, accumulator h holding M-half h.
        const uint32_t acc = MH == 2 ? 0u : (lt & 1u);
        const uint32_t acc_ph = MH == 2 ? (lt & 1u) : ((lt >> 1) & 1u);
        const uint32_t d_tmem = tmem_base + acc * BN;
        const uint32_t kb_end = kGenerations ? generation_end(p, kb0) : k_blocks;
        for (uint32_t kb = kb0; kb < kb_end; kb += Cfg::kKbPerStage) {
          ok = wait_bounded(full_bar, ph, abort_flag, p.status, code_base | 3u);
          if (!ok) break;
          tc_fence_after_sync();
          if (kb == kb0) {
            // first write of the accumulator: the epilogue must have drained it
            ok = wait_bounded(smem_u32(&tail->tmem_empty[acc]), acc_ph ^ 1u, abort_flag, p.status,
                              code_base | 2u);
            if (!ok) break;
            tc_fence_after_sync();
            umma_x4<KIND, CG>(d_tmem, a_lo, a_hi, a_step, b_lo, b_hi, b_step, idesc, 0u);
            if constexpr (MH == 2) {
              ok = wait_bounded(smem_u32(&tail->tmem_empty[1]), acc_ph ^ 1u, abort_flag, p.status,
                                code_base | 2u);
              if (!ok) break;
              tc_fence_after_sync();
              umma_x4<KIND, CG>(d_tmem + BN, a_lo + (kHalfA >> 4), a_hi, a_step, b_lo, b_hi, b_step, idesc, 0u);
            }
          } else {
            umma_x4<KIND, CG>(d_tmem, a_lo, a_hi, a_step, b_lo, b_hi, b_step, idesc, 1u);
            if constexpr (MH == 2)
              umma_x4<KIND, CG>(d_tmem + BN, a_lo + (kHalfA >> 4), a_hi, a_step, b_lo, b_hi, b_step, idesc, 1u);
          }
          if constexpr (Cfg::kKbPerStage == 2) {   // the stage's second k-block (absent at an odd end of K)
            if (kb + 1u < kb_end)
              umma_x4<KIND, CG>(d_tmem, a_lo + (Cfg::kStageA1 >> 4), a_hi, a_step, b_lo + (Cfg::kStageB1 >> 4), b_hi, b_step, idesc, 1u);
          }
          // frees the stage (in both CTAs of a pair) when these MMAs retire
          if constexpr (PAIR) umma_commit_2cta(empty_bar, 3);
          else umma_commit_1cta(empty_bar);
          if (++s == kStages) {
            s = 0; ph ^= 1u;
            a_lo = a_lo0; b_lo = b_lo0;
            full_bar = smem_u32(&tail->full[0]); empty_bar = smem_u32(&tail->empty[0]);
          } else {
            a_lo += kStageA >> 4; b_lo += kStageB >> 4;
            full_bar += 8u; empty_bar += 8u;
          }
        }
        if (!ok) break;
        // the accumulator(s) are complete once every MMA issued so far has retired
#pragma unroll
        for (uint32_t h = 0; h < static_cast<uint32_t>(MH); ++h) {
          if constexpr (PAIR) umma_commit_2cta(smem_u32(&tail->tmem_full[acc + h]), 3);
          else umma_commit_1cta(smem_u32(&tail->tmem_full[acc + h]));
        }
        ++lt;
        kb0 = kb_end;
      } while (kGenerations && kb0 < k_blocks);
      }
      if (*abort_flag) {
        if constexpr (PAIR) umma_commit_2cta(smem_u32(&tail->drain), 1);
        else umma_commit_1cta(smem_u32(&tail->drain));
        wait_drain(smem_u32(&tail->drain), 0u);
      }
    }
    __syncwarp();
  } else {
    // ------------------------------------------------------------ epilogue (warps 2..5, and 7..18 when MH == 2)
    // Groups of four consecutive epilogue warps cover the four TMEM lane quadrants (warp % 4).
    // MH == 2: groups 0,1 drain accumulator 0 (left and right half of its columns), groups 2,3
    // accumulator 1.
    constexpr uint32_t kColGroups = epi_col_groups(MH);
    const uint32_t q = warp & 3u;                         // TMEM lane quadrant this warp may read
    const uint32_t e_group = (warp < 6u ? warp - 2u : warp - 3u) >> 2;
    const uint32_t half = e_group / kColGroups;           // which M-half (accumulator)
    const uint32_t col_group = e_group % kColGroups;      // which share of the output columns
    constexpr uint32_t kChunks = kOutCols / 32 / kColGroups;
    const uint32_t e_warp = warp < 6u ? warp - 2u : warp - 3u;  // index among the epilogue warps
    const uint32_t stage_buf = base_u32 + kStages * (kStageA + kStageB) + e_warp * Cfg::kEpiStage;
    constexpr bool kStaged = (OUT == OUT_F32 || OUT == OUT_I32 || OUT == OUT_BF16 || OUT == OUT_F16);
    const uint32_t osz = OutBytes<OUT>::value;
    const uint32_t tmem_empty0 =
        PAIR ? mapa_shared(smem_u32(&tail->tmem_empty[0]), 0u) : smem_u32(&tail->tmem_empty[0]);
    uint32_t lt = 0;
    bool epi_ok = true;
    [[maybe_unused]] bool split_synced = false;   // this warp has been through the K-slice barrier
    for (uint32_t t = first_tile; epi_ok && t < p.num_tiles; t += tile_step) {
    // Where this tile's rows go: worked out BEFORE the wait for the accumulator (these divisions
    // and 64-bit products measured ~800 cycles, which were exposed after the wait).
    const TileCoord tc = t == first_tile ? first_tc : decode_tile(p, t);
    const uint32_t row = tc.mt * kTileM + rank * 128u * MH + half * 128u + q * 32u + lane;
    const uint32_t n0 = tc.nt * kOutCols;
    const bool row_ok = row < p.M;
    uint8_t* out_row = static_cast<uint8_t*>(p.out) +
                       (static_cast<unsigned long long>(tc.batch) * p.out_batch_stride +
                        static_cast<unsigned long long>(row) * p.ldc + n0) * osz;
    uint8_t* out_tile = static_cast<uint8_t*>(p.out) +
                        static_cast<unsigned long long>(tc.batch) * p.out_batch_stride * osz;
    uint32_t kb0 = 0;
    do {   // one pass per accumulator generation (a single pass unless kGenerations)
      const bool later_gen = kGenerations && kb0 != 0;   // add this generation's sums to the stored ones
      const uint32_t acc = MH == 2 ? half : (lt & 1u);
      const uint32_t acc_ph = MH == 2 ? (lt & 1u) : ((lt >> 1) & 1u);
      bool ok = wait_bounded(smem_u32(&tail->tmem_full[acc]), acc_ph, abort_flag, p.status,
                             code_base | 4u);
      ok = __all_sync(0xFFFFFFFFu, ok);
      if (!ok) { epi_ok = false; break; }
      tc_fence_after_sync();
      const uint32_t t_row = tmem_base + acc * BN + ((q * 32u) << 16);
      // Scale and bias of chunk c, applied to the finished sums.
      auto finish_chunk = [&](uint32_t c, uint32_t (&v)[32]) {
        if constexpr (!SWIGLU && !kIntAcc) {
          if (p.alpha != 1.0f) {
#pragma unroll
            for (int j = 0; j < 32; ++j) v[j] = __float_as_uint(__uint_as_float(v[j]) * p.alpha);
          }
          if constexpr (OUT == OUT_F32 || OUT == OUT_BF16 || OUT == OUT_F16) {
            if (p.bias != nullptr && !later_gen) {  // uniform over the grid; once per output
              // Lane l fetches the bias of column c*32 + l; the 32 values go round by shuffle.
              const uint32_t bcol = n0 + c * 32u + lane;
              const float mine = bcol < p.N ? load_bias<OUT>(p.bias, static_cast<long long>(bcol) * p.bias_stride) : 0.0f;
              const bool each = (p.bias_flags == HODU_B200_LINEAR_ROUND_EACH_OP);
#pragma unroll
              for (int j = 0; j < 32; ++j) {
                float x = __uint_as_float(v[j]);
                if (each) x = round_to_storage<OUT>(x);
                v[j] = __float_as_uint(x + __shfl_sync(0xFFFFFFFFu, mine, j));
              }
            }
          }
        }
      };
      // Loads chunk c of this warp's rows from TMEM and applies the epilogue arithmetic; v then
      // holds the 32 final values (floats, or raw s32).
      auto load_chunk = [&](uint32_t c, uint32_t (&v)[32]) {
        tmem_ld_32x32(t_row + c * 32u, v);
        if constexpr (SWIGLU) {
          uint32_t u[32];
          tmem_ld_32x32(t_row + kOutCols + c * 32u, u);
          tmem_wait_ld();
          const bool each = (p.swiglu_flags == HODU_B200_SWIGLU_ROUND_EACH_OP);
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            float g = __uint_as_float(v[j]), up = __uint_as_float(u[j]);
            if (each) {
              g = round_to_storage<OUT>(g);
              up = round_to_storage<OUT>(up);
              const float sg = round_to_storage<OUT>(silu_f32(g));
              v[j] = __float_as_uint(sg * up);
            } else {
              v[j] = __float_as_uint(silu_f32(g) * up);
            }
          }
        } else {
          tmem_wait_ld();
          finish_chunk(c, v);
        }
      };
      const bool staged = kStaged && (p.out_vec_ok & 1u);  // uniform over the warp
      // Converts the 32 final values of chunk c and stores them (through the warp's 2 KB staging
      // buffer when the output rows allow 16-byte stores).
      auto store_chunk = [&](uint32_t c, uint32_t (&v)[32]) {
        const uint32_t col = n0 + c * 32u;
        if (staged) {
          if constexpr (kStaged) {
            uint32_t pk[ChunkWords<OUT>::value];
            pack_chunk<OUT>(v, pk);
            store_packed_staged<ChunkWords<OUT>::value>(out_tile, p.ldc * osz, row - lane, p.M, col * osz,
                                                        p.N * osz, pk, stage_buf, lane,
                                                        OUT == OUT_F32 && later_gen);
          }
        } else if (row_ok) {
          const int ncols = static_cast<int>(min(32u, p.N - col));
          if constexpr (OUT == OUT_F32 && kGenerations) {
            if (later_gen) {  // the lane that stored these elements adds the new generation to them
              const float* old = reinterpret_cast<const float*>(out_row + static_cast<size_t>(c) * 32u * osz);
#pragma unroll
              for (int j = 0; j < 32; ++j)
                if (j < ncols) v[j] = __float_as_uint(old[j] + __uint_as_float(v[j]));
            }
          }
          store_row_chunk<OUT>(out_row + static_cast<size_t>(c) * 32u * osz, v, ncols,
                               (p.out_vec_ok & 1u) != 0u);
        }
      };
      // The 512x256 form cannot hide its epilogue behind the next tile, so for 2-byte outputs
      // the warp first pulls ALL its chunks out of TMEM into registers (already packed), hands
      // the accumulator back to the MMA issuer, and only then does the global stores.
      constexpr bool kEarlyRelease = MH == 2 && (OUT == OUT_BF16 || OUT == OUT_F16);
      bool released = false;
      // SwiGLU in the op-by-op rounding form first rounds gate and up to the storage dtype, so
      // the two can leave TMEM as packed 16-bit pairs and silu / product run after the release.
      const bool swiglu_split = SWIGLU && p.swiglu_flags == HODU_B200_SWIGLU_ROUND_EACH_OP;
      // A CTA's LAST tile has no successor waiting for the accumulator, so it takes the chunk by
      // chunk path below instead: its stores start after the first TMEM load rather than after
      // the last, which shortens the tail of the launch (all of it, when every CTA has one tile).
      const bool last_tile = t + tile_step >= p.num_tiles;
      // ... and when the output has a tensor map, through TMA: by now every MMA of this CTA has
      // retired, so the operand ring is idle and each epilogue warp takes 8 KB of it as staging.
      // The warp converts a chunk, writes it there, and one lane hands it to the TMA unit, which
      // streams the stores at the rate the SM's store port allows while the warp is already
      // converting the next chunk; tails of M and N are clipped by the tensor map.
      bool tail_tma = false;
      if constexpr (kStaged) tail_tma = staged && last_tile && p.out_tma != 0u && !(kGenerations && p.k_gen < p.k_blocks);
      bool split_tile = false;
      if constexpr (kSplitCapable) split_tile = k_splits > 1u;
      if (split_tile) {
        if constexpr (kSplitCapable) {
          // K slices of one tile in the CTAs of this cluster: see the kernel's header.
          static_assert(kChunks * 16384u <= static_cast<uint32_t>(kStages * (kStageA + kStageB)),
                        "the partial sums of a tile must fit the operand ring");
          const uint32_t per = kChunks / k_splits;             // chunks each slice owns
          // A chunk of partial sums (128 rows x 32 columns of f32, 16 KB) lies as eight 2 KB planes,
          // plane j holding columns 4j..4j+3 of every row, 16 bytes per row: a warp's 32 rows are
          // 512 contiguous bytes of a plane, both for the local stores and for the reads from
          // another CTA (which the cluster network serves per contiguous run, not per lane).
          const uint32_t my_row = (q * 32u + lane) * 16u;
          auto dump_chunk = [&](uint32_t c, const uint32_t (&v)[32]) {
            const uint32_t dst = base_u32 + c * 16384u + my_row;
#pragma unroll
            for (uint32_t j = 0; j < 8; ++j)
              asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(dst + j * 2048u), "r"(v[4 * j]),
                           "r"(v[4 * j + 1]), "r"(v[4 * j + 2]), "r"(v[4 * j + 3])
                           : "memory");
          };
          // 1. The chunks other slices own: accumulator -> this CTA's idle operand ring.  Two at a
          // time, so that the TMEM load of one runs under the stores of the other.
          const uint32_t n_valid = min(kChunks, (p.N - n0 + 31u) / 32u);   // chunks inside N (uniform)
          const uint32_t own_lo = slice * per, own_hi = own_lo + per;
          auto foreign = [&](uint32_t i) { return i < own_lo ? i : i + per; };   // i-th chunk not owned
          const uint32_t n_foreign = n_valid <= own_lo ? n_valid : (n_valid <= own_hi ? own_lo : n_valid - per);
#pragma unroll 1
          for (uint32_t i = 0; i < n_foreign; i += 2u) {
            uint32_t va[32], vb[32];
            const uint32_t ca = foreign(i), cb = foreign(i + 1u);
            const bool two = i + 1u < n_foreign;
            tmem_ld_32x32(t_row + ca * 32u, va);
            tmem_wait_ld();
            if (two) tmem_ld_32x32(t_row + cb * 32u, vb);
            dump_chunk(ca, va);
            if (two) {
              tmem_wait_ld();
              dump_chunk(cb, vb);
            }
          }
          cluster_sync_all();   // every slice's partial sums are in place (and visible cluster-wide)
          split_synced = true;
          // 2. The chunks this slice owns: own accumulator plus what the other slices hold, always
          // added in the same order (own, then the slices after this one, cyclically), three
          // slices per round of reads.  The first round for the next chunk is issued before the
          // current chunk is converted and stored.
          uint4 x[3][8];
          auto fetch_remote = [&](uint32_t c, uint32_t t0) {   // slices slice + t0 .. slice + t0 + 2
#pragma unroll
            for (uint32_t i = 0; i < 3; ++i) {
              if (t0 + i < k_splits) {
                const uint32_t s2 = (slice + t0 + i) & (k_splits - 1u);
                const uint32_t src = mapa_shared(base_u32 + c * 16384u + my_row, s2);
#pragma unroll
                for (uint32_t j = 0; j < 8; ++j) x[i][j] = ld_cluster_v4(src + j * 2048u);
              }
            }
          };
          const uint32_t own_end = min(own_hi, n_valid);
          if (own_lo < own_end) fetch_remote(own_lo, 1u);
#pragma unroll 1
          for (uint32_t c = own_lo; c < own_end; ++c) {
            uint32_t v[32];
            tmem_ld_32x32(t_row + c * 32u, v);
            tmem_wait_ld();
#pragma unroll 1
            for (uint32_t t0 = 1; t0 < k_splits; t0 += 3u) {
#pragma unroll
              for (uint32_t i = 0; i < 3; ++i) {
                if (t0 + i < k_splits) {
#pragma unroll
                  for (uint32_t j = 0; j < 8; ++j) {
                    const uint32_t w[4] = {x[i][j].x, x[i][j].y, x[i][j].z, x[i][j].w};
#pragma unroll
                    for (uint32_t e = 0; e < 4; ++e) {
                      if constexpr (kIntAcc) v[4 * j + e] += w[e];
                      else v[4 * j + e] = __float_as_uint(__uint_as_float(v[4 * j + e]) + __uint_as_float(w[e]));
                    }
                  }
                }
              }
              if (t0 + 3u < k_splits) fetch_remote(c, t0 + 3u);
              else if (c + 1u < own_end) fetch_remote(c + 1u, 1u);
            }
            finish_chunk(c, v);
            store_chunk(c, v);
          }
        }
      } else if (tail_tma) {
        if constexpr (kStaged) {
          constexpr uint32_t kWords = ChunkWords<OUT>::value;      // 16 or 32 words per lane and chunk
          constexpr uint32_t kChunkBytes = kWords * 4u * 32u;      // 2 KB or 4 KB
          constexpr uint32_t kBufs = 8192u / kChunkBytes;
          const uint32_t ring = base_u32 + e_warp * 8192u;
          const uint32_t row0 = row - lane;
          uint32_t n_issued = 0;
#pragma unroll 1
          for (uint32_t c = col_group * kChunks; c < (col_group + 1u) * kChunks; ++c) {
            const uint32_t col = n0 + c * 32u;
            if (col >= p.N) break;  // uniform over the warp
            uint32_t v[32];
            load_chunk(c, v);
            uint32_t pk[kWords];
            pack_chunk<OUT>(v, pk);
            const uint32_t buf = ring + (n_issued % kBufs) * kChunkBytes;
            if (n_issued >= kBufs) {   // the store that last read this buffer must be done with it
              if (lane == 0) bulk_wait_group_read<static_cast<int>(kBufs) - 1>();
              __syncwarp();
            }
#pragma unroll
            for (uint32_t g = 0; g < kWords / 16u; ++g) stage_write_row64(buf + g * 2048u, lane, &pk[16u * g]);
            fence_proxy_async_smem();
            __syncwarp();
            if (lane == 0 && row0 < p.M) {
#pragma unroll
              for (uint32_t g = 0; g < kWords / 16u; ++g) {
                const uint32_t cg = col + g * (64u / OutBytes<OUT>::value);
                if (cg < p.N)
                  tma_store_3d(&map_out, buf + g * 2048u, static_cast<int32_t>(cg), static_cast<int32_t>(row0),
                               static_cast<int32_t>(tc.batch));
              }
            }
            if (lane == 0) bulk_commit_group();
            ++n_issued;
          }
          if (lane == 0) bulk_wait_group_read<0>();   // the ring may go away once the stores have read it
          __syncwarp();
        }
      } else if (kEarlyRelease && staged && (!SWIGLU || swiglu_split) && !last_tile) {
        uint32_t pk[kChunks][16];
        [[maybe_unused]] uint32_t pu[SWIGLU ? kChunks : 1][16];
#pragma unroll
        for (uint32_t i = 0; i < kChunks; ++i) {
          const uint32_t c = col_group * kChunks + i;
          if (n0 + c * 32u < p.N) {
            uint32_t v[32];
            if constexpr (SWIGLU) {
              tmem_ld_32x32(t_row + c * 32u, v);
              tmem_wait_ld();
              pack_chunk<OUT>(v, *reinterpret_cast<uint32_t(*)[ChunkWords<OUT>::value]>(&pk[i]));
              tmem_ld_32x32(t_row + kOutCols + c * 32u, v);
              tmem_wait_ld();
              pack_chunk<OUT>(v, *reinterpret_cast<uint32_t(*)[ChunkWords<OUT>::value]>(&pu[i]));
            } else {
              load_chunk(c, v);
              pack_chunk<OUT>(v, *reinterpret_cast<uint32_t(*)[ChunkWords<OUT>::value]>(&pk[i]));
            }
          }
        }
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive_cluster_addr(tmem_empty0 + acc * 8u);
        released = true;
        if constexpr (SWIGLU) {
#pragma unroll
          for (uint32_t i = 0; i < kChunks; ++i) {
#pragma unroll
            for (int j = 0; j < 16; ++j) {
              float g0, g1, u0, u1;
              unpack_pair<OUT>(pk[i][j], g0, g1);
              unpack_pair<OUT>(pu[i][j], u0, u1);
              const float r0 = round_to_storage<OUT>(silu_f32(g0)) * u0;
              const float r1 = round_to_storage<OUT>(silu_f32(g1)) * u1;
              pk[i][j] = pack_pair<OUT>(r0, r1);
            }
          }
        }
#pragma unroll
        for (uint32_t i = 0; i < kChunks; ++i) {
          const uint32_t c = col_group * kChunks + i;
          if (n0 + c * 32u < p.N)
            store_packed_staged<16>(out_tile, p.ldc * osz, row - lane, p.M, (n0 + c * 32u) * osz, p.N * osz,
                                    pk[i], stage_buf, lane);
        }
      } else {
#pragma unroll 1
        for (uint32_t c = col_group * kChunks; c < (col_group + 1u) * kChunks; ++c) {
          const uint32_t col = n0 + c * 32u;
          if (col >= p.N) break;  // uniform over the warp
          uint32_t v[32];
          load_chunk(c, v);
          store_chunk(c, v);
        }
      }
      if (!released) {
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) {
          if constexpr (PAIR) mbar_arrive_cluster_addr(tmem_empty0 + acc * 8u);
          else mbar_arrive(tmem_empty0 + acc * 8u);
        }
      }
      ++lt;
      kb0 = generation_end(p, kb0);
    } while (kGenerations && kb0 < p.k_blocks);
    }
    if constexpr (kSplitCapable) {
      // A warp that gave up before the K-slice barrier still owes the cluster its arrival.
      if (k_splits > 1u && !split_synced) cluster_sync_all();
    }
  }
  if constexpr (kSplitCapable) {
    // The warps without a share in the epilogue take part in the K-slice barrier here.
    if (k_splits > 1u && (warp < 2u || warp == 6u)) cluster_sync_all();
  }

  // A CTA of a pair may not leave (or free TMEM) while its peer can still read its shared
  // memory, signal its barriers or write its TMEM.
  tc_fence_before_sync();
  // ... and a K slice not while the others can still read its partial sums.
  // (A pair keeps the release form: its last remote mbarrier arrive must have landed before the
  // peer's shared memory can pass to another CTA.  K slices only READ each other's memory, and
  // every read has delivered its value before its thread arrives, so they meet without the
  // fence, which would first wait for the CTA's global stores to complete.)
  if constexpr (PAIR) cluster_sync_all();   // also a barrier over this CTA's own threads
  else if (k_splits > 1u) cluster_sync_all_relaxed();
  else __syncthreads();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc<CG>(tmem_base, Cfg::kTmemCols);
  }
}

// A wait that nothing satisfies: shows, without faulting or hanging anything, that a
// bounded wait gives up, records its code and lets the kernel return normally.
__global__ void wait_timeout_probe_kernel(uint32_t* status, uint64_t limit_ns) {
  __shared__ uint64_t bar;
  __shared__ uint32_t abort_flag;
  if (threadIdx.x == 0) {
    mbar_init(smem_u32(&bar), 1);
    abort_flag = 0;
    fence_barrier_init();
  }
  __syncthreads();
  if (threadIdx.x == 0)
    wait_bounded(smem_u32(&bar), 0u, &abort_flag, status, 0x80000000u | 7u, limit_ns);
  __syncthreads();
}

// -------------------------------------------------------------- host side
EncodeTiledFn encode_fn() { return tensor_map_encoder(); }

// Everything cuTensorMapEncodeTiled is given (swizzle, interleave, promotion and fill are fixed).
struct MapKey {
  uintptr_t base;
  uint64_t dims[5];
  uint64_t strides[4];
  uint32_t box[5];
  uint32_t esize;
  uint32_t kind;   // 0: operand map (5-D, 128-byte swizzle), 1: output map (3-D, 64-byte swizzle)
};
struct MapCacheEntry {
  bool used = false;
  MapKey key;
  CUtensorMap map;
};
constexpr int kMapCacheEntries = 32;
// Per thread: no lock, and a map encoded under one thread's current context is only reused there.
struct MapCache {
  MapCacheEntry e[kMapCacheEntries];
  int next = 0;
};
thread_local MapCache t_map_cache;
bool map_cache_get(const MapKey& key, CUtensorMap* out) {
  MapCache& c = t_map_cache;
  for (int i = 0; i < kMapCacheEntries; ++i) {
    if (c.e[i].used && memcmp(&c.e[i].key, &key, sizeof(MapKey)) == 0) {
      *out = c.e[i].map;
      return true;
    }
  }
  return false;
}
void map_cache_put(const MapKey& key, const CUtensorMap& map) {
  MapCache& c = t_map_cache;
  MapCacheEntry& slot = c.e[c.next];
  c.next = (c.next + 1) % kMapCacheEntries;
  slot.used = true;
  slot.key = key;
  slot.map = map;
}

struct OperandMap {
  bool mn_major = false;
  bool slab_dim = false;
  uint32_t bmul[3] = {0, 0, 0};
  CUtensorMap map;
};

struct BatchDims {
  int n = 0;
  int64_t size[kMaxBatchDims] = {1, 1, 1};      // outermost first
  int64_t a_stride[kMaxBatchDims] = {0, 0, 0};
  int64_t b_stride[kMaxBatchDims] = {0, 0, 0};
  int64_t b2_stride[kMaxBatchDims] = {0, 0, 0};
};

// Drops size-1 batch dims and merges neighbours that every operand walks with one stride.
bool collapse_batch(const Problem& pb, BatchDims* out) {
  int64_t size[16], as[16], bs[16], b2s[16];
  int n = 0;
  for (int d = 0; d < pb.batch_ndim; ++d) {
    if (pb.batch_shape[d] == 1) continue;
    size[n] = pb.batch_shape[d];
    as[n] = pb.a.bstride[d];
    bs[n] = pb.b.bstride[d];
    b2s[n] = pb.swiglu ? pb.b2.bstride[d] : 0;
    ++n;
  }
  int m = 0;
  for (int d = 0; d < n; ++d) {
    if (m > 0 && as[m - 1] == as[d] * size[d] && bs[m - 1] == bs[d] * size[d] &&
        b2s[m - 1] == b2s[d] * size[d]) {
      size[m - 1] *= size[d];
      as[m - 1] = as[d];
      bs[m - 1] = bs[d];
      b2s[m - 1] = b2s[d];
    } else {
      size[m] = size[d]; as[m] = as[d]; bs[m] = bs[d]; b2s[m] = b2s[d];
      ++m;
    }
  }
  if (m > kMaxBatchDims) return false;
  out->n = m;
  // right-align into the three slots (slot 2 is the fastest-varying batch dim)
  for (int d = 0; d < m; ++d) {
    const int slot = kMaxBatchDims - m + d;
    out->size[slot] = size[d];
    out->a_stride[slot] = as[d];
    out->b_stride[slot] = bs[d];
    out->b2_stride[slot] = b2s[d];
  }
  return true;
}

inline bool pitch_ok(int64_t s, int esize) {
  return s > 0 && (s * esize) % 16 == 0 && s * esize < (1ll << 40);
}
// Which matrix index of an operand is contiguous.  An operand is K-major when the
// K index has stride 1 and MN-major when the M (lhs) / N (rhs) index has; the
// other index must step by a multiple of 16 bytes for TMA.  K-major wins a tie.
// Returns 0 = K-major, 1 = MN-major, -1 = neither.
int classify_operand(const Operand& op, int esize, int64_t rows, int64_t cols, bool k_is_col) {
  const int64_t mn = k_is_col ? rows : cols;
  const int64_t kk = k_is_col ? cols : rows;
  const int64_t s_mn = k_is_col ? op.stride_r : op.stride_c;
  const int64_t s_k = k_is_col ? op.stride_c : op.stride_r;
  if ((s_k == 1 || kk == 1) && (mn == 1 || pitch_ok(s_mn, esize))) return 0;
  if ((s_mn == 1 || mn == 1) && (kk == 1 || pitch_ok(s_k, esize))) return 1;
  return -1;
}

// Builds the 5-D tensor map of one operand.  rows/cols: logical matrix extents; `k_is_col`
// says whether K is the column index (lhs) or the row index (rhs).
//   K-major : dims {K, MN, batch2, batch1, batch0}, box {128 B of K, tile_mn rows}.
//   MN-major: dims {MN, K, batch2, batch1, batch0}, box {128 B of MN, 128/esize rows of K}:
//             one box per 128-byte slab of the tile.
//   MN-major with `slabs_per_box` > 1 (needs MN % (128/esize) == 0 and at most two batch dims):
//             dims {128 B of MN, K, MN slabs, batch2, batch1}, box {128 B, K rows, slabs}: the
//             whole tile in ONE box, laid out slab after slab exactly as separate boxes would be.
const char* build_operand_map(const Operand& op, int esize, int64_t rows, int64_t cols,
                              bool k_is_col, const BatchDims& bd, const int64_t* bstride,
                              uint32_t tile_mn, uint32_t slabs_per_box, OperandMap* out) {
  const int64_t mn = k_is_col ? rows : cols;
  const int64_t kk = k_is_col ? cols : rows;
  const int64_t s_mn = k_is_col ? op.stride_r : op.stride_c;
  const int64_t s_k = k_is_col ? op.stride_c : op.stride_r;
  const uintptr_t base = reinterpret_cast<uintptr_t>(op.ptr) + static_cast<uintptr_t>(op.offset) * esize;
  if (base % 16 != 0) return "operand base address is not 16-byte aligned";
  if (mn > 0x7FFFFFFFll || kk > 0x7FFFFFFFll) return "extent exceeds 2^31 (TMA coordinates are signed 32-bit)";

  const int cls = classify_operand(op, esize, rows, cols, k_is_col);
  if (cls < 0) return "neither matrix index is contiguous with a 16-byte-multiple pitch";
  const bool k_major = cls == 0;
  out->mn_major = !k_major;
  const uint32_t inner_box = 128u / esize;  // 128 bytes: one swizzle row
  out->slab_dim = !k_major && slabs_per_box > 1 && mn % inner_box == 0 && bd.size[0] == 1;

  const int64_t inner = k_major ? kk : mn;
  const int64_t outer = k_major ? mn : kk;
  int64_t pitch = k_major ? s_mn : s_k;  // elements between consecutive `outer` indices
  if (outer == 1 || !pitch_ok(pitch, esize)) pitch = ((inner * esize + 15) / 16 * 16) / esize;
  if (!pitch_ok(pitch, esize)) return "pitch is not a positive multiple of 16 bytes";

  cuuint64_t dims[5] = {static_cast<cuuint64_t>(inner), static_cast<cuuint64_t>(outer), 1, 1, 1};
  cuuint64_t strides[4];
  cuuint32_t box[5] = {inner_box, k_major ? tile_mn : inner_box, 1, 1, 1};
  strides[0] = static_cast<cuuint64_t>(pitch) * esize;
  int first_batch_dim = 2;
  if (out->slab_dim) {
    dims[0] = inner_box;
    dims[2] = static_cast<cuuint64_t>(mn / inner_box);
    strides[1] = 128;
    box[2] = slabs_per_box;
    first_batch_dim = 3;
  }
  cuuint64_t natural = strides[0] * dims[1];
  for (int j = 0; first_batch_dim + j < 5; ++j) {  // j = 0 is the fastest-varying batch dim (slot 2)
    const int slot = kMaxBatchDims - 1 - j;
    const int64_t sz = bd.size[slot], bs = bstride[slot];
    const int d = first_batch_dim + j;
    if (sz > 1 && bs != 0) {
      if (!pitch_ok(bs, esize)) return "batch stride is not a positive multiple of 16 bytes";
      dims[d] = static_cast<cuuint64_t>(sz);
      strides[d - 1] = static_cast<cuuint64_t>(bs) * esize;
      out->bmul[slot] = 1;
    } else {
      dims[d] = 1;
      strides[d - 1] = (natural + 15) / 16 * 16;
      out->bmul[slot] = 0;
    }
    natural = strides[d - 1] * dims[d];
  }
  cuuint32_t estr[5] = {1, 1, 1, 1, 1};
  const CUtensorMapDataType dt = esize == 1 ? CU_TENSOR_MAP_DATA_TYPE_UINT8
                                 : esize == 2 ? CU_TENSOR_MAP_DATA_TYPE_UINT16
                                              : CU_TENSOR_MAP_DATA_TYPE_UINT32;
  // A tensor map is a pure function of the arguments below, so the encoded 128 bytes are kept
  // per thread and reused when the same operand comes back (a layer called every step, the
  // weights of an MLP): the driver call is then skipped.
  MapKey key{};
  key.base = base; key.esize = static_cast<uint32_t>(esize);
  for (int i = 0; i < 5; ++i) { key.dims[i] = dims[i]; key.box[i] = box[i]; }
  for (int i = 0; i < 4; ++i) key.strides[i] = strides[i];
  if (map_cache_get(key, &out->map)) return nullptr;
  EncodeTiledFn enc = encode_fn();
  if (!enc) return "cuTensorMapEncodeTiled is not available from the driver";
  const CUresult r = enc(&out->map, dt, 5, reinterpret_cast<void*>(base), dims, strides, box, estr,
                         CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                         CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r == CUDA_ERROR_INVALID_VALUE) return "cuTensorMapEncodeTiled rejected the layout";
  // Anything else (no current context, driver shut down) is a failure of the call, not a
  // property of the layout: the leading '!' makes the caller report it instead of falling back.
  if (r != CUDA_SUCCESS) return "!cuTensorMapEncodeTiled failed (no usable CUDA context on this thread?)";
  map_cache_put(key, out->map);
  return nullptr;
}

// Tensor map of the output for the TMA stores of a CTA's last tile: dims {N, M, batches}, box
// {64 bytes of a row, 32 rows, 1}, 64-byte swizzle (the layout stage_write_row64 produces).
// False when the output cannot be described (then the kernel keeps its ordinary stores).
bool build_output_map(const TcParams& p, int osz, uint32_t batches, CUtensorMap* out) {
  if (!(p.out_vec_ok & 1u) || (osz != 2 && osz != 4)) return false;
  const uint64_t row_pitch = p.ldc * static_cast<uint64_t>(osz), batch_pitch = p.out_batch_stride * static_cast<uint64_t>(osz);
  if (row_pitch >= (1ull << 40) || batch_pitch >= (1ull << 40) || p.N == 0 || p.M == 0 || batches == 0) return false;
  cuuint64_t dims[3] = {p.N, p.M, batches};
  cuuint64_t strides[2] = {row_pitch, batches > 1 ? batch_pitch : row_pitch * p.M};
  if (strides[1] % 16 != 0 || strides[1] >= (1ull << 40)) return false;
  cuuint32_t box[3] = {static_cast<cuuint32_t>(64 / osz), 32, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  MapKey key{};
  key.base = reinterpret_cast<uintptr_t>(p.out); key.esize = static_cast<uint32_t>(osz); key.kind = 1;
  for (int i = 0; i < 3; ++i) { key.dims[i] = dims[i]; key.box[i] = box[i]; }
  for (int i = 0; i < 2; ++i) key.strides[i] = strides[i];
  if (map_cache_get(key, out)) return true;
  EncodeTiledFn enc = encode_fn();
  if (!enc) return false;
  const CUresult r = enc(out, osz == 2 ? CU_TENSOR_MAP_DATA_TYPE_UINT16 : CU_TENSOR_MAP_DATA_TYPE_UINT32, 3, p.out, dims,
                         strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_64B,
                         CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return false;
  map_cache_put(key, *out);
  return true;
}

// Clusters of 2, 4 and 8 one-CTA tiles' K slices that can be resident at once, per device
// (index log2(slices)); 0 = not measured yet.  launch_inst fills it in, the planner reads it.
std::atomic<int> g_split_capacity[kMaxDevices][4];
constexpr int kSplitDoesNotFit = -0x5117;   // launch_inst: more tiles than resident clusters, nothing launched

template <int KIND, int BN, int OUT, bool SWIGLU, bool PAIR, int MH>
int launch_inst(const CUtensorMap& ma, const CUtensorMap& mb, const CUtensorMap& mb2, const CUtensorMap& mo,
                const TcParams& p, int device, int sm_count, cudaStream_t stream) {
  using Cfg = TileCfg<BN, PAIR, MH>;
  constexpr size_t smem = Cfg::kStages * (Cfg::kStageA + Cfg::kStageB) + Cfg::kEpiWarps * Cfg::kEpiStage +
                          256 /* SmemTail */ + 1024 /* alignment slack */;
  static_assert(sizeof(SmemTail) <= 256, "barrier block outgrew its slot");
  // CTAs (1-CTA form) or CTA pairs that can be resident; concurrent first callers compute the
  // same value, so relaxed atomics are enough.
  static std::atomic<int> max_ctas[kMaxDevices][4];   // by log2(K slices)
  if (p.k_splits != 1u && (PAIR || SWIGLU || KIND == KIND_TF32 || (p.k_splits != 2u && p.k_splits != 4u && p.k_splits != 8u) ||
                           (BN / 32) % p.k_splits != 0u))
    return fail(HODU_B200_ERR_LAUNCH, "K slices asked of a tile form that has none");
  const int split_log2 = p.k_splits >= 8u ? 3 : (p.k_splits >= 4u ? 2 : (p.k_splits == 2u ? 1 : 0));
  const unsigned cluster_ctas = (PAIR ? 2u : 1u) * p.k_splits;
  auto kern = gemm_tc_kernel<KIND, BN, OUT, SWIGLU, PAIR, MH>;
  cudaLaunchConfig_t cfg = {};
  cfg.blockDim = dim3(threads_for(MH), 1, 1);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attrs[2];
  int n_attrs = 0;
  if (cluster_ctas > 1u) {
    attrs[n_attrs].id = cudaLaunchAttributeClusterDimension;
    attrs[n_attrs].val.clusterDim.x = cluster_ctas; attrs[n_attrs].val.clusterDim.y = 1; attrs[n_attrs].val.clusterDim.z = 1;
    ++n_attrs;
  }
  if (dependent_launch_enabled()) {
    // The kernel's set-up (barriers, TMEM, tensor-map prefetch) may overlap the tail of the
    // kernel before it in the stream; it waits for that kernel before touching global memory.
    attrs[n_attrs].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attrs[n_attrs].val.programmaticStreamSerializationAllowed = 1;
    ++n_attrs;
  }
  cfg.attrs = attrs;
  cfg.numAttrs = n_attrs;
  int resident = max_ctas[device][split_log2].load(std::memory_order_relaxed);
  if (resident == 0) {
    HODU_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       static_cast<int>(smem)),
                  HODU_B200_ERR_LAUNCH);
    int n = sm_count / static_cast<int>(cluster_ctas);
    if (cluster_ctas > 1u) {
      cfg.gridDim = dim3(cluster_ctas, 1, 1);
      int q = 0;
      if (cudaOccupancyMaxActiveClusters(&q, kern, &cfg) == cudaSuccess && q >= 1) n = q;
      else cudaGetLastError();
    }
    resident = n > 0 ? n : 1;
    max_ctas[device][split_log2].store(resident, std::memory_order_relaxed);
    if (!PAIR) g_split_capacity[device][split_log2].store(resident, std::memory_order_relaxed);
  }
  // K slices are planned for ONE wave of clusters (the hardware keeps the CTAs of a cluster
  // together, so more tiles than resident clusters would still be correct, but they would run
  // in waves, which is what slicing is there to avoid): such a plan goes back to the planner.
  if (p.k_splits > 1u && p.num_tiles > static_cast<uint32_t>(resident)) return kSplitDoesNotFit;
  const int units = static_cast<int>(p.num_tiles < static_cast<uint32_t>(resident) ? p.num_tiles : resident);
  cfg.gridDim = dim3(cluster_ctas * static_cast<unsigned>(units), 1, 1);
  if (debug_enabled())
    fprintf(stderr, "[hodu_b200] gemm_tc %s: %u tiles of %dx%d, %u K slice(s), grid %u, %zu B smem, A %s x%u, B %s x%u%s\n",
            PAIR ? "pair" : "1-CTA", p.num_tiles, PAIR ? 256 * MH : 128, SWIGLU ? BN / 2 : BN, p.k_splits, cfg.gridDim.x, smem,
            p.a.mn_major ? "M-major" : "K-major", p.a.boxes, p.b.mn_major ? "N-major" : "K-major", p.b.boxes,
            p.b.slab_dim ? " (slab dim)" : "");
  if (debug_enabled()) {
    // Everything the kernel takes on trust, checked on the host before it runs.
    constexpr uint32_t kTileRows = PAIR ? 256u * MH : 128u, kTileCols = SWIGLU ? BN / 2 : BN;
    const char* bad = nullptr;
    if (p.a.boxes * p.a.box_bytes != static_cast<uint32_t>(Cfg::kStageA1)) bad = "lhs boxes do not fill a k-block of a stage";
    else if (p.b.boxes * p.b.box_bytes != static_cast<uint32_t>(Cfg::kStageB1)) bad = "rhs boxes do not fill a k-block of a stage";
    else if (Cfg::kKbPerStage == 2 && KIND == KIND_TF32 && p.k_gen < p.k_blocks &&
             ((p.k_gen & 1u) || (p.k_gen_limit < p.k_blocks && (p.k_gen_limit & 1u))))
      bad = "accumulator generations must start at even k-blocks when a stage holds two";
    else if (Cfg::kTmemCols > 512 || (Cfg::kTmemCols & (Cfg::kTmemCols - 1)) != 0) bad = "TMEM columns not a power of two <= 512";
    else if (static_cast<uint64_t>(p.tiles_m) * kTileRows < p.M || static_cast<uint64_t>(p.tiles_m - 1) * kTileRows >= p.M)
      bad = "row tiles do not cover M exactly";
    else if (static_cast<uint64_t>(p.tiles_n) * kTileCols < p.N || static_cast<uint64_t>(p.tiles_n - 1) * kTileCols >= p.N)
      bad = "column tiles do not cover N exactly";
    else if (static_cast<uint64_t>(p.k_blocks) * p.bk < p.K || static_cast<uint64_t>(p.k_blocks - 1) * p.bk >= p.K)
      bad = "k-blocks do not cover K exactly";
    else if (static_cast<uint64_t>(p.tiles_m) * kTileRows > 0x7FFFFFFFull || static_cast<uint64_t>(p.tiles_n) * BN > 0x7FFFFFFFull ||
             static_cast<uint64_t>(p.k_blocks) * p.bk > 0x7FFFFFFFull)
      bad = "a TMA coordinate would not fit 32 signed bits";
    else if (p.num_tiles % (p.tiles_m * p.tiles_n) != 0) bad = "tile count is not batches x tiles_m x tiles_n";
    else if (p.ldc < p.N || p.out_batch_stride < static_cast<unsigned long long>(p.M - 1) * p.ldc + p.N) bad = "output rows or batches overlap";
    else if (p.k_gen == 0 || p.k_gen > p.k_blocks || p.k_gen_limit > p.k_blocks) bad = "accumulator generations out of range";
    else if (cfg.gridDim.x == 0 || cfg.gridDim.x % cluster_ctas != 0u) bad = "grid size";
    else if (p.k_splits != 1u && p.k_splits != 2u && p.k_splits != 4u && p.k_splits != 8u) bad = "K slices not 1, 2, 4 or 8";
    else if (p.k_splits > 1u && (PAIR || SWIGLU || KIND == KIND_TF32 || cluster_ctas > 8u || (BN / 32) % p.k_splits != 0u ||
                                 cfg.gridDim.x != cluster_ctas * p.num_tiles ||
                                 static_cast<uint64_t>(p.kb_per_split) * (p.k_splits - 1u) >= p.k_blocks ||
                                 static_cast<uint64_t>(p.kb_per_split) * p.k_splits < p.k_blocks))
      bad = "K slices do not fit this form, this grid or K";
    else if (smem > 232448) bad = "shared memory beyond the 227 KB a CTA can have";
    if (bad) return fail(HODU_B200_ERR_LAUNCH, "debug check before launch: %s", bad);
  }
  HODU_CUDA_TRY(cudaLaunchKernelEx(&cfg, kern, ma, mb, mb2, mo, p), HODU_B200_ERR_LAUNCH);
  count_launch();
  if (debug_enabled()) {
    // ... and the outcome, at once: wait for the kernel, then read what its bounded waits recorded.
    HODU_CUDA_TRY(cudaStreamSynchronize(stream), HODU_B200_ERR_LAUNCH);
    uint32_t w = 0;
    HODU_CUDA_TRY(cudaMemcpy(&w, p.status, sizeof(w), cudaMemcpyDeviceToHost), HODU_B200_ERR_MEMORY);
    if (w != 0)
      return fail(HODU_B200_ERR_DEVICE_STATUS, "debug check after launch: device status word 0x%08x (cta %u, wait %u)", w,
                  (w >> 4) & 0xFFFFu, w & 0xFu);
  }
  return 0;
}

template <int KIND, int OUT, bool SWIGLU>
int launch_shape(int bn, int pair /* 0: 1-CTA, 1: 256x256 pair, 2: 512x256 pair */, const CUtensorMap& ma, const CUtensorMap& mb, const CUtensorMap& mb2,
                 const CUtensorMap& mo, const TcParams& p, int device, int sm_count, cudaStream_t stream) {
  if (pair == 2) return launch_inst<KIND, 256, OUT, SWIGLU, true, 2>(ma, mb, mb2, mo, p, device, sm_count, stream);
  if (pair == 1) return launch_inst<KIND, 256, OUT, SWIGLU, true, 1>(ma, mb, mb2, mo, p, device, sm_count, stream);
  if constexpr (SWIGLU) {
    return launch_inst<KIND, 256, OUT, true, false, 1>(ma, mb, mb2, mo, p, device, sm_count, stream);
  } else {
    switch (bn) {
      case 256: return launch_inst<KIND, 256, OUT, false, false, 1>(ma, mb, mb2, mo, p, device, sm_count, stream);
      case 128: return launch_inst<KIND, 128, OUT, false, false, 1>(ma, mb, mb2, mo, p, device, sm_count, stream);
      default: return launch_inst<KIND, 64, OUT, false, false, 1>(ma, mb, mb2, mo, p, device, sm_count, stream);
    }
  }
}

}  // namespace

int launch_wait_timeout_probe(DeviceState* st, cudaStream_t stream, uint32_t limit_ms) {
  wait_timeout_probe_kernel<<<1, 32, 0, stream>>>(st->status, static_cast<uint64_t>(limit_ms) * 1000000ull);
  HODU_CUDA_TRY(cudaGetLastError(), HODU_B200_ERR_LAUNCH);
  count_launch();
  return 0;
}

// Whether TMA can describe `op` as it lies in memory (the per-operand rules of build_operand_map).
bool tc_operand_describable(const Problem& pb, const Operand& op, bool is_lhs, int esize) {
  const int64_t rows = is_lhs ? pb.M : pb.K, cols = is_lhs ? pb.K : pb.N;
  const uintptr_t base = reinterpret_cast<uintptr_t>(op.ptr) + static_cast<uintptr_t>(op.offset) * esize;
  if (base % 16 != 0 || rows > 0x7FFFFFFFll || cols > 0x7FFFFFFFll) return false;
  if (classify_operand(op, esize, rows, cols, is_lhs) < 0) return false;
  for (int d = 0; d < pb.batch_ndim; ++d)
    if (pb.batch_shape[d] > 1 && op.bstride[d] != 0 && !pitch_ok(op.bstride[d], esize)) return false;
  return true;
}

namespace {
// Plans and launches; with `plan_only` it stops after the plan and reports the K slices chosen.
int launch_gemm_tc_planned(const Problem& pb, DeviceState* st, cudaStream_t stream, const char** why, bool allow_split,
                           int* plan_only);
}

int tc_planned_k_slices(const Problem& pb, DeviceState* st) {
  const char* why = nullptr;
  int slices = 1;
  if (launch_gemm_tc_planned(pb, st, nullptr, &why, true, &slices) != 0) return 1;
  return slices;
}

int launch_gemm_tc(const Problem& pb, DeviceState* st, cudaStream_t stream, const char** why) {
  // A plan with K slices assumes how many clusters fit the device; the first launch of each
  // cluster size measures it, and when the plan then does not fit it is made again without.
  int rc = launch_gemm_tc_planned(pb, st, stream, why, true, nullptr);
  if (rc == kSplitDoesNotFit) rc = launch_gemm_tc_planned(pb, st, stream, why, true, nullptr);
  if (rc == kSplitDoesNotFit) rc = launch_gemm_tc_planned(pb, st, stream, why, false, nullptr);
  return rc;
}

namespace {
int launch_gemm_tc_planned(const Problem& pb, DeviceState* st, cudaStream_t stream, const char** why, bool allow_split,
                           int* plan_only) {
  static const char* none = "";
  *why = none;
  int kind, esize, fmt;
  switch (pb.in_dtype) {
    case HODU_DTYPE_BF16: kind = KIND_F16; esize = 2; fmt = 1; break;
    case HODU_DTYPE_F16: kind = KIND_F16; esize = 2; fmt = 0; break;
    case HODU_DTYPE_F8E4M3: kind = KIND_F8; esize = 1; fmt = 0; break;
    case HODU_DTYPE_I8: kind = KIND_I8; esize = 1; fmt = 1; break;
    case HODU_DTYPE_F32:
      if (!pb.f32_presplit) { *why = "f32 reaches the tensor cores only through the TF32 split (gemm_f32.cu)"; return 1; }
      kind = KIND_TF32; esize = 4; fmt = 2; break;
    default: *why = "input dtype has no tensor-core kernel"; return 1;
  }
  if (st->cc_major != 10) { *why = "device is not sm_100"; return 1; }
  if (pb.M < 1 || pb.N < 1 || pb.K < 1 || pb.batches < 1) { *why = "empty problem"; return 1; }

  BatchDims bd;
  if (!collapse_batch(pb, &bd)) { *why = "more than three independent batch dims"; return 1; }
  if (pb.batches > 0x7FFFFFFFll) { *why = "too many batches"; return 1; }
  const int b_cls = classify_operand(pb.b, esize, pb.K, pb.N, /*k_is_col=*/false);
  if (b_cls < 0) { *why = "rhs: neither matrix index is contiguous with a 16-byte-multiple pitch"; return 1; }

  // Tile shape: the candidate with the least estimated time = waves x cycles per tile.
  //   form 2: CTA pair, 512 x 256 tile, two 128-row accumulators per CTA (all of TMEM: the
  //           epilogue of a tile is not hidden behind the next tile's main loop)
  //   form 1: CTA pair, 256 x 256 tile, double-buffered accumulator
  //   form 0: one CTA, 128 x BN tile; an 8-bit N-contiguous rhs needs BN >= 128 (one 128-byte
  //           swizzle row holds 128 of its elements)
  // Cycles per k-block = max(MMA cycles, operand bytes one SM takes in / ~50 B per cycle): a fit
  // to the measured tensor-pipe utilisations of large products (512x256: 0.9, 256x256: 0.78,
  // 128x256: 0.53), which follow the bytes per MMA cycle each form needs (48, 64, 96 B/clk).
  // (Launches of few tiles are judged by a second estimate further down.)
  const int forced = forced_path();
  const int units_pair = st->sm_count / 2 > 0 ? st->sm_count / 2 : 1;
  const double k_blocks_d = static_cast<double>((pb.K + (128 / esize) - 1) / (128 / esize));
  int device = 0;
  cudaGetDevice(&device);
  if (device < 0 || device >= kMaxDevices) device = 0;
  // HODU_B200_KSPLIT: 1 = never slice K across a cluster, 2 / 4 / 8 = that many slices whenever
  // a form allows it (tuning aid); unset or 0 = by estimated time.
  static const int split_forced = [] { const char* e = getenv("HODU_B200_KSPLIT"); return e ? atoi(e) : 0; }();
  int form = 0, bn = 256, splits = 1;
  {
    double best = 1e300;
    auto consider = [&](int f, int c) {
      const int64_t tm = f == 2 ? 512 : (f == 1 ? 256 : 128);
      const int64_t oc = pb.swiglu ? c / 2 : c;
      const int64_t tiles = ((pb.M + tm - 1) / tm) * ((pb.N + oc - 1) / oc) * pb.batches;
      const int64_t units = f ? units_pair : st->sm_count;
      const double mma_clk = (c == 256 ? 128.0 : (c == 128 ? 64.0 : 50.0)) * 4.0 * (f == 2 ? 2.0 : 1.0);
      const double bytes = (f == 2 ? 32768.0 : 16384.0) + (f ? 128.0 : c) * 128.0;
      const double kblock = 1.08 * (mma_clk > bytes / 50.0 ? mma_clk : bytes / 50.0);
      // Short-K tiles are bound by draining and storing the output instead: measured on
      // 128-deep bf16 products, cycles per 64 KB of output one CTA stores: 4400 (one CTA per
      // tile), 5500 (CTA pairs, whose per-tile handshakes cross the cluster).
      const double out_bytes_cta = 128.0 * (f == 2 ? 2.0 : 1.0) * static_cast<double>(oc) * dtype_size(pb.out_dtype);
      const double drain_clk = (f ? 5500.0 : 4400.0) * out_bytes_cta / 65536.0;
      const double main_clk = k_blocks_d * kblock + (f == 2 ? 8000.0 : 0.0) + 1500.0;
      const double tile_clk = main_clk > drain_clk ? main_clk : drain_clk;
      // CTA pairs pay a fixed price per launch (cluster launch, cross-CTA set-up and teardown):
      // measured on 1536^3 .. 3072 x 768 x 3072 products, where one CTA per tile wins by 5-15 %.
      const double t = static_cast<double>((tiles + units - 1) / units) * tile_clk + (f ? 12000.0 : 0.0);
      if (t < best) { best = t; form = f; bn = c; }
    };
    const bool allow_pair = forced != HODU_B200_PATH_TENSOR_1CTA && st->sm_count >= 2;
    const bool only_pair = forced == HODU_B200_PATH_TENSOR_2CTA || forced == HODU_B200_PATH_TENSOR_2CTA_512;
    if (allow_pair && forced != HODU_B200_PATH_TENSOR_2CTA) consider(2, 256);
    if (allow_pair && forced != HODU_B200_PATH_TENSOR_2CTA_512) consider(1, 256);
    if (!only_pair) {
      consider(0, 256);
      if (!pb.swiglu) {
        consider(0, 128);
        if (!(b_cls == 1 && esize == 1)) consider(0, 64);
      }
    }
    // K slices across a cluster, when the tiles chosen above leave SMs idle: decided on a second
    // estimate, fitted to launches of few tiles (cycles at the clock such launches run at):
    //   5200 per launch (set-up, first loads, teardown); per k-block 460 / 570 / 680 for one CTA
    //   with 64 / 128 / 256 columns, 620 per CTA of a 256 x 256 pair, 1110 of a 512 x 256 pair;
    //   590 (800 for 4-byte outputs) per 32-column chunk drained and stored; with slices, 285
    //   per chunk handed to another slice, 700 for the barrier, 700 per chunk read from another.
    if (allow_split && split_forced != 1 && !only_pair && !pb.swiglu && kind != KIND_TF32) {
      const double chunk_clk = dtype_size(pb.out_dtype) == 4 ? 800.0 : 590.0;
      auto kblock_fit = [](int f, int c) { return f == 2 ? 1110.0 : (f == 1 ? 620.0 : (c == 256 ? 680.0 : (c == 128 ? 570.0 : 460.0))); };
      const int64_t tm0 = form == 2 ? 512 : (form == 1 ? 256 : 128);
      const int64_t tiles0 = ((pb.M + tm0 - 1) / tm0) * ((pb.N + bn - 1) / bn) * pb.batches;
      const int64_t units0 = form ? units_pair : st->sm_count;
      const double whole = 5200.0 + static_cast<double>((tiles0 + units0 - 1) / units0) * k_blocks_d * kblock_fit(form, bn) +
                           (bn / 32) * (form == 2 ? 2 : 1) * chunk_clk;
      double best_split = 1e300;
      int split_bn = 0, split_ks = 1;
      for (int ks = 2; ks <= 8; ks *= 2) {
        if (split_forced > 1 && split_forced != ks) continue;
        for (int c = 256; c >= 64; c /= 2) {
          if ((c / 32) % ks != 0 || (c == 64 && b_cls == 1 && esize == 1)) continue;
          const int64_t tiles = ((pb.M + 127) / 128) * ((pb.N + c - 1) / c) * pb.batches;
          const int measured = g_split_capacity[device][ks == 8 ? 3 : (ks == 4 ? 2 : 1)].load(std::memory_order_relaxed);
          const int64_t capacity = measured > 0 ? measured : st->sm_count / ks;
          if (tiles > capacity || k_blocks_d < 4.0 * ks) continue;   // one wave of clusters; >= 4 k-blocks a slice
          const int chunks = c / 32, per = chunks / ks;
          const double t = 5200.0 + static_cast<double>((static_cast<int64_t>(k_blocks_d) + ks - 1) / ks) * kblock_fit(0, c) +
                           (chunks - per) * 285.0 + 700.0 + per * (chunk_clk + (ks - 1) * 700.0);
          if (t < best_split) { best_split = t; split_bn = c; split_ks = ks; }
        }
      }
      if (split_ks > 1 && (split_forced > 1 || best_split < 0.93 * whole)) { form = 0; bn = split_bn; splits = split_ks; }
    }
  }
  if (plan_only) { *plan_only = splits; return 0; }
  const bool use_pair = form != 0;
  const int mh = form == 2 ? 2 : 1;
  const int64_t tile_m = form == 2 ? 512 : (form == 1 ? 256 : BM);
  const int64_t tiles_m = (pb.M + tile_m - 1) / tile_m;
  const int out_cols = pb.swiglu ? bn / 2 : bn;       // output columns per tile
  const int64_t tiles_n = (pb.N + out_cols - 1) / out_cols;
  const int64_t num_tiles = tiles_m * tiles_n * pb.batches;
  if (num_tiles > 0x7FFFFFFFll) { *why = "too many tiles"; return 1; }
  // Columns of B one CTA stages per k-block, and how many TMA boxes bring them in.
  const uint32_t b_cols_staged = use_pair ? 128u : static_cast<uint32_t>(bn);
  const uint32_t b_sources = (pb.swiglu && !use_pair) ? 2u : 1u;   // gate and up halves from two maps
  const uint32_t b_cols_per_box = b_cols_staged / b_sources;
  const uint32_t mn_per_slab = 128u / esize;

  OperandMap oa, ob, ob2;
  const uint32_t a_rows_staged = static_cast<uint32_t>(BM * mh);
  const char* err = build_operand_map(pb.a, esize, pb.M, pb.K, /*k_is_col=*/true, bd, bd.a_stride, a_rows_staged,
                                      a_rows_staged / mn_per_slab, &oa);
  auto refuse = [&](const char* e) { *why = e; return e[0] == '!' ? fail(HODU_B200_ERR_LAUNCH, "%s", e + 1) : 1; };
  if (err) return refuse(err);
  err = build_operand_map(pb.b, esize, pb.K, pb.N, /*k_is_col=*/false, bd, bd.b_stride, b_cols_per_box,
                          b_cols_per_box / mn_per_slab, &ob);
  if (err) return refuse(err);
  if (pb.swiglu) {
    err = build_operand_map(pb.b2, esize, pb.K, pb.N, false, bd, bd.b2_stride, b_cols_per_box,
                            b_cols_per_box / mn_per_slab, &ob2);
    if (err) return refuse(err);
    if (ob2.mn_major != ob.mn_major || ob2.slab_dim != ob.slab_dim) { *why = "gate and up weights differ in layout"; return 1; }
    for (int j = 0; j < 3; ++j)
      if (ob2.bmul[j] != ob.bmul[j]) { *why = "gate and up weights differ in batch broadcast"; return 1; }
  } else {
    ob2 = ob;
  }

  TcParams p{};
  p.M = static_cast<uint32_t>(pb.M); p.N = static_cast<uint32_t>(pb.N); p.K = static_cast<uint32_t>(pb.K);
  p.tiles_m = static_cast<uint32_t>(tiles_m); p.tiles_n = static_cast<uint32_t>(tiles_n);
  p.num_tiles = static_cast<uint32_t>(num_tiles);
  p.bk = 128u / esize;
  p.k_blocks = static_cast<uint32_t>((pb.K + p.bk - 1) / p.bk);
  p.k_splits = static_cast<uint32_t>(splits);
  p.kb_per_split = (p.k_blocks + p.k_splits - 1u) / p.k_splits;
  if (p.k_splits > 1u && static_cast<uint64_t>(p.kb_per_split) * (p.k_splits - 1u) >= p.k_blocks) {
    p.k_splits = 1u;   // the last slice would be empty
    p.kb_per_split = p.k_blocks;
  }
  // Rows of A per raster group: 4096 in the 512x256 form (measured on the 8192^3 and MLP shapes:
  // 2048 and 8192 rows are 1-2 % slower, 16384 rows 10 % slower), 2048 in the others.
  p.group_m = form == 2 ? 8 : (form == 1 ? 8 : 16);
  {
    // HODU_B200_GROUP_ROWS=<rows of A per raster group> overrides the default (tuning aid).
    static const int rows_override = [] { const char* e = getenv("HODU_B200_GROUP_ROWS"); return e ? atoi(e) : 0; }();
    if (rows_override >= 128) {
      const uint32_t tile_rows = form == 2 ? 512u : (form == 1 ? 256u : 128u);
      p.group_m = static_cast<uint32_t>(rows_override) / tile_rows;
      if (p.group_m < 1) p.group_m = 1;
    }
  }
  p.bdim1 = static_cast<uint32_t>(bd.size[1]); p.bdim2 = static_cast<uint32_t>(bd.size[2]);

  const uint32_t slab_bytes = 128u * p.bk;          // MN-major slab: bk rows of 128 bytes
  const uint32_t kstep_rows = 32u / esize;          // K elements one MMA consumes
  const uint32_t desc_hi = (1024u >> 4) | (1u << 14) | (2u << 29);  // SBO 1024 B, version 1, 128B swizzle
  auto fill = [&](OperandLoad& o, const OperandMap& m, uint32_t mn_staged, uint32_t sources) {
    o.mn_major = m.mn_major; o.slab_dim = m.slab_dim; o.inner = mn_per_slab;
    for (int j = 0; j < 3; ++j) o.bmul[j] = m.bmul[j];
    o.desc_hi = desc_hi;
    if (m.mn_major) {
      const uint32_t slabs = mn_staged / mn_per_slab;
      if (m.slab_dim) { o.boxes = sources; o.box_bytes = slab_bytes * (slabs / sources); o.box_mn = mn_staged / sources; }
      else { o.boxes = slabs; o.box_bytes = slab_bytes; o.box_mn = mn_per_slab; }
      o.desc_lo = (slab_bytes >> 4) << 16; o.kstep16 = (kstep_rows * 128u) >> 4;
    } else {
      o.boxes = sources; o.box_mn = mn_staged / sources; o.box_bytes = o.box_mn * 128u;
      o.desc_lo = 1u << 16; o.kstep16 = 2;
    }
  };
  fill(p.a, oa, a_rows_staged, 1);
  fill(p.b, ob, b_cols_staged, b_sources);
  // SwiGLU without the slab dimension walks gate slabs then up slabs: the producer switches
  // maps at boxes / 2, which needs an even box count -- true for every case above.
  const uint32_t c_fmt = kind == KIND_I8 ? 2u : 1u;
  p.idesc = (c_fmt << 4) | (static_cast<uint32_t>(fmt) << 7) | (static_cast<uint32_t>(fmt) << 10) |
            (static_cast<uint32_t>(oa.mn_major) << 15) | (static_cast<uint32_t>(ob.mn_major) << 16) |
            (static_cast<uint32_t>(bn >> 3) << 17) | (static_cast<uint32_t>((use_pair ? 256 : BM) >> 4) << 24);
  p.alpha = pb.alpha;
  p.swiglu_flags = pb.swiglu_flags;
  p.bias = pb.bias ? static_cast<const uint8_t*>(pb.bias) + pb.bias_offset * dtype_size(pb.out_dtype) : nullptr;
  p.bias_stride = pb.bias_stride;
  p.bias_flags = pb.bias_flags;
  p.ldc = static_cast<unsigned long long>(pb.ldc > 0 ? pb.ldc : pb.N);
  p.out_batch_stride = static_cast<unsigned long long>(pb.M) * p.ldc;
  p.out = pb.out;
  p.status = st->status;
  const int osz = dtype_size(pb.out_dtype);
  p.out_vec_ok = (reinterpret_cast<uintptr_t>(pb.out) % 16 == 0 && (p.ldc * osz) % 16 == 0 &&
                  (p.out_batch_stride * osz) % 16 == 0) ? 1u : 0u;
  // The tensor core adds into its f32 accumulator with truncation, so the error of a long sum
  // grows with its length (7e-5 of the largest output at K = 8192 with one accumulator per
  // tile, against the 1e-4 bar of the f32 path).  Long f32 products therefore run as
  // generations of 128 k-blocks (4096 elements of K; 64 beyond K = 32768: 1e-5 measured
  // at every K up to 65536, for 12 % of the throughput): each generation starts a
  // fresh accumulator and the epilogue adds it to the output in round-to-nearest f32.
  // (Generations over the hi x hi third of K' only, with the two small thirds as one last
  // generation, measured 5 % faster but is wrong for K slices of a split product, which do not
  // line up with the thirds; the limit below therefore stays at the whole K'.)
  p.k_gen = p.k_blocks;
  p.k_gen_limit = p.k_blocks;
  if (kind == KIND_TF32 && pb.f32_presplit && !pb.swiglu && p.k_blocks > 128u)
    p.k_gen = p.k_blocks > 3072u ? 64u : 128u;

  // The output's own tensor map, when it has one (HODU_B200_TMA_STORE=0 keeps ordinary stores).
  CUtensorMap out_map;
  memset(&out_map, 0, sizeof(out_map));
  static const bool tma_store_on = [] { const char* e = getenv("HODU_B200_TMA_STORE"); return !(e && e[0] == '0'); }();
  p.out_tma = (tma_store_on && build_output_map(p, osz, static_cast<uint32_t>(pb.batches), &out_map)) ? 1u : 0u;
  if (p.out_tma == 0u) out_map = oa.map;   // a valid descriptor for the prefetch; never used for a store

#define HODU_TC(KIND, OUTE, SW) \
  return launch_shape<KIND, OUTE, SW>(bn, form, oa.map, ob.map, ob2.map, out_map, p, device, st->sm_count, stream)
  if (pb.swiglu) {
    if (kind != KIND_F16) { *why = "SwiGLU epilogue exists for bf16/f16 only"; return 1; }
    if (pb.out_dtype == HODU_DTYPE_BF16) HODU_TC(KIND_F16, OUT_BF16, true);
    if (pb.out_dtype == HODU_DTYPE_F16) HODU_TC(KIND_F16, OUT_F16, true);
    *why = "unsupported SwiGLU output dtype"; return 1;
  }
  if (kind == KIND_F16) {
    if (pb.out_dtype == HODU_DTYPE_BF16) HODU_TC(KIND_F16, OUT_BF16, false);
    if (pb.out_dtype == HODU_DTYPE_F16) HODU_TC(KIND_F16, OUT_F16, false);
    if (pb.out_dtype == HODU_DTYPE_F32) HODU_TC(KIND_F16, OUT_F32, false);
  } else if (kind == KIND_TF32) {
    if (pb.out_dtype == HODU_DTYPE_F32) HODU_TC(KIND_TF32, OUT_F32, false);
  } else if (kind == KIND_F8) {
    if (pb.out_dtype == HODU_DTYPE_BF16) HODU_TC(KIND_F8, OUT_BF16, false);
    if (pb.out_dtype == HODU_DTYPE_F16) HODU_TC(KIND_F8, OUT_F16, false);
    if (pb.out_dtype == HODU_DTYPE_F32) HODU_TC(KIND_F8, OUT_F32, false);
    if (pb.out_dtype == HODU_DTYPE_F8E4M3) HODU_TC(KIND_F8, OUT_E4M3, false);
  } else {
    if (pb.out_dtype == HODU_DTYPE_I32) HODU_TC(KIND_I8, OUT_I32, false);
    if (pb.out_dtype == HODU_DTYPE_I8) HODU_TC(KIND_I8, OUT_I8, false);
  }
#undef HODU_TC
  *why = "output dtype has no tensor-core epilogue";
  return 1;
}
}  // namespace

}  // namespace hodu_b200
