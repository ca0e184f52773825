// Thin inline-PTX wrappers for the sm_100a features the GEMM kernels use:
// mbarrier, TMA tiled loads (no multicast), tcgen05 alloc / mma / commit / ld.
// Everything here is device-only and has no state.
#pragma once
#include <cuda.h>
#include <stdint.h>

namespace hodu_b200 {
namespace ptx {

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ uint64_t globaltimer_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

// ---------------------------------------------------------------- programmatic dependent launch
// A kernel launched with the programmatic-stream-serialisation attribute may start while the
// kernel before it in the stream is still running.  `grid_dependency_wait` returns once that
// earlier kernel has finished and its writes are visible (at once when there is none, or when
// the launch did not carry the attribute); `grid_launch_dependents` lets the NEXT kernel in the
// stream start its own set-up early.
__device__ __forceinline__ void grid_dependency_wait() {
  asm volatile("griddepcontrol.wait;" ::: "memory");
}
__device__ __forceinline__ void grid_launch_dependents() {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}

// ---------------------------------------------------------------- mbarrier
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void fence_barrier_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void fence_proxy_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes)
               : "memory");
}
// The producer's arrive publishes no ordinary writes (TMA completion is tracked by the
// transaction count), so it needs no release ordering.
__device__ __forceinline__ void mbar_arrive_expect_tx_relaxed(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.relaxed.cta.shared::cta.b64 _, [%0], %1;" ::"r"(bar),
               "r"(bytes)
               : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t"
      "}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}

// Non-blocking probe of a phase (never suspends the thread).
__device__ __forceinline__ bool mbar_test_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t"
      "}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}

// Remote arrive on the same-offset barrier of another CTA of the cluster.
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t bar, uint32_t cta_rank) {
  asm volatile(
      "{\n\t"
      ".reg .b32 remote;\n\t"
      "mapa.shared::cluster.u32 remote, %0, %1;\n\t"
      "mbarrier.arrive.release.cluster.shared::cluster.b64 _, [remote];\n\t"
      "}" ::"r"(bar),
      "r"(cta_rank)
      : "memory");
}

// ---------------------------------------------------------------- TMA
__device__ __forceinline__ void prefetch_tensormap(const CUtensorMap* m) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(m)) : "memory");
}

// Tiled 5-D load global -> this CTA's shared memory, completion on an mbarrier of this CTA.
// c0 is the innermost coordinate; c0 * element size must be a multiple of 16 bytes.
__device__ __forceinline__ void tma_load_5d(uint32_t dst, const CUtensorMap* map, uint32_t bar,
                                            int32_t c0, int32_t c1, int32_t c2, int32_t c3,
                                            int32_t c4) {
  asm volatile(
      "cp.async.bulk.tensor.5d.shared::cluster.global.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4, %5, %6, %7}], [%2];" ::"r"(dst),
      "l"(reinterpret_cast<uint64_t>(map)), "r"(bar), "r"(c0), "r"(c1), "r"(c2), "r"(c3), "r"(c4)
      : "memory");
}

// Tiled 2-D load global -> this CTA's shared memory, completion on an mbarrier of this CTA.
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int32_t c0, int32_t c1) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];" ::"r"(dst),
      "l"(reinterpret_cast<uint64_t>(map)), "r"(bar), "r"(c0), "r"(c1)
      : "memory");
}

// The same load issued by one CTA of a 2-CTA pair: data lands in the issuing CTA's
// shared memory, completion may be signalled on an mbarrier of either CTA of the pair
// (`bar` is a shared::cluster address, see mapa_shared).
__device__ __forceinline__ void tma_load_5d_pair(uint32_t dst, const CUtensorMap* map, uint32_t bar,
                                                 int32_t c0, int32_t c1, int32_t c2, int32_t c3,
                                                 int32_t c4) {
  asm volatile(
      "cp.async.bulk.tensor.5d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4, %5, %6, %7}], [%2];" ::"r"(dst),
      "l"(reinterpret_cast<uint64_t>(map)), "r"(bar), "r"(c0), "r"(c1), "r"(c2), "r"(c3), "r"(c4)
      : "memory");
}

// Tiled 3-D store of this CTA's shared memory to global memory (bulk async group completion).
// c0 is the innermost coordinate; c0 * element size must be a multiple of 16 bytes and no
// coordinate may be negative.  Elements of the box that fall outside the tensor are not written.
__device__ __forceinline__ void tma_store_3d(const CUtensorMap* map, uint32_t src, int32_t c0, int32_t c1, int32_t c2) {
  asm volatile("cp.async.bulk.tensor.3d.global.shared::cta.tile.bulk_group [%0, {%2, %3, %4}], [%1];" ::"l"(
                   reinterpret_cast<uint64_t>(map)),
               "r"(src), "r"(c0), "r"(c1), "r"(c2)
               : "memory");
}
__device__ __forceinline__ void bulk_commit_group() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
// Waits until at most N of this thread's bulk groups still READ their shared-memory source.
template <int N> __device__ __forceinline__ void bulk_wait_group_read() {
  asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}

// shared::cta address -> shared::cluster address of the same offset in CTA `cta_rank`.
__device__ __forceinline__ uint32_t mapa_shared(uint32_t addr, uint32_t cta_rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(cta_rank));
  return r;
}
// 16 bytes of another CTA's shared memory (shared::cluster address from mapa_shared).
__device__ __forceinline__ uint4 ld_cluster_v4(uint32_t cluster_addr) {
  uint4 v;
  asm volatile("ld.shared::cluster.v4.b32 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "r"(cluster_addr)
               : "memory");
  return v;
}
// Arrive (+ expected transaction bytes) on an mbarrier given by a shared::cluster address.
__device__ __forceinline__ void mbar_arrive_expect_tx_cluster(uint32_t cluster_bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.release.cluster.shared::cluster.b64 _, [%0], %1;" ::"r"(
                   cluster_bar),
               "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void mbar_arrive_cluster_addr(uint32_t cluster_bar) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_bar)
               : "memory");
}

// ---------------------------------------------------------------- tcgen05
template <int CTA_GROUP>
__device__ __forceinline__ void tmem_alloc(uint32_t smem_result, uint32_t ncols) {
  if constexpr (CTA_GROUP == 1)
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                     smem_result),
                 "r"(ncols)
                 : "memory");
  else
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                     smem_result),
                 "r"(ncols)
                 : "memory");
}
template <int CTA_GROUP>
__device__ __forceinline__ void tmem_relinquish() {
  if constexpr (CTA_GROUP == 1)
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  else
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
template <int CTA_GROUP>
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
  if constexpr (CTA_GROUP == 1)
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols)
                 : "memory");
  else
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols)
                 : "memory");
}
__device__ __forceinline__ void tc_fence_before_sync() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after_sync() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}

// MMA kinds (compile-time: they select the PTX opcode).
enum : int { KIND_F16 = 0, KIND_TF32 = 1, KIND_F8 = 2, KIND_I8 = 3 };

// D[tmem] (+)= A[smem desc] * B[smem desc]; issued by ONE thread.
template <int KIND, int CTA_GROUP>
__device__ __forceinline__ void umma(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc,
                                     uint32_t idesc, uint32_t accumulate) {
#define HODU_UMMA(KSTR, GSTR)                                                             \
  asm volatile(                                                                           \
      "{\n\t"                                                                             \
      ".reg .pred p;\n\t"                                                                 \
      "setp.ne.b32 p, %4, 0;\n\t"                                                         \
      "tcgen05.mma.cta_group::" GSTR ".kind::" KSTR " [%0], %1, %2, %3, p;\n\t"           \
      "}" ::"r"(d_tmem),                                                                  \
      "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)                               \
      : "memory")
  if constexpr (CTA_GROUP == 1) {
    if constexpr (KIND == KIND_F16) HODU_UMMA("f16", "1");
    else if constexpr (KIND == KIND_TF32) HODU_UMMA("tf32", "1");
    else if constexpr (KIND == KIND_F8) HODU_UMMA("f8f6f4", "1");
    else HODU_UMMA("i8", "1");
  } else {
    if constexpr (KIND == KIND_F16) HODU_UMMA("f16", "2");
    else if constexpr (KIND == KIND_TF32) HODU_UMMA("tf32", "2");
    else if constexpr (KIND == KIND_F8) HODU_UMMA("f8f6f4", "2");
    else HODU_UMMA("i8", "2");
  }
#undef HODU_UMMA
}

// The four MMAs of one stage into one accumulator as ONE asm block: descriptor low words are
// (a_lo + k * a_step, b_lo + k * b_step), the high words are shared.  The issuing thread is the
// bottleneck of the main loop (every scalar instruction of its stream is serial latency), so
// the block spends two adds and two register-pair moves per MMA and nothing else.
// `first` = 0 makes the first MMA overwrite the accumulator instead of adding to it.
template <int KIND, int CTA_GROUP>
__device__ __forceinline__ void umma_x4(uint32_t d_tmem, uint32_t a_lo, uint32_t a_hi, uint32_t a_step,
                                        uint32_t b_lo, uint32_t b_hi, uint32_t b_step, uint32_t idesc,
                                        uint32_t first) {
#define HODU_UMMA4(KSTR, GSTR)                                                                    \
  asm volatile(                                                                                   \
      "{\n\t"                                                                                     \
      ".reg .pred p, t;\n\t"                                                                      \
      ".reg .b64 da, db;\n\t"                                                                     \
      ".reg .b32 al, bl;\n\t"                                                                     \
      "setp.ne.b32 p, %8, 0;\n\t"                                                                 \
      "setp.eq.u32 t, 0, 0;\n\t"                                                                  \
      "mov.b64 da, {%1, %2};\n\t"                                                                 \
      "mov.b64 db, {%4, %5};\n\t"                                                                 \
      "tcgen05.mma.cta_group::" GSTR ".kind::" KSTR " [%0], da, db, %7, p;\n\t"                   \
      "add.u32 al, %1, %3;\n\t"                                                                   \
      "add.u32 bl, %4, %6;\n\t"                                                                   \
      "mov.b64 da, {al, %2};\n\t"                                                                 \
      "mov.b64 db, {bl, %5};\n\t"                                                                 \
      "tcgen05.mma.cta_group::" GSTR ".kind::" KSTR " [%0], da, db, %7, t;\n\t"                   \
      "add.u32 al, al, %3;\n\t"                                                                   \
      "add.u32 bl, bl, %6;\n\t"                                                                   \
      "mov.b64 da, {al, %2};\n\t"                                                                 \
      "mov.b64 db, {bl, %5};\n\t"                                                                 \
      "tcgen05.mma.cta_group::" GSTR ".kind::" KSTR " [%0], da, db, %7, t;\n\t"                   \
      "add.u32 al, al, %3;\n\t"                                                                   \
      "add.u32 bl, bl, %6;\n\t"                                                                   \
      "mov.b64 da, {al, %2};\n\t"                                                                 \
      "mov.b64 db, {bl, %5};\n\t"                                                                 \
      "tcgen05.mma.cta_group::" GSTR ".kind::" KSTR " [%0], da, db, %7, t;\n\t"                   \
      "}" ::"r"(d_tmem),                                                                          \
      "r"(a_lo), "r"(a_hi), "r"(a_step), "r"(b_lo), "r"(b_hi), "r"(b_step), "r"(idesc), "r"(first) \
      : "memory")
  if constexpr (CTA_GROUP == 1) {
    if constexpr (KIND == KIND_F16) HODU_UMMA4("f16", "1");
    else if constexpr (KIND == KIND_TF32) HODU_UMMA4("tf32", "1");
    else if constexpr (KIND == KIND_F8) HODU_UMMA4("f8f6f4", "1");
    else HODU_UMMA4("i8", "1");
  } else {
    if constexpr (KIND == KIND_F16) HODU_UMMA4("f16", "2");
    else if constexpr (KIND == KIND_TF32) HODU_UMMA4("tf32", "2");
    else if constexpr (KIND == KIND_F8) HODU_UMMA4("f8f6f4", "2");
    else HODU_UMMA4("i8", "2");
  }
#undef HODU_UMMA4
}

// Make an mbarrier of THIS CTA track completion of all MMAs issued so far by
// this thread.
__device__ __forceinline__ void umma_commit_1cta(uint32_t bar) {
  asm volatile(
      "tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar)
      : "memory");
}
// 2-CTA form: arrive on the same-offset barrier in each CTA selected by mask.
// (commit with cluster multicast signals barriers only; it moves no tile data.)
__device__ __forceinline__ void umma_commit_2cta(uint32_t bar, uint16_t cta_mask) {
  asm volatile(
      "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64"
      " [%0], %1;" ::"r"(bar),
      "h"(cta_mask)
      : "memory");
}

// 32 lanes x 32 columns of 32-bit: thread t of the warp receives columns
// [col, col+32) of TMEM lane (lane_base + t).
__device__ __forceinline__ void tmem_ld_32x32(uint32_t taddr, uint32_t (&v)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]),
        "=r"(v[7]), "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]),
        "=r"(v[14]), "=r"(v[15]), "=r"(v[16]), "=r"(v[17]), "=r"(v[18]), "=r"(v[19]),
        "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]), "=r"(v[24]), "=r"(v[25]),
        "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_wait_ld() {
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
// The two halves of a cluster-wide barrier: every thread of every CTA arrives, and may do work
// that needs nothing from its peers before it waits.  A completed cluster barrier also orders the
// threads of ONE CTA among themselves, so it stands in for __syncthreads() where both are due.
__device__ __forceinline__ void cluster_arrive() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
}
__device__ __forceinline__ void cluster_wait() {
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;"
               ::: "memory");
}
// The same barrier without memory ordering: for a rendezvous that only has to keep a CTA (its
// shared memory, its barriers, its TMEM) alive until its peers are done with it.  The release
// form would first wait for every global store of the arriving thread to complete.
__device__ __forceinline__ void cluster_sync_all_relaxed() {
  asm volatile("barrier.cluster.arrive.relaxed.aligned;\n\tbarrier.cluster.wait.aligned;" ::: "memory");
}

}  // namespace ptx
}  // namespace hodu_b200
