// Bounded waits on mbarriers, shared by the tensor-core kernels.  Every wait polls `try_wait`
// with a time limit and a per-CTA abort flag; a wait that runs out records a code in the device
// status word (first one wins), raises the flag so that the CTA's other roles stop too, and
// returns false: the kernel then drains what it started, frees its TMEM and returns normally.
#pragma once
#include <stdint.h>

#include "sm100_ptx.cuh"

namespace hodu_b200 {

constexpr uint64_t kWaitLimitNs = 2000000000ull;

__device__ __forceinline__ bool wait_bounded(uint32_t bar, uint32_t parity,
                                             volatile uint32_t* abort_flag, uint32_t* status,
                                             uint32_t code, uint64_t limit_ns = kWaitLimitNs) {
  using namespace ptx;
  if (mbar_try_wait(bar, parity)) return true;
  uint64_t t0 = 0;
  for (uint32_t i = 1;; ++i) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((i & 0xFFu) == 0) {
      if (*abort_flag) return false;
      const uint64_t now = globaltimer_ns();
      if (t0 == 0) {
        t0 = now;
      } else if (now - t0 > limit_ns) {
        *abort_flag = 1;
        atomicCAS(status, 0u, code);
        return false;
      }
    }
  }
}
// Used only after an abort: give work already in flight a short time to land.
__device__ __forceinline__ void wait_drain(uint32_t bar, uint32_t parity) {
  using namespace ptx;
  const uint64_t t0 = globaltimer_ns();
  for (uint32_t i = 0; i < (1u << 22); ++i) {
    if (mbar_try_wait(bar, parity)) return;
    if ((i & 0xFFu) == 0xFFu && globaltimer_ns() - t0 > 200000000ull) return;
  }
}

}  // namespace hodu_b200
