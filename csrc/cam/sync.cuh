// Flag and barrier primitives for kernels that talk to peer GPUs or to other CTAs of the same grid.
//
// All flags are monotone epoch values: a writer publishes `epoch + 1` with a system-scope release store and a reader
// polls with system-scope acquire loads until it sees a value >= the one it expects. Nothing is ever cleared, so a
// stale value from an earlier launch can never satisfy a wait, and consecutive launches need no barrier between them
// (the buffers they guard are double-buffered on epoch parity). This follows the "magic << 32 | value, compare >="
// idiom of the reference's SyncCollectives (src/cam/comm_operator/ascend_kernels/utils/op_kernel/sync_collectives.h:303-347),
// but unlike the reference's operator kernels (unbounded spins, e.g. moe_dispatch_normal.h:495) every wait here has
// a cycle budget and reports a status instead of hanging.
#pragma once
#include "common.h"
#include "ptx.cuh"

namespace umdk {

// Polls *flag (system scope) until it is >= want. Returns false on timeout.
__device__ __forceinline__ bool wait_flag_ge_sys(const uint64_t* flag, uint64_t want,
                                                 long long limit = kSpinLimitCycles) {
  if (ld_acquire_sys(flag) >= want) return true;
  const long long t0 = clock64();
  while (ld_acquire_sys(flag) < want) {
    if (clock64() - t0 > limit) return false;
    __nanosleep(20);
  }
  return true;
}
__device__ __forceinline__ bool wait_flag_ge_sys(const uint32_t* flag, uint32_t want,
                                                 long long limit = kSpinLimitCycles) {
  if (ld_acquire_sys(flag) >= want) return true;
  const long long t0 = clock64();
  while (ld_acquire_sys(flag) < want) {
    if (clock64() - t0 > limit) return false;
    __nanosleep(20);
  }
  return true;
}
__device__ __forceinline__ bool wait_flag_ge_gpu(const uint32_t* flag, uint32_t want,
                                                 long long limit = kSpinLimitCycles) {
  if (ld_acquire_gpu(flag) >= want) return true;
  const long long t0 = clock64();
  while (ld_acquire_gpu(flag) < want) {
    if (clock64() - t0 > limit) return false;
    __nanosleep(20);
  }
  return true;
}

// Grid-wide barrier for co-resident grids (grid size <= number of CTAs the device can hold at once).
// `bar[0]` is the arrival counter, `bar[1]` the generation. Called by all threads of every CTA.
// Returns false if the generation did not advance within the cycle budget.
__device__ __forceinline__ bool grid_barrier(uint32_t* bar, uint32_t num_ctas) {
  __shared__ int s_ok;
  __syncthreads();
  if (threadIdx.x == 0) {
    s_ok = 1;
    const uint32_t gen = ld_acquire_gpu(&bar[1]);
    __threadfence();
    const uint32_t old = atomicAdd(&bar[0], 1u);
    if (old == num_ctas - 1) {
      bar[0] = 0;
      __threadfence();
      red_add_release_gpu(&bar[1], 1u);
    } else {
      const long long t0 = clock64();
      while (ld_acquire_gpu(&bar[1]) == gen) {
        if (clock64() - t0 > kSpinLimitCycles) {
          s_ok = 0;
          break;
        }
        __nanosleep(20);
      }
    }
    __threadfence();
  }
  __syncthreads();
  return s_ok != 0;
}

// "Last CTA" detector: every CTA calls it once when its part of a phase is complete (all threads, after their
// stores). Returns true in exactly one CTA - the last to arrive - and resets the counter for the next launch.
__device__ __forceinline__ bool cta_done_is_last(uint32_t* counter, uint32_t num_ctas) {
  __shared__ int s_last;
  // All threads' stores are ordered before the barrier; one system-scope fence by the thread that signals then
  // orders them (cumulatively) before the counter update, the same shape as a cooperative grid barrier.
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence_system();
    const uint32_t old = atomicAdd(counter, 1u);
    s_last = (old == num_ctas - 1) ? 1 : 0;
    if (s_last) {
      *counter = 0;
      __threadfence_system();
    }
  }
  __syncthreads();
  return s_last != 0;
}

}  // namespace umdk
