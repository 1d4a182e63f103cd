// Self-test kernel of the device-side symmetric-memory API (shmem_device.cuh): every operation is exercised against
// a peer's heap and checked by the host. Phase 1 of every PE (puts, signals, atomics) is launched before phase 2 of
// any PE (waits, gets), so several PEs can live on one GPU without a launch ever waiting on a later launch.
// Heap use: [0, 16 KiB) data slots of 1 KiB per source PE, [16 KiB, 17 KiB) signal words, [17 KiB, 18 KiB) atomics.
#include "shmem_device.cuh"

namespace umdk {
namespace {

constexpr int kSlotInts = 256;
constexpr uint64_t kSigOff = 16384, kAtomOff = 17408;

__global__ void shmem_selftest_kernel(shmem::Team tm, int phase, uint64_t tag, long long wait_limit, int* result) {
  uint8_t* self = tm.peers.base[tm.my_pe];
  int* slots = reinterpret_cast<int*>(self);
  uint64_t* sig = reinterpret_cast<uint64_t*>(self + kSigOff);
  uint64_t* atom64 = reinterpret_cast<uint64_t*>(self + kAtomOff);
  uint32_t* atom32 = reinterpret_cast<uint32_t*>(self + kAtomOff + 512);
  __shared__ int src[kSlotInts];
  const int right = (tm.my_pe + 1) % tm.n_pes, left = (tm.my_pe + tm.n_pes - 1) % tm.n_pes;
  if (phase == 1) {
    for (int i = threadIdx.x; i < kSlotInts; i += blockDim.x) src[i] = tm.my_pe * 1000 + i + (int)tag;
    __syncthreads();
    // CTA-wide put into my slot on the right neighbour, then one signal
    const bool ok = shmem::put_nbi_block(tm, slots + tm.my_pe * kSlotInts, src, kSlotInts, right);
    shmem::quiet_block();
    if (threadIdx.x == 0) {
      if (!ok) atomicOr(&result[0], 1);
      shmem::signal_set(tm, sig + tm.my_pe, tag, right);
      // atomics on PE 0
      shmem::atomic_add<uint64_t>(tm, atom64 + 0, (uint64_t)(tm.my_pe + 1), 0);
      shmem::atomic_or<uint64_t>(tm, atom64 + 1, 1ull << tm.my_pe, 0);
      shmem::atomic_xor<uint32_t>(tm, atom32 + 0, 1u << tm.my_pe, 0);
      shmem::atomic_inc<uint32_t>(tm, atom32 + 1, 0);
      const uint64_t old = shmem::atomic_compare_swap<uint64_t>(tm, atom64 + 2, 0ull, (uint64_t)(tm.my_pe + 1), 0);
      result[4] = (int)old;                                        // 0 for exactly one PE per run
      result[5] = (int)shmem::atomic_fetch_inc<uint32_t>(tm, atom32 + 2, 0);   // a permutation of 0..n-1
      shmem::atomic_and<uint32_t>(tm, atom32 + 3, ~(1u << tm.my_pe), 0);
      // an address outside the heap must be refused
      if (shmem::ptr(tm, reinterpret_cast<int*>(self + tm.heap_bytes), right) != nullptr) atomicOr(&result[0], 2);
      if (shmem::ptr(tm, slots, tm.n_pes) != nullptr) atomicOr(&result[0], 4);
      shmem::quiet();
    }
  } else if (phase == 2) {
    __shared__ int s_ok;
    if (threadIdx.x == 0) s_ok = shmem::signal_wait_until_ge(sig + left, tag, wait_limit) ? 1 : 0;
    __syncthreads();
    if (!s_ok) {
      if (threadIdx.x == 0) atomicOr(&result[0], 8);
      return;
    }
    // what the left neighbour put here
    int bad = 0;
    for (int i = threadIdx.x; i < kSlotInts; i += blockDim.x) {
      if (slots[left * kSlotInts + i] != left * 1000 + i + (int)tag) bad = 1;
    }
    // read my own slot back from the right neighbour with a warp-wide get
    if (threadIdx.x < 32) {
      shmem::get_nbi_warp(tm, src, slots + tm.my_pe * kSlotInts, kSlotInts, right);
    }
    __syncthreads();
    for (int i = threadIdx.x; i < kSlotInts; i += blockDim.x) {
      if (src[i] != tm.my_pe * 1000 + i + (int)tag) bad = 1;
    }
    if (bad) atomicOr(&result[0], 16);
    if (threadIdx.x == 0) {
      result[1] = (int)shmem::atomic_fetch<uint64_t>(tm, atom64 + 0, 0);
      result[2] = (int)shmem::atomic_fetch<uint64_t>(tm, atom64 + 1, 0);
      result[3] = (int)shmem::atomic_fetch<uint32_t>(tm, atom32 + 0, 0);
      result[6] = (int)shmem::atomic_fetch<uint32_t>(tm, atom32 + 1, 0);
      result[7] = (int)shmem::atomic_fetch<uint32_t>(tm, atom32 + 3, 0);
    }
  } else {
    // phase 3: a wait that nothing satisfies must come back with `false` within its budget
    if (threadIdx.x == 0) {
      const long long t0 = clock64();
      const bool got = shmem::signal_wait_until_ge(sig + 100, ~0ull, wait_limit);
      result[8] = got ? 1 : 0;
      result[9] = (int)((clock64() - t0) >> 10);
    }
  }
}

}  // namespace
}  // namespace umdk

using namespace umdk;

// peers: R base pointers; result: >= 10 ints on the device, zeroed by the caller before phase 1.
UMDK_API int umdk_shmem_selftest(void* const* peers, int R, int rank, uint64_t heap_bytes, int phase, uint64_t tag,
                                 long long wait_limit_cycles, int* result, void* stream) {
  if (R < 1 || R > kMaxRanks || rank < 0 || rank >= R || heap_bytes < 18432 || R > 16) return -UMDK_ERR_BAD_ARG;
  shmem::Team tm;
  for (int i = 0; i < kMaxRanks; ++i) tm.peers.base[i] = i < R ? static_cast<uint8_t*>(peers[i]) : nullptr;
  tm.heap_bytes = heap_bytes;
  tm.my_pe = rank;
  tm.n_pes = R;
  shmem_selftest_kernel<<<1, 128, 0, static_cast<cudaStream_t>(stream)>>>(tm, phase, tag, wait_limit_cycles, result);
  UMDK_CUDA_CHECK(cudaGetLastError());
  return 0;
}
