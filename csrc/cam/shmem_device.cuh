// Device-side symmetric-memory API: put / get / quiet / atomics / signals on a peer GPU's part of the symmetric heap,
// callable from inside any kernel.
//
// The reference exposes the same operation set as "NDA" device-initiated RDMA, where a kernel fills a work-queue
// entry, rings the doorbell of a queue pair and polls its completion queue
// (src/cam/framework/nda/include/device/gm2gm/engine/shmem_device_rdma.h:26-401: roce_ptr, get_nbi, put_nbi, quiet,
// atomic fetch / set / compare_swap / swap / inc / add / and / or / xor and their fetch_ forms;
// src/cam/framework/nda/src/device/gm2gm/engine/rdma_backends/rdma_device_backend_base.h:55-325 for the WQE path).
// Inside one NVSwitch domain no queue pair is needed: every peer's heap is mapped into this GPU's address space, so
// a put is a vectorised store, a get a vectorised load, an atomic an `atom.sys`, and quiet a system-scope fence.
// The operation names and argument order follow the reference so that kernels written against it carry over.
//
// Addresses are symmetric: the caller passes the address of the object in ITS OWN heap together with a processing
// element (pe) number, and `ptr()` rebases it onto the peer's mapping. Objects outside the heap are rejected
// (nullptr), not dereferenced.
#pragma once
#include "ep_common.cuh"
#include "ptx.cuh"
#include "sync.cuh"

namespace umdk {
namespace shmem {

struct Team {
  PeerTable peers;     // base address of every PE's heap as mapped on this GPU
  uint64_t heap_bytes;
  int my_pe, n_pes;
};

// Peer address of a symmetric object (nullptr if `local` is not inside this PE's heap or pe is out of range).
template <typename T>
__device__ __forceinline__ T* ptr(const Team& tm, const T* local, int pe) {
  const uint64_t off = reinterpret_cast<const uint8_t*>(local) - tm.peers.base[tm.my_pe];
  if (pe < 0 || pe >= tm.n_pes || off >= tm.heap_bytes) return nullptr;
  return reinterpret_cast<T*>(tm.peers.base[pe] + off);
}

// ---- put / get (non-blocking: complete at the next quiet()) --------------------------------------------------
// Called by ONE thread: copies elem_count elements one by one (small control messages).
template <typename T>
__device__ __forceinline__ bool put_nbi(const Team& tm, T* dst, const T* src, uint32_t elem_count, int pe) {
  T* d = ptr(tm, dst, pe);
  if (!d) return false;
  for (uint32_t i = 0; i < elem_count; ++i) d[i] = src[i];
  return true;
}
template <typename T>
__device__ __forceinline__ bool get_nbi(const Team& tm, T* dst, const T* src, uint32_t elem_count, int pe) {
  const T* s = ptr(tm, src, pe);
  if (!s) return false;
  for (uint32_t i = 0; i < elem_count; ++i) dst[i] = s[i];
  return true;
}

// Called by ALL threads of a warp / of a CTA with the same arguments: 16-byte vector copies striped over the
// threads, scalar tail. Both addresses must be 16-byte aligned for the vector part to be used.
__device__ __forceinline__ void copy_striped(uint8_t* d, const uint8_t* s, size_t bytes, int tid, int nthreads) {
  if (((reinterpret_cast<uintptr_t>(d) | reinterpret_cast<uintptr_t>(s)) & 15) == 0) {
    const size_t nvec = bytes / 16;
    for (size_t i = tid; i < nvec; i += nthreads) {
      reinterpret_cast<int4*>(d)[i] = reinterpret_cast<const int4*>(s)[i];
    }
    for (size_t i = nvec * 16 + tid; i < bytes; i += nthreads) d[i] = s[i];
  } else {
    for (size_t i = tid; i < bytes; i += nthreads) d[i] = s[i];
  }
}
template <typename T>
__device__ __forceinline__ bool put_nbi_warp(const Team& tm, T* dst, const T* src, uint32_t elem_count, int pe) {
  T* d = ptr(tm, dst, pe);
  if (!d) return false;
  copy_striped(reinterpret_cast<uint8_t*>(d), reinterpret_cast<const uint8_t*>(src), sizeof(T) * (size_t)elem_count,
               threadIdx.x & 31, 32);
  return true;
}
template <typename T>
__device__ __forceinline__ bool get_nbi_warp(const Team& tm, T* dst, const T* src, uint32_t elem_count, int pe) {
  const T* s = ptr(tm, src, pe);
  if (!s) return false;
  copy_striped(reinterpret_cast<uint8_t*>(dst), reinterpret_cast<const uint8_t*>(s), sizeof(T) * (size_t)elem_count,
               threadIdx.x & 31, 32);
  return true;
}
template <typename T>
__device__ __forceinline__ bool put_nbi_block(const Team& tm, T* dst, const T* src, uint32_t elem_count, int pe) {
  T* d = ptr(tm, dst, pe);
  if (!d) return false;
  copy_striped(reinterpret_cast<uint8_t*>(d), reinterpret_cast<const uint8_t*>(src), sizeof(T) * (size_t)elem_count,
               threadIdx.x, blockDim.x);
  return true;
}
template <typename T>
__device__ __forceinline__ bool get_nbi_block(const Team& tm, T* dst, const T* src, uint32_t elem_count, int pe) {
  const T* s = ptr(tm, src, pe);
  if (!s) return false;
  copy_striped(reinterpret_cast<uint8_t*>(dst), reinterpret_cast<const uint8_t*>(s), sizeof(T) * (size_t)elem_count,
               threadIdx.x, blockDim.x);
  return true;
}

// Orders all earlier puts / atomics of the calling thread before anything it does afterwards, system wide.
// (The reference polls the completion queue of the queue pair here; a fence is the whole job on NVLink.)
__device__ __forceinline__ void quiet() { __threadfence_system(); }
// CTA-wide form: every thread's earlier puts are visible system wide when it returns.
__device__ __forceinline__ void quiet_block() {
  __threadfence_system();
  __syncthreads();
}

// ---- atomics (32- and 64-bit integers) -------------------------------------------------------------------------
template <typename T> struct AtomWord;
template <> struct AtomWord<int32_t> { using type = int; };
template <> struct AtomWord<uint32_t> { using type = unsigned int; };
template <> struct AtomWord<int64_t> { using type = unsigned long long; };
template <> struct AtomWord<uint64_t> { using type = unsigned long long; };
template <typename T> using atom_word_t = typename AtomWord<T>::type;

#define UMDK_SHMEM_RMW(name, expr)                                                                   \
  template <typename T>                                                                              \
  __device__ __forceinline__ T atomic_fetch_##name(const Team& tm, T* dst, T value, int pe) {        \
    using W = atom_word_t<T>;                                                                        \
    W* d = reinterpret_cast<W*>(ptr(tm, dst, pe));                                                   \
    if (!d) return T(0);                                                                             \
    const W v = static_cast<W>(value);                                                               \
    return static_cast<T>(expr);                                                                     \
  }                                                                                                  \
  template <typename T>                                                                              \
  __device__ __forceinline__ void atomic_##name(const Team& tm, T* dst, T value, int pe) {           \
    (void)atomic_fetch_##name(tm, dst, value, pe);                                                   \
  }
UMDK_SHMEM_RMW(add, atomicAdd_system(d, v))
UMDK_SHMEM_RMW(and, atomicAnd_system(d, v))
UMDK_SHMEM_RMW(or, atomicOr_system(d, v))
UMDK_SHMEM_RMW(xor, atomicXor_system(d, v))
#undef UMDK_SHMEM_RMW

template <typename T>
__device__ __forceinline__ T atomic_fetch_inc(const Team& tm, T* dst, int pe) {
  return atomic_fetch_add<T>(tm, dst, T(1), pe);
}
template <typename T>
__device__ __forceinline__ void atomic_inc(const Team& tm, T* dst, int pe) {
  (void)atomic_fetch_add<T>(tm, dst, T(1), pe);
}
template <typename T>
__device__ __forceinline__ T atomic_swap(const Team& tm, T* dst, T value, int pe) {
  using W = atom_word_t<T>;
  W* d = reinterpret_cast<W*>(ptr(tm, dst, pe));
  if (!d) return T(0);
  return static_cast<T>(atomicExch_system(d, static_cast<W>(value)));
}
template <typename T>
__device__ __forceinline__ T atomic_compare_swap(const Team& tm, T* dst, T cond, T value, int pe) {
  using W = atom_word_t<T>;
  W* d = reinterpret_cast<W*>(ptr(tm, dst, pe));
  if (!d) return T(0);
  return static_cast<T>(atomicCAS_system(d, static_cast<W>(cond), static_cast<W>(value)));
}
template <typename T>
__device__ __forceinline__ T atomic_fetch(const Team& tm, const T* src, int pe) {
  using W = atom_word_t<T>;
  W* s = reinterpret_cast<W*>(const_cast<T*>(ptr(tm, src, pe)));
  if (!s) return T(0);
  return static_cast<T>(atomicOr_system(s, W(0)));
}
template <typename T>
__device__ __forceinline__ void atomic_set(const Team& tm, T* dst, T value, int pe) {
  (void)atomic_swap<T>(tm, dst, value, pe);
}

// ---- signals ---------------------------------------------------------------------------------------------------
// put-with-signal: data first, then a release store of the signal word on the same PE (one thread; for a CTA-wide
// put call put_nbi_block, quiet_block, and signal from one thread).
__device__ __forceinline__ bool signal_set(const Team& tm, uint64_t* sig, uint64_t value, int pe) {
  uint64_t* s = ptr(tm, sig, pe);
  if (!s) return false;
  st_release_sys(s, value);
  return true;
}
// Waits until the LOCAL signal word is >= value; false after the cycle budget (nothing hangs).
__device__ __forceinline__ bool signal_wait_until_ge(const uint64_t* sig, uint64_t value,
                                                     long long limit = kSpinLimitCycles) {
  return wait_flag_ge_sys(sig, value, limit);
}

}  // namespace shmem
}  // namespace umdk
