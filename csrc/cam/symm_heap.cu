// Symmetric-heap runtime: one device slab per rank, exported with CUDA IPC and mapped by every peer of the box.
// This is the NVLink/NVSwitch counterpart of the HCCL "windows" that the reference kernels obtain from
// HcclOpResParam (src/cam/comm_operator/ascend_kernels/utils/op_kernel/moe_distribute_base.h:123-173): a table of
// peer base pointers that kernels dereference directly with loads, stores and atomics.
#include "common.h"

#include <string.h>

UMDK_API int umdk_symm_alloc(size_t bytes, void** out) {
  void* p = nullptr;
  UMDK_CUDA_CHECK(cudaMalloc(&p, bytes));
  UMDK_CUDA_CHECK(cudaMemset(p, 0, bytes));
  UMDK_CUDA_CHECK(cudaDeviceSynchronize());
  *out = p;
  return 0;
}

UMDK_API int umdk_symm_free(void* p) {
  UMDK_CUDA_CHECK(cudaFree(p));
  return 0;
}

// `handle` must have room for 64 bytes (sizeof(cudaIpcMemHandle_t)).
UMDK_API int umdk_symm_export(void* p, void* handle) {
  cudaIpcMemHandle_t h;
  UMDK_CUDA_CHECK(cudaIpcGetMemHandle(&h, p));
  memcpy(handle, &h, sizeof(h));
  return 0;
}

UMDK_API int umdk_symm_import(const void* handle, void** out) {
  cudaIpcMemHandle_t h;
  memcpy(&h, handle, sizeof(h));
  void* p = nullptr;
  UMDK_CUDA_CHECK(cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess));
  *out = p;
  return 0;
}

UMDK_API int umdk_symm_unimport(void* p) {
  UMDK_CUDA_CHECK(cudaIpcCloseMemHandle(p));
  return 0;
}

static long long g_rendezvous_ms = 16000;
UMDK_API void umdk_set_rendezvous_timeout_ms(int ms) { g_rendezvous_ms = ms > 0 ? ms : 16000; }
long long umdk_rendezvous_cycles() { return g_rendezvous_ms * 2000000LL; }   // the SM clock is just under 2 GHz

UMDK_API int umdk_ipc_handle_bytes() { return static_cast<int>(sizeof(cudaIpcMemHandle_t)); }

// Pinned, device-mapped host memory used to mirror small results (receive counts) to the CPU without a
// cudaMemcpy: the kernel stores to the device alias, the host polls the host alias.
UMDK_API int umdk_host_mapped_alloc(size_t bytes, void** host_ptr, void** dev_ptr) {
  void* h = nullptr;
  UMDK_CUDA_CHECK(cudaHostAlloc(&h, bytes, cudaHostAllocMapped));
  memset(h, 0, bytes);
  void* d = nullptr;
  UMDK_CUDA_CHECK(cudaHostGetDevicePointer(&d, h, 0));
  *host_ptr = h;
  *dev_ptr = d;
  return 0;
}

UMDK_API int umdk_host_mapped_free(void* host_ptr) {
  UMDK_CUDA_CHECK(cudaFreeHost(host_ptr));
  return 0;
}

UMDK_API int umdk_can_access_peer(int dev, int peer) {
  int ok = 0;
  if (cudaDeviceCanAccessPeer(&ok, dev, peer) != cudaSuccess) return 0;
  return ok;
}
