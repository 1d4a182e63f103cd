// Symmetric heap with an NVLink multicast (NVLS) mapping, built on the driver's virtual-memory-management calls.
//
// Every rank creates one physical allocation on its GPU (cuMemCreate, exportable as a POSIX file descriptor), maps it
// for itself, hands the descriptor to its peers (who map it too: the per-peer pointers kernels dereference) and binds
// it to a multicast object that rank 0 created for the group (cuMulticastCreate / AddDevice / BindMem). The multicast
// object is then mapped as one more address range: a `multimem.ld_reduce` on it returns the sum over all ranks'
// copies, computed inside NVSwitch, and a `multimem.st` / `multimem.red` reaches all copies.
//
// The calls are split into steps because the ranks have to meet between them (descriptors travel between processes,
// every device must be added before memory is bound); the Python side (umdk_b200/parallel/symm.py) runs the steps
// with `torch.distributed` collectives in between. File descriptors cross processes with pidfd_getfd(2), so no
// socket plumbing is needed: a rank publishes (pid, fd) and its peers duplicate the descriptor.
//
// The driver entry points are looked up at run time (cudaGetDriverEntryPoint): the library loads and the rest of it
// works on machines without a driver, and on GPUs without multicast support `umdk_mc_supported` says so.
//
// Same role as the HCCL window set-up that the reference's kernels rely on
// (src/cam/comm_operator/ascend_kernels/utils/op_kernel/moe_distribute_base.h:123-173), here for the NVSwitch
// in-network reduction.
#include <cuda.h>
#include <errno.h>
#include <stdint.h>
#include <stdio.h>
#include <sys/syscall.h>
#include <unistd.h>

#include <vector>

#include "common.h"

namespace {

struct Drv {
  bool ok = false;
  decltype(&cuDeviceGetAttribute) DeviceGetAttribute = nullptr;
  decltype(&cuMemCreate) MemCreate = nullptr;
  decltype(&cuMemRelease) MemRelease = nullptr;
  decltype(&cuMemAddressReserve) MemAddressReserve = nullptr;
  decltype(&cuMemAddressFree) MemAddressFree = nullptr;
  decltype(&cuMemMap) MemMap = nullptr;
  decltype(&cuMemUnmap) MemUnmap = nullptr;
  decltype(&cuMemSetAccess) MemSetAccess = nullptr;
  decltype(&cuMemGetAllocationGranularity) MemGetAllocationGranularity = nullptr;
  decltype(&cuMemExportToShareableHandle) MemExportToShareableHandle = nullptr;
  decltype(&cuMemImportFromShareableHandle) MemImportFromShareableHandle = nullptr;
  decltype(&cuMulticastCreate) MulticastCreate = nullptr;
  decltype(&cuMulticastAddDevice) MulticastAddDevice = nullptr;
  decltype(&cuMulticastBindMem) MulticastBindMem = nullptr;
  decltype(&cuMulticastUnbind) MulticastUnbind = nullptr;
  decltype(&cuMulticastGetGranularity) MulticastGetGranularity = nullptr;
};

template <typename F>
bool entry(const char* name, F* out) {
  void* p = nullptr;
  cudaDriverEntryPointQueryResult q;
  if (cudaGetDriverEntryPoint(name, &p, cudaEnableDefault, &q) != cudaSuccess || q != cudaDriverEntryPointSuccess || !p) {
    cudaGetLastError();
    return false;
  }
  *out = reinterpret_cast<F>(p);
  return true;
}

const Drv& drv() {
  static const Drv d = [] {
    Drv x;
    x.ok = entry("cuDeviceGetAttribute", &x.DeviceGetAttribute) && entry("cuMemCreate", &x.MemCreate) &&
           entry("cuMemRelease", &x.MemRelease) && entry("cuMemAddressReserve", &x.MemAddressReserve) &&
           entry("cuMemAddressFree", &x.MemAddressFree) && entry("cuMemMap", &x.MemMap) &&
           entry("cuMemUnmap", &x.MemUnmap) && entry("cuMemSetAccess", &x.MemSetAccess) &&
           entry("cuMemGetAllocationGranularity", &x.MemGetAllocationGranularity) &&
           entry("cuMemExportToShareableHandle", &x.MemExportToShareableHandle) &&
           entry("cuMemImportFromShareableHandle", &x.MemImportFromShareableHandle) &&
           entry("cuMulticastCreate", &x.MulticastCreate) && entry("cuMulticastAddDevice", &x.MulticastAddDevice) &&
           entry("cuMulticastBindMem", &x.MulticastBindMem) && entry("cuMulticastUnbind", &x.MulticastUnbind) &&
           entry("cuMulticastGetGranularity", &x.MulticastGetGranularity);
    return x;
  }();
  return d;
}

struct Mapping {
  CUdeviceptr va = 0;
  CUmemGenericAllocationHandle handle = 0;
  bool mapped = false;
};

struct McHeap {
  int device = 0;
  int num_devices = 0;
  size_t size = 0;          // padded to the larger of the two granularities
  Mapping local;            // this rank's physical memory
  int local_fd = -1;
  std::vector<Mapping> peers;
  CUmemGenericAllocationHandle mc = 0;
  bool have_mc = false, bound = false;
  int mc_fd = -1;
  CUdeviceptr mc_va = 0;
  bool mc_mapped = false;
};

#define MC_DRV_CHECK(call)                                                                     \
  do {                                                                                         \
    const CUresult r_ = (call);                                                                \
    if (r_ != CUDA_SUCCESS) {                                                                  \
      fprintf(stderr, "umdk symm_mc: %s failed with driver error %d (%s:%d)\n", #call, (int)r_, \
              __FILE__, __LINE__);                                                             \
      return -UMDK_ERR_CUDA;                                                                   \
    }                                                                                          \
  } while (0)

CUmulticastObjectProp mc_prop(int num_devices, size_t size) {
  CUmulticastObjectProp p{};
  p.numDevices = static_cast<unsigned>(num_devices);
  p.size = size;
  p.handleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
  return p;
}

int map_rw(const Drv& d, int device, CUmemGenericAllocationHandle h, size_t size, CUdeviceptr* va) {
  MC_DRV_CHECK(d.MemAddressReserve(va, size, 0, 0, 0));
  if (d.MemMap(*va, size, 0, h, 0) != CUDA_SUCCESS) {
    d.MemAddressFree(*va, size);
    *va = 0;
    return -UMDK_ERR_CUDA;
  }
  CUmemAccessDesc a{};
  a.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
  a.location.id = device;
  a.flags = CU_MEM_ACCESS_FLAGS_PROT_READWRITE;
  if (d.MemSetAccess(*va, size, &a, 1) != CUDA_SUCCESS) {
    d.MemUnmap(*va, size);
    d.MemAddressFree(*va, size);
    *va = 0;
    return -UMDK_ERR_CUDA;
  }
  return 0;
}

}  // namespace

// 1 when the current device (and the driver) can take part in a multicast object, 0 otherwise.
UMDK_API int umdk_mc_supported(void) {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) {
    cudaGetLastError();
    return 0;
  }
  const Drv& d = drv();
  if (!d.ok) return 0;
  int v = 0;
  if (d.DeviceGetAttribute(&v, CU_DEVICE_ATTRIBUTE_MULTICAST_SUPPORTED, dev) != CUDA_SUCCESS) return 0;
  return v ? 1 : 0;
}

// Step 1, every rank: physical memory of at least `bytes` on the current device, zeroed, mapped read-write, and a
// file descriptor for it. `*padded` is the size every later step uses (the same on all ranks for the same request).
UMDK_API int umdk_mc_local_create(size_t bytes, int num_devices, void** heap_out, void** local_ptr, int* fd_out,
                                  size_t* padded) {
  const Drv& d = drv();
  if (!d.ok || !heap_out || !local_ptr || !fd_out || !padded || num_devices < 1) return -UMDK_ERR_BAD_ARG;
  McHeap* h = new McHeap();
  UMDK_CUDA_CHECK(cudaGetDevice(&h->device));
  UMDK_CUDA_CHECK(cudaFree(nullptr));   // the driver calls below need the primary context to be current
  h->num_devices = num_devices;
  CUmemAllocationProp prop{};
  prop.type = CU_MEM_ALLOCATION_TYPE_PINNED;
  prop.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
  prop.location.id = h->device;
  prop.requestedHandleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
  size_t g_mem = 0, g_mc = 0;
  MC_DRV_CHECK(d.MemGetAllocationGranularity(&g_mem, &prop, CU_MEM_ALLOC_GRANULARITY_RECOMMENDED));
  const CUmulticastObjectProp mp = mc_prop(num_devices, bytes);
  MC_DRV_CHECK(d.MulticastGetGranularity(&g_mc, &mp, CU_MULTICAST_GRANULARITY_RECOMMENDED));
  const size_t g = g_mem > g_mc ? g_mem : g_mc;
  h->size = (bytes + g - 1) / g * g;
  MC_DRV_CHECK(d.MemCreate(&h->local.handle, h->size, &prop, 0));
  if (map_rw(d, h->device, h->local.handle, h->size, &h->local.va) != 0) {
    d.MemRelease(h->local.handle);
    delete h;
    return -UMDK_ERR_CUDA;
  }
  h->local.mapped = true;
  UMDK_CUDA_CHECK(cudaMemset(reinterpret_cast<void*>(h->local.va), 0, h->size));
  UMDK_CUDA_CHECK(cudaDeviceSynchronize());
  MC_DRV_CHECK(d.MemExportToShareableHandle(&h->local_fd, h->local.handle, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR, 0));
  *heap_out = h;
  *local_ptr = reinterpret_cast<void*>(h->local.va);
  *fd_out = h->local_fd;
  *padded = h->size;
  return 0;
}

// Step 2, rank 0 only: the multicast object of the group and a descriptor for it.
UMDK_API int umdk_mc_group_create(void* heap, int* mc_fd_out) {
  const Drv& d = drv();
  McHeap* h = static_cast<McHeap*>(heap);
  if (!h || !mc_fd_out) return -UMDK_ERR_BAD_ARG;
  const CUmulticastObjectProp mp = mc_prop(h->num_devices, h->size);
  MC_DRV_CHECK(d.MulticastCreate(&h->mc, &mp));
  h->have_mc = true;
  MC_DRV_CHECK(d.MemExportToShareableHandle(&h->mc_fd, h->mc, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR, 0));
  *mc_fd_out = h->mc_fd;
  return 0;
}

// Step 2, the other ranks: take the multicast object from a descriptor that is valid in THIS process.
UMDK_API int umdk_mc_group_import(void* heap, int mc_fd) {
  const Drv& d = drv();
  McHeap* h = static_cast<McHeap*>(heap);
  if (!h || mc_fd < 0) return -UMDK_ERR_BAD_ARG;
  MC_DRV_CHECK(d.MemImportFromShareableHandle(&h->mc, reinterpret_cast<void*>(static_cast<intptr_t>(mc_fd)),
                                              CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR));
  h->have_mc = true;
  return 0;
}

// Step 3, every rank: join the object. All ranks must have done this before any of them binds memory.
UMDK_API int umdk_mc_add_device(void* heap) {
  const Drv& d = drv();
  McHeap* h = static_cast<McHeap*>(heap);
  if (!h || !h->have_mc) return -UMDK_ERR_BAD_ARG;
  MC_DRV_CHECK(d.MulticastAddDevice(h->mc, h->device));
  return 0;
}

// Step 4, every rank (after a barrier): bind the local memory at offset 0 and map the object. `*mc_ptr` is the
// address `multimem` instructions use; offsets into it equal offsets into every rank's local memory.
UMDK_API int umdk_mc_bind_map(void* heap, void** mc_ptr) {
  const Drv& d = drv();
  McHeap* h = static_cast<McHeap*>(heap);
  if (!h || !h->have_mc || !mc_ptr) return -UMDK_ERR_BAD_ARG;
  MC_DRV_CHECK(d.MulticastBindMem(h->mc, 0, h->local.handle, 0, h->size, 0));
  h->bound = true;
  if (map_rw(d, h->device, h->mc, h->size, &h->mc_va) != 0) return -UMDK_ERR_CUDA;
  h->mc_mapped = true;
  *mc_ptr = reinterpret_cast<void*>(h->mc_va);
  return 0;
}

// Maps a peer's memory from a descriptor that is valid in this process.
UMDK_API int umdk_mc_import_peer(void* heap, int fd, void** ptr) {
  const Drv& d = drv();
  McHeap* h = static_cast<McHeap*>(heap);
  if (!h || fd < 0 || !ptr) return -UMDK_ERR_BAD_ARG;
  Mapping m;
  MC_DRV_CHECK(d.MemImportFromShareableHandle(&m.handle, reinterpret_cast<void*>(static_cast<intptr_t>(fd)),
                                              CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR));
  if (map_rw(d, h->device, m.handle, h->size, &m.va) != 0) {
    d.MemRelease(m.handle);
    return -UMDK_ERR_CUDA;
  }
  m.mapped = true;
  h->peers.push_back(m);
  *ptr = reinterpret_cast<void*>(m.va);
  return 0;
}

// Unmaps everything and releases the handles. Call it on every rank with no kernel in flight; the multicast object
// itself goes away when the last rank has released it.
UMDK_API int umdk_mc_destroy(void* heap) {
  const Drv& d = drv();
  McHeap* h = static_cast<McHeap*>(heap);
  if (!h) return 0;
  cudaDeviceSynchronize();
  if (h->mc_mapped) {
    d.MemUnmap(h->mc_va, h->size);
    d.MemAddressFree(h->mc_va, h->size);
  }
  if (h->bound) d.MulticastUnbind(h->mc, h->device, 0, h->size);
  if (h->have_mc) d.MemRelease(h->mc);
  for (Mapping& m : h->peers) {
    if (m.mapped) {
      d.MemUnmap(m.va, h->size);
      d.MemAddressFree(m.va, h->size);
    }
    d.MemRelease(m.handle);
  }
  if (h->local.mapped) {
    d.MemUnmap(h->local.va, h->size);
    d.MemAddressFree(h->local.va, h->size);
  }
  if (h->local.handle) d.MemRelease(h->local.handle);
  if (h->local_fd >= 0) close(h->local_fd);
  if (h->mc_fd >= 0) close(h->mc_fd);
  delete h;
  return 0;
}

// Duplicates descriptor `fd` of process `pid` into this process (pidfd_open + pidfd_getfd). The kernel allows it to
// a process that may ptrace the other one: root, or the same user where the ptrace scope permits it; where it does
// not, this returns -EPERM, the heap set-up fails on every rank together and the callers stay on the peer-pointer
// algorithms. Returns the new descriptor or a negative errno.
UMDK_API int umdk_fd_from_process(int pid, int fd) {
#if defined(SYS_pidfd_open) && defined(SYS_pidfd_getfd)
  const int pidfd = static_cast<int>(syscall(SYS_pidfd_open, pid, 0));
  if (pidfd < 0) return -errno;
  const int got = static_cast<int>(syscall(SYS_pidfd_getfd, pidfd, fd, 0));
  const int err = errno;
  close(pidfd);
  return got < 0 ? -err : got;
#else
  (void)pid;
  (void)fd;
  return -ENOSYS;
#endif
}
