// Host/device shared definitions for the CAM CUDA library: status codes written by kernels whose bounded waits
// ran out, error-check macros, and the host-side TMA tensor-map builder.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>

#define UMDK_API extern "C" __attribute__((visibility("default")))

// Status word layout written to the caller-provided `int* status` (device memory, 4 ints):
//   [0] code (0 = ok), [1] phase/where, [2] detail a (e.g. source rank), [3] detail b
enum UmdkStatus : int {
  UMDK_OK = 0,
  UMDK_ERR_TIMEOUT = 1,      // a bounded spin-wait ran out of its cycle budget
  UMDK_ERR_BAD_ARG = 2,      // launcher rejected the arguments
  UMDK_ERR_OVERFLOW = 3,     // a receive slab / slot index went past its capacity (access skipped)
  UMDK_ERR_CUDA = 4,         // a CUDA runtime call failed on the host
};

enum UmdkPhase : int {
  UMDK_PH_NONE = 0,
  UMDK_PH_TMA_EMPTY = 1,
  UMDK_PH_TMA_FULL = 2,
  UMDK_PH_TMEM_FULL = 3,
  UMDK_PH_TMEM_EMPTY = 4,
  UMDK_PH_DISPATCH_COUNT = 5,
  UMDK_PH_DISPATCH_DATA = 6,
  UMDK_PH_COMBINE_DATA = 7,
  UMDK_PH_BARRIER = 8,
  UMDK_PH_GROUP_READY = 9,
  UMDK_PH_ALLREDUCE = 10,
  UMDK_PH_AG_CHUNK = 11,
  UMDK_PH_RS_CHUNK = 12,
};

#ifdef __CUDACC__
__device__ __forceinline__ void umdk_set_status(int* status, int code, int phase, int a = 0, int b = 0) {
  if (status != nullptr && atomicCAS(status, 0, code) == 0) {
    status[1] = phase;
    status[2] = a;
    status[3] = b;
  }
}
#endif

#define UMDK_CUDA_CHECK(expr)                                                                   \
  do {                                                                                          \
    cudaError_t _e = (expr);                                                                    \
    if (_e != cudaSuccess) {                                                                    \
      fprintf(stderr, "[umdk] CUDA error %s at %s:%d: %s\n", cudaGetErrorName(_e), __FILE__,    \
              __LINE__, cudaGetErrorString(_e));                                                \
      return -static_cast<int>(_e);                                                             \
    }                                                                                           \
  } while (0)

namespace umdk {

enum TmapDtype { TMAP_U8 = 0, TMAP_BF16 = 1, TMAP_F32 = 2 };
enum TmapSwizzle { TMAP_SW_NONE = 0, TMAP_SW_128B = 3 };

// Builds a 2-D tiled tensor map over a row-major [outer, inner] matrix whose rows are `row_stride_bytes` apart.
// Returns 0 on success. `base` must be 16-byte aligned and `row_stride_bytes` a multiple of 16.
int make_tmap_2d(CUtensorMap* out, TmapDtype dt, const void* base, uint64_t inner, uint64_t outer,
                 uint64_t row_stride_bytes, uint32_t box_inner, uint32_t box_outer, TmapSwizzle sw);

// 3-D variant: [d2, d1, inner] with byte strides for d1 and d2.
int make_tmap_3d(CUtensorMap* out, TmapDtype dt, const void* base, uint64_t inner, uint64_t d1, uint64_t d2,
                 uint64_t stride1_bytes, uint64_t stride2_bytes, uint32_t box_inner, uint32_t box1, uint32_t box2,
                 TmapSwizzle sw);

int sm_count();

}  // namespace umdk

// Budget of the waits at which a collective call MEETS its peers for the first time (the count exchange of the
// expert-parallel dispatches): ranks may enter a step seconds apart (allocation, graph capture, host work), so this
// wait is far more patient than the waits inside a call, which see their data within microseconds once every rank
// has arrived. Default 16 s; tests that make a wait run out set it to a fraction of a second.
UMDK_API void umdk_set_rendezvous_timeout_ms(int ms);
long long umdk_rendezvous_cycles();
