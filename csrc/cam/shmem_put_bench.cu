// Put-bandwidth probe of the symmetric heap: copies `rows` rows of `row_bytes` from local memory to (scattered) rows
// of a destination that may be a peer's heap, with the access patterns the communication kernels use, so that the
// link rate each pattern reaches can be measured in isolation (the role urma_perftest's write-bandwidth test plays
// for the host path, tools/urma_perftest/perftest_run_test.c in the reference).
//   mode 0  grid-stride stream of 16-byte stores over the whole range (the all-reduce pattern)
//   mode 1  one warp per row: 16-byte loads, then 16-byte stores (the dispatch / combine pattern)
//   mode 2  one warp per row: loads into a shared-memory stage, then one bulk shared->global copy per piece
//   mode 3  one warp per row: bulk global->shared load, then bulk shared->global store (no register path)
#include "ptx.cuh"
#include "common.h"

namespace umdk {
namespace {

__device__ __forceinline__ size_t scatter_row(size_t r, size_t rows) { return (r * 9973u + 17u) % rows; }

__global__ void __launch_bounds__(512, 1) shmem_put_bench_kernel(uint8_t* dst, const uint8_t* src, size_t rows,
                                                                  int row_bytes, int piece, int mode, int* status) {
  extern __shared__ __align__(128) uint8_t smem[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;
  if (mode == 0) {
    const size_t nvec = rows * (size_t)row_bytes / 16;
    const int4* s = reinterpret_cast<const int4*>(src);
    int4* d = reinterpret_cast<int4*>(dst);
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t v = (size_t)blockIdx.x * blockDim.x + threadIdx.x; v < nvec; v += 4 * stride) {
      int4 r[4];
#pragma unroll
      for (int u = 0; u < 4; ++u)
        if (v + u * stride < nvec) r[u] = ld_nc_v4(s + v + u * stride);
#pragma unroll
      for (int u = 0; u < 4; ++u)
        if (v + u * stride < nvec) st_na_v4(d + v + u * stride, r[u]);
    }
    return;
  }
  const int nvec = row_bytes / 16;
  if (mode == 1) {
    for (size_t r = (size_t)blockIdx.x * nwarps + warp; r < rows; r += (size_t)gridDim.x * nwarps) {
      const int4* s = reinterpret_cast<const int4*>(src + r * row_bytes);
      int4* d = reinterpret_cast<int4*>(dst + scatter_row(r, rows) * row_bytes);
      for (int v0 = 0; v0 < nvec; v0 += 8 * 32) {
        int4 x[8];
#pragma unroll
        for (int u = 0; u < 8; ++u)
          if (v0 + u * 32 + lane < nvec) x[u] = ld_nc_v4(s + v0 + u * 32 + lane);
#pragma unroll
        for (int u = 0; u < 8; ++u)
          if (v0 + u * 32 + lane < nvec) st_na_v4(d + v0 + u * 32 + lane, x[u]);
      }
    }
    return;
  }
  uint8_t* stage = smem + (size_t)warp * 2 * piece;   // two pieces per warp
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + (size_t)nwarps * 2 * piece) + warp * 2;
  uint32_t use[2] = {0, 0};
  if (mode == 3 && lane == 0) {
    mbar_init(&bars[0], 1);
    mbar_init(&bars[1], 1);
    mbar_fence_init();
  }
  __syncwarp();
  int b = 0;
  bool ok = true;
  for (size_t r = (size_t)blockIdx.x * nwarps + warp; r < rows && ok; r += (size_t)gridDim.x * nwarps) {
    const uint8_t* s = src + r * row_bytes;
    uint8_t* d = dst + scatter_row(r, rows) * row_bytes;
    for (int off = 0; off < row_bytes; off += piece, b ^= 1) {
      const int n = min(piece, row_bytes - off);
      if (lane == 0) tma_store_wait_read<1>();   // the copy that last read this buffer has drained it
      __syncwarp();
      if (mode == 2) {
        const int4* sv = reinterpret_cast<const int4*>(s + off);
        int4* bv = reinterpret_cast<int4*>(stage + (size_t)b * piece);
        for (int v0 = 0; v0 < n / 16; v0 += 8 * 32) {
          int4 x[8];
#pragma unroll
          for (int u = 0; u < 8; ++u)
            if (v0 + u * 32 + lane < n / 16) x[u] = ld_nc_v4(sv + v0 + u * 32 + lane);
#pragma unroll
          for (int u = 0; u < 8; ++u)
            if (v0 + u * 32 + lane < n / 16) bv[v0 + u * 32 + lane] = x[u];
        }
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) {
          bulk_store_1d(d + off, stage + (size_t)b * piece, (uint32_t)n);
          tma_store_commit();
        }
      } else if (lane == 0) {
        mbar_expect_tx(&bars[b], (uint32_t)n);
        bulk_load_1d(stage + (size_t)b * piece, s + off, (uint32_t)n, &bars[b]);
        if (!mbar_wait(&bars[b], use[b] & 1)) {
          umdk_set_status(status, UMDK_ERR_TIMEOUT, UMDK_PH_TMA_FULL, warp, (int)r);
          ok = false;
        } else {
          ++use[b];
          bulk_store_1d(d + off, stage + (size_t)b * piece, (uint32_t)n);
          tma_store_commit();
        }
      }
      ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
      if (!ok) break;
    }
  }
  if (lane == 0) tma_store_wait<0>();
}

}  // namespace
}  // namespace umdk

using namespace umdk;

// dst / src: 16-byte aligned; row_bytes a multiple of 16; piece (modes 2, 3) a multiple of 16 up to 16 KiB.
UMDK_API int umdk_shmem_put_bench(void* dst, const void* src, long long rows, int row_bytes, int piece, int mode,
                                  int grid, int* status, void* stream) {
  if (!dst || !src || rows < 1 || row_bytes < 16 || (row_bytes % 16) || mode < 0 || mode > 3 || grid < 1)
    return -UMDK_ERR_BAD_ARG;
  int threads = 512;
  size_t smem = 0;
  if (mode >= 2) {
    if (piece < 16 || (piece % 16) || piece > 16384) return -UMDK_ERR_BAD_ARG;
    while (threads > 64 && (size_t)(threads / 32) * 2 * piece > 160 * 1024) threads /= 2;
    smem = (size_t)(threads / 32) * (2 * piece + 16);
    UMDK_CUDA_CHECK(cudaFuncSetAttribute(shmem_put_bench_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  }
  shmem_put_bench_kernel<<<grid, threads, smem, static_cast<cudaStream_t>(stream)>>>(
      static_cast<uint8_t*>(dst), static_cast<const uint8_t*>(src), (size_t)rows, row_bytes, piece, mode, status);
  UMDK_CUDA_CHECK(cudaGetLastError());
  return 0;
}
