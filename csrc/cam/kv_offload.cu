// KV-cache offload to pinned host DRAM and asynchronous prefetch back, on a dedicated copy stream.
//
// Pages are fixed-size blobs (64 tokens x 576 bf16 = 73,728 bytes for the MLA cache). The manager owns a pinned
// host pool and a non-blocking side stream; `offload` copies device pages out, `prefetch` copies host pages into
// device slots with cudaMemcpyAsync - runs of pages that are consecutive on both sides are merged into one copy so
// a whole sequence (or a whole layer) moves with a single large transfer. Events order the copies against the
// compute stream in both directions (data ready before attention reads it; attention finished before the slots are
// overwritten by the next prefetch). There is no KV-cache code in the reference project (its roadmap lists
// "KVCache transfer" as future work, src/cam/README.md:21-23); this is specified by the serving configuration.
//
// Second prefetch form, for sparse attention: `umdk_kv_prefetch_rows` runs a gather kernel on the same side stream
// that reads ONLY the selected token rows of host-resident pages straight out of the pinned pool (the pool is mapped
// into the device address space, so the loads travel over PCIe as 512-byte warp requests) and lands them in a small
// device area; the index list is rewritten so that attention finds those rows there. With top-2048 of 32768 tokens
// selected per query this moves 1/16 of the bytes of a page-granular prefetch and needs 1/8 of the landing memory.
#include "common.h"

#include <stdlib.h>
#include <string.h>

#include <vector>

namespace {

struct KvGatherArgs {
  const int* indices;       // [B, topk] token positions (-1 = unused)
  const int* host_table;    // [B, n_log_pages] host slot of each logical page, -1 if the page is on the device
  const uint8_t* host_pool; // device alias of the pinned pool
  uint8_t* landing;         // [B * topk] rows on the device
  int* indices_out;         // [B, topk] positions for attention: unchanged, or virt_base + i for a landed row
  unsigned long long* row_counter;
  int* status;
  long long host_rows;      // rows in the pool (bounds check)
  int B, topk, n_log_pages, page_tokens, row_bytes, virt_base;
};

// One warp per selected row. Rows of device-resident pages are left where they are. The launch uses a handful of
// 1024-thread CTAs: the transfer is PCIe-bound, a few hundred KB of loads in flight saturate the link, and a small
// grid occupies only that many SMs, so a persistent compute kernel that runs at the same time on the other SMs
// (one CTA per SM, all registers) is not held up.
__global__ void __launch_bounds__(1024) kv_gather_rows_kernel(const KvGatherArgs a) {
  const int lane = threadIdx.x & 31;
  const int warps = gridDim.x * (blockDim.x >> 5);
  const int total = a.B * a.topk;
  const int nvec = a.row_bytes >> 4;
  unsigned long long moved = 0;
  for (int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); row < total; row += warps) {
    const int b = row / a.topk, i = row - b * a.topk;
    const int idx = a.indices[row];
    int out = idx;
    if (idx >= 0) {
      const int page = idx / a.page_tokens;
      if (page < a.n_log_pages) {
        const int slot = a.host_table[(size_t)b * a.n_log_pages + page];
        if (slot >= 0) {
          const long long hrow = (long long)slot * a.page_tokens + (idx - page * a.page_tokens);
          if (hrow >= a.host_rows) {
            if (lane == 0) umdk_set_status(a.status, UMDK_ERR_OVERFLOW, UMDK_PH_NONE, b, slot);
            out = -1;
          } else {
            const int4* s = reinterpret_cast<const int4*>(a.host_pool + (size_t)hrow * a.row_bytes);
            int4* d = reinterpret_cast<int4*>(a.landing + (size_t)row * a.row_bytes);
            for (int c = lane; c < nvec; c += 32) d[c] = __ldcs(s + c);
            out = a.virt_base + i;
            ++moved;
          }
        }
      }
    }
    if (lane == 0) a.indices_out[row] = out;
  }
  if (lane == 0 && moved && a.row_counter) atomicAdd(a.row_counter, moved);
}

struct KvOffload {
  size_t page_bytes = 0;
  size_t host_pages = 0;
  uint8_t* host_pool = nullptr;
  uint8_t* host_pool_dev = nullptr;    // the same memory as seen from kernels
  unsigned long long* row_counter = nullptr;  // device: host rows fetched by the gather kernel so far
  cudaStream_t copy_stream = nullptr;
  bool own_stream = true;
  std::vector<cudaEvent_t> ready;      // per channel: prefetch finished
  std::vector<cudaEvent_t> consumed;   // per channel: compute finished reading the prefetched slots
  std::vector<char> consumed_valid;
  unsigned long long bytes_h2d = 0, bytes_d2h = 0, copies = 0;
};

}  // namespace

// `stream`: side stream to use (owned by the caller, must outlive the manager), or nullptr to create one.
UMDK_API void* umdk_kv_create_on_stream(size_t page_bytes, size_t host_pages, int channels, void* stream) {
  if (page_bytes == 0 || (page_bytes % 16) || host_pages == 0 || channels < 1 || channels > 1024) return nullptr;
  KvOffload* k = new KvOffload();
  k->page_bytes = page_bytes;
  k->host_pages = host_pages;
  if (cudaHostAlloc(reinterpret_cast<void**>(&k->host_pool), page_bytes * host_pages,
                    cudaHostAllocMapped | cudaHostAllocPortable) != cudaSuccess) {
    cudaGetLastError();
    delete k;
    return nullptr;
  }
  if (cudaHostGetDevicePointer(reinterpret_cast<void**>(&k->host_pool_dev), k->host_pool, 0) != cudaSuccess) {
    cudaGetLastError();
    k->host_pool_dev = nullptr;  // page-granular copies still work; the row gather reports an error
  }
  if (cudaMalloc(reinterpret_cast<void**>(&k->row_counter), 8) == cudaSuccess) {
    cudaMemset(k->row_counter, 0, 8);
  } else {
    cudaGetLastError();
    k->row_counter = nullptr;
  }
  if (stream) {
    k->copy_stream = static_cast<cudaStream_t>(stream);
    k->own_stream = false;
  } else if (cudaStreamCreateWithFlags(&k->copy_stream, cudaStreamNonBlocking) != cudaSuccess) {
    cudaFreeHost(k->host_pool);
    delete k;
    return nullptr;
  }
  k->ready.resize(channels);
  k->consumed.resize(channels);
  k->consumed_valid.assign(channels, 0);
  for (int i = 0; i < channels; ++i) {
    cudaEventCreateWithFlags(&k->ready[i], cudaEventDisableTiming);
    cudaEventCreateWithFlags(&k->consumed[i], cudaEventDisableTiming);
  }
  return k;
}

UMDK_API void* umdk_kv_create(size_t page_bytes, size_t host_pages, int channels) {
  return umdk_kv_create_on_stream(page_bytes, host_pages, channels, nullptr);
}

UMDK_API void umdk_kv_destroy(void* h) {
  KvOffload* k = static_cast<KvOffload*>(h);
  if (!k) return;
  cudaStreamSynchronize(k->copy_stream);
  for (auto e : k->ready) cudaEventDestroy(e);
  for (auto e : k->consumed) cudaEventDestroy(e);
  if (k->own_stream) cudaStreamDestroy(k->copy_stream);
  cudaFreeHost(k->host_pool);
  if (k->row_counter) cudaFree(k->row_counter);
  delete k;
}

UMDK_API void* umdk_kv_host_pool(void* h) { return static_cast<KvOffload*>(h)->host_pool; }
UMDK_API void* umdk_kv_copy_stream(void* h) { return static_cast<KvOffload*>(h)->copy_stream; }

// Copies n pages: host_slots[i] <-> dev_pages[i] (indices into the host pool / the device pool at dev_pool).
// to_host != 0: device -> host (offload), else host -> device (prefetch). Consecutive runs become one copy.
static int copy_pages(KvOffload* k, void* dev_pool, const int* dev_pages, const int* host_slots, int n, int to_host) {
  int i = 0;
  while (i < n) {
    int j = i + 1;
    while (j < n && dev_pages[j] == dev_pages[j - 1] + 1 && host_slots[j] == host_slots[j - 1] + 1) ++j;
    if (host_slots[i] < 0 || (size_t)host_slots[j - 1] >= k->host_pages || dev_pages[i] < 0) return -UMDK_ERR_BAD_ARG;
    uint8_t* d = static_cast<uint8_t*>(dev_pool) + (size_t)dev_pages[i] * k->page_bytes;
    uint8_t* hp = k->host_pool + (size_t)host_slots[i] * k->page_bytes;
    const size_t bytes = (size_t)(j - i) * k->page_bytes;
    if (to_host) {
      UMDK_CUDA_CHECK(cudaMemcpyAsync(hp, d, bytes, cudaMemcpyDeviceToHost, k->copy_stream));
      k->bytes_d2h += bytes;
    } else {
      UMDK_CUDA_CHECK(cudaMemcpyAsync(d, hp, bytes, cudaMemcpyHostToDevice, k->copy_stream));
      k->bytes_h2d += bytes;
    }
    ++k->copies;
    i = j;
  }
  return 0;
}

// Device -> host. The copy stream first waits for `compute_stream` (the producer of the pages), if given.
UMDK_API int umdk_kv_offload(void* h, void* dev_pool, const int* dev_pages, const int* host_slots, int n,
                             void* compute_stream) {
  KvOffload* k = static_cast<KvOffload*>(h);
  {
    cudaEvent_t e;
    UMDK_CUDA_CHECK(cudaEventCreateWithFlags(&e, cudaEventDisableTiming));
    UMDK_CUDA_CHECK(cudaEventRecord(e, static_cast<cudaStream_t>(compute_stream)));
    UMDK_CUDA_CHECK(cudaStreamWaitEvent(k->copy_stream, e, 0));
    UMDK_CUDA_CHECK(cudaEventDestroy(e));
  }
  return copy_pages(k, dev_pool, dev_pages, host_slots, n, 1);
}

// Host -> device on the copy stream. If the channel's slots were read by an earlier compute step
// (umdk_kv_release), the copies wait for that step first. Marks the channel ready when the copies land.
UMDK_API int umdk_kv_prefetch(void* h, int channel, void* dev_pool, const int* dev_pages, const int* host_slots,
                              int n) {
  KvOffload* k = static_cast<KvOffload*>(h);
  if (channel < 0 || channel >= (int)k->ready.size()) return -UMDK_ERR_BAD_ARG;
  if (k->consumed_valid[channel]) UMDK_CUDA_CHECK(cudaStreamWaitEvent(k->copy_stream, k->consumed[channel], 0));
  if (int rc = copy_pages(k, dev_pool, dev_pages, host_slots, n, 0)) return rc;
  UMDK_CUDA_CHECK(cudaEventRecord(k->ready[channel], k->copy_stream));
  return 0;
}

// Row-granular prefetch for sparse attention (see the top of the file). The gather kernel runs on the copy stream
// after (a) everything queued so far on `compute_stream` if `after_compute` is set (the indices were produced there;
// pass 0 when they are already final or were written on the copy stream itself), and (b) the last reader of the
// channel's landing area. landing: [B * topk] rows of row_bytes; indices_out: [B, topk].
UMDK_API int umdk_kv_prefetch_rows(void* h, int channel, const int* indices, const int* host_table, void* landing,
                                   int* indices_out, int B, int topk, int n_log_pages, int page_tokens, int row_bytes,
                                   int virt_base, int* status, int after_compute, int num_ctas, void* compute_stream) {
  KvOffload* k = static_cast<KvOffload*>(h);
  if (channel < 0 || channel >= (int)k->ready.size() || B < 1 || topk < 1 || n_log_pages < 1 || page_tokens < 1 ||
      row_bytes < 16 || (row_bytes % 16) || (size_t)page_tokens * row_bytes != k->page_bytes)
    return -UMDK_ERR_BAD_ARG;
  if (!k->host_pool_dev) return -UMDK_ERR_CUDA;
  if (after_compute) {
    cudaEvent_t e;
    UMDK_CUDA_CHECK(cudaEventCreateWithFlags(&e, cudaEventDisableTiming));
    UMDK_CUDA_CHECK(cudaEventRecord(e, static_cast<cudaStream_t>(compute_stream)));
    UMDK_CUDA_CHECK(cudaStreamWaitEvent(k->copy_stream, e, 0));
    UMDK_CUDA_CHECK(cudaEventDestroy(e));
  }
  if (k->consumed_valid[channel]) UMDK_CUDA_CHECK(cudaStreamWaitEvent(k->copy_stream, k->consumed[channel], 0));
  KvGatherArgs a;
  a.indices = indices;
  a.host_table = host_table;
  a.host_pool = k->host_pool_dev;
  a.landing = static_cast<uint8_t*>(landing);
  a.indices_out = indices_out;
  a.row_counter = k->row_counter;
  a.status = status;
  a.host_rows = (long long)k->host_pages * page_tokens;
  a.B = B;
  a.topk = topk;
  a.n_log_pages = n_log_pages;
  a.page_tokens = page_tokens;
  a.row_bytes = row_bytes;
  a.virt_base = virt_base;
  const long long rows = (long long)B * topk;
  int grid = num_ctas > 0 ? num_ctas : 8;
  if (grid > (rows + 31) / 32) grid = (int)((rows + 31) / 32);
  if (grid > umdk::sm_count()) grid = umdk::sm_count();
  kv_gather_rows_kernel<<<grid, 1024, 0, k->copy_stream>>>(a);
  UMDK_CUDA_CHECK(cudaGetLastError());
  UMDK_CUDA_CHECK(cudaEventRecord(k->ready[channel], k->copy_stream));
  return 0;
}

// Host rows fetched by the gather kernel since creation (synchronises the copy stream).
UMDK_API long long umdk_kv_rows_fetched(void* h) {
  KvOffload* k = static_cast<KvOffload*>(h);
  if (!k->row_counter) return -1;
  unsigned long long v = 0;
  if (cudaStreamSynchronize(k->copy_stream) != cudaSuccess ||
      cudaMemcpy(&v, k->row_counter, 8, cudaMemcpyDeviceToHost) != cudaSuccess)
    return -1;
  return (long long)v;
}

// Makes `compute_stream` wait until the channel's prefetch has landed.
UMDK_API int umdk_kv_wait(void* h, int channel, void* compute_stream) {
  KvOffload* k = static_cast<KvOffload*>(h);
  if (channel < 0 || channel >= (int)k->ready.size()) return -UMDK_ERR_BAD_ARG;
  UMDK_CUDA_CHECK(cudaStreamWaitEvent(static_cast<cudaStream_t>(compute_stream), k->ready[channel], 0));
  return 0;
}

// Records that everything queued so far on `compute_stream` is the last reader of the channel's slots.
UMDK_API int umdk_kv_release(void* h, int channel, void* compute_stream) {
  KvOffload* k = static_cast<KvOffload*>(h);
  if (channel < 0 || channel >= (int)k->ready.size()) return -UMDK_ERR_BAD_ARG;
  UMDK_CUDA_CHECK(cudaEventRecord(k->consumed[channel], static_cast<cudaStream_t>(compute_stream)));
  k->consumed_valid[channel] = 1;
  return 0;
}

UMDK_API int umdk_kv_sync(void* h) {
  KvOffload* k = static_cast<KvOffload*>(h);
  UMDK_CUDA_CHECK(cudaStreamSynchronize(k->copy_stream));
  return 0;
}

UMDK_API void umdk_kv_stats(void* h, unsigned long long* out3) {
  KvOffload* k = static_cast<KvOffload*>(h);
  out3[0] = k->bytes_h2d;
  out3[1] = k->bytes_d2h;
  out3[2] = k->copies;
}
