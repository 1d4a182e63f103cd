// KV-cache offload to pinned host DRAM and asynchronous prefetch back, on a dedicated copy stream.
//
// Pages are fixed-size blobs (64 tokens x 576 bf16 = 73,728 bytes for the MLA cache). The manager owns a pinned
// host pool and a non-blocking side stream; `offload` copies device pages out, `prefetch` copies host pages into
// device slots with cudaMemcpyAsync - runs of pages that are consecutive on both sides are merged into one copy so
// a whole sequence (or a whole layer) moves with a single large transfer. Events order the copies against the
// compute stream in both directions (data ready before attention reads it; attention finished before the slots are
// overwritten by the next prefetch). There is no KV-cache code in the reference project (its roadmap lists
// "KVCache transfer" as future work, src/cam/README.md:21-23); this is specified by the serving configuration.
#include "common.h"

#include <stdlib.h>
#include <string.h>

#include <vector>

namespace {

struct KvOffload {
  size_t page_bytes = 0;
  size_t host_pages = 0;
  uint8_t* host_pool = nullptr;
  cudaStream_t copy_stream = nullptr;
  std::vector<cudaEvent_t> ready;      // per channel: prefetch finished
  std::vector<cudaEvent_t> consumed;   // per channel: compute finished reading the prefetched slots
  std::vector<char> consumed_valid;
  unsigned long long bytes_h2d = 0, bytes_d2h = 0, copies = 0;
};

}  // namespace

UMDK_API void* umdk_kv_create(size_t page_bytes, size_t host_pages, int channels) {
  if (page_bytes == 0 || (page_bytes % 16) || host_pages == 0 || channels < 1 || channels > 1024) return nullptr;
  KvOffload* k = new KvOffload();
  k->page_bytes = page_bytes;
  k->host_pages = host_pages;
  if (cudaHostAlloc(reinterpret_cast<void**>(&k->host_pool), page_bytes * host_pages, cudaHostAllocDefault) !=
      cudaSuccess) {
    delete k;
    return nullptr;
  }
  if (cudaStreamCreateWithFlags(&k->copy_stream, cudaStreamNonBlocking) != cudaSuccess) {
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

UMDK_API void umdk_kv_destroy(void* h) {
  KvOffload* k = static_cast<KvOffload*>(h);
  if (!k) return;
  cudaStreamSynchronize(k->copy_stream);
  for (auto e : k->ready) cudaEventDestroy(e);
  for (auto e : k->consumed) cudaEventDestroy(e);
  cudaStreamDestroy(k->copy_stream);
  cudaFreeHost(k->host_pool);
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
