// Allocation-free variant of the dispatch-layout entry point. It has no counterpart in the reference project.
//
// Who needs it: code that is not allowed to ask the CUDA driver for memory at the point where it computes a
// routing layout. Typical cases are a serving engine that hands every free byte of device memory to its KV-cache
// pool at start-up (a later cudaMalloc would simply fail), a custom-op plug-in running inside another runtime's
// "enqueue" hook where allocation is forbidden by contract, and latency-critical decode loops that cannot afford
// the implicit device synchronisation of cudaMalloc / cudaFree. Such callers can still own the input and output
// buffers (they were carved out of their own pool), but they have nowhere to get the kernel's scratch from.
//
// What it does: the same computation as `umdk_ep_layout`, with the per-chunk histogram scratch and the grid-barrier
// words kept in one file-scope `__device__` array inside the library. The array is UMDK_EP_LAYOUT_NOALLOC_BYTES
// (about 0.55 MB) of device memory on every GPU that loads the library, held until the process exits.
//
// Limits: T <= UMDK_EP_LAYOUT_NOALLOC_MAX_TOKENS and num_experts + num_ranks <= UMDK_EP_LAYOUT_NOALLOC_MAX_COLS;
// anything larger is rejected with -2 (bad argument) and a message on stderr - nothing is launched.
//
// Rules for callers:
//   * The first call on a device looks up the array's device address (cudaGetSymbolAddress, once per device, with
//     that device current). Make that first call during start-up, before any stream capture begins.
//   * The array itself becomes resident when the CUDA driver loads this library's module on a device. With CUDA's
//     default lazy module loading that happens at the first call of this entry point, or at any earlier kernel of
//     this library on that device - not at dlopen time. A process that later gives away all free device memory
//     must therefore make that first call (or run any other kernel of the library) BEFORE it does so; after the
//     module is loaded, calls neither take nor return device memory.
//   * The address is cached per device ordinal. cudaDeviceReset destroys the context the address belongs to; a
//     process that resets a device must not call this entry point on that device afterwards.
//   * All calls on one device share the array. Two calls whose kernels may overlap on the GPU (different streams
//     without an ordering between them) race on it; keep calls on one stream or order them with events.
//   * Nothing in the array has to survive between calls. The barrier words are reset on the caller's stream at the
//     start of every call; the histogram part is fully rewritten by the kernel before it is read.
//   * The entry point itself calls no cudaMalloc, cudaFree or allocating library routine, on the first call or
//     later; the only memory event is the driver's one-time module load described above.
#pragma once
#include <stdint.h>

#define UMDK_EP_LAYOUT_NOALLOC_MAX_TOKENS 8192
#define UMDK_EP_LAYOUT_NOALLOC_MAX_COLS 544 /* num_experts + num_ranks, e.g. 512 experts + 32 ranks */
#define UMDK_EP_LAYOUT_NOALLOC_BYTES (256 + 4 * (UMDK_EP_LAYOUT_NOALLOC_MAX_TOKENS / 32) * UMDK_EP_LAYOUT_NOALLOC_MAX_COLS)

#ifdef __cplusplus
extern "C" {
#endif

// Same arguments and results as umdk_ep_layout minus the scratch and barrier pointers. All pointers are device
// pointers owned by the caller: topk_idx [T, K] int64 in; num_per_expert [E], num_per_rank [R] int32,
// in_rank [T, R] uint8, send_idx [T, K] int32, rank_slot [T, R] int32 out; status: 4 ints, zeroed by the caller.
// Returns 0, or a negative error code (-2: argument or size limit, other: -cudaError).
int umdk_ep_layout_noalloc(const int64_t* topk_idx, int T, int K, int E, int R, int* num_per_expert,
                           int* num_per_rank, uint8_t* in_rank, int* send_idx, int* rank_slot, int* status,
                           void* stream);

#ifdef __cplusplus
}
#endif
