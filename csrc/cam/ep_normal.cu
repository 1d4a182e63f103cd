// Normal-mode (prefill / high-throughput) expert-parallel kernels: layout, dispatch, combine.
//
// What the reference does (Ascend, src/cam/comm_operator/ascend_kernels/):
//   dispatch_layout/op_kernel/dispatch_layout.h:112-165   per-expert histogram + per-(token,k) bucket slot
//   notify_dispatch/op_kernel/notify_dispatch.h:91-110     all-to-all of per-expert counts, prefix sums
//   moe_dispatch_normal/op_kernel/moe_dispatch_normal.h:346-591  per-(token,k) record written to the sender's own
//       window, flag per (expert, srcRank), receiver pulls records
//   moe_combine_normal/op_kernel/moe_combine_normal.h:224-377    push rows to the owner's (t*K+k) slot, weighted sum
//
// What this file does instead (B200, NVLink 5 through NVSwitch, peer pointers from the symmetric heap):
//   * ep_layout: one launch; stable bucket positions for (token,k) per expert AND per destination rank.
//   * ep_dispatch: ONE kernel = notify + quantise + push + expand. Each token crosses NVLink once per destination
//     rank (the reference sends it once per expert), already quantised to fp8 e4m3 with one fp32 scale per 1x128
//     block, using 16-byte stores into the receiver's arrival buffer; the receiver then expands arrivals into the
//     expert-major / source-rank-minor slab that the grouped GEMM consumes (same order as the reference's
//     recv_x: index = localExpert * R + srcRank, notify_dispatch.h:264-412).
//   * ep_combine: expert side pre-reduces the rows of one token on this rank (fp32), pushes one bf16 row per
//     (token, rank) to the owner, owner sums over ranks. A row-per-(token,k) mode reproduces the reference's
//     stateless moe_combine_prefill contract.
// Flags are epoch-tagged and buffers are double-buffered on epoch parity, so no barrier is needed between calls.
#include "ep_common.cuh"
#include "ptx.cuh"
#include "sync.cuh"

namespace umdk {
namespace {

constexpr int kLayoutWarps = 8;
constexpr int kEpThreads = 512;
constexpr int kEpWarps = kEpThreads / 32;

// ------------------------------------------------------------------------------------------------------------
// Layout
// ------------------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(kLayoutWarps * 32)
ep_layout_kernel(const int64_t* __restrict__ topk_idx, int T, int K, int E, int R, int* __restrict__ num_per_expert,
                 int* __restrict__ num_per_rank, uint8_t* __restrict__ in_rank, int* __restrict__ send_idx,
                 int* __restrict__ rank_slot, int* __restrict__ scratch, uint32_t* bar, int* status) {
  extern __shared__ int sm_layout[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int cols = E + R;
  const int E_local = E / R;
  int* hist = sm_layout + warp * cols;
  int* stage = sm_layout + kLayoutWarps * cols + warp * 32 * kMaxTopk;
  const int num_chunks = (T + 31) / 32;
  const int gwarp = blockIdx.x * kLayoutWarps + warp;
  const int total_warps = gridDim.x * kLayoutWarps;

  // Phase A: per-chunk histograms and positions inside the chunk (stable in token order).
  for (int c = gwarp; c < num_chunks; c += total_warps) {
    for (int i = lane; i < cols; i += 32) hist[i] = 0;
    const int t0 = c * 32;
    const int nt = min(32, T - t0);
    for (int i = lane; i < nt * K; i += 32) {
      long long e = topk_idx[(size_t)t0 * K + i];
      stage[i] = (e >= 0 && e < E) ? (int)e : -1;
    }
    __syncwarp();
    for (int i = 0; i < nt; ++i) {
      const int t = t0 + i;
      const int e = lane < K ? stage[i * K + lane] : -1;
      const uint32_t rm = __reduce_or_sync(0xffffffffu, e >= 0 ? (1u << (e / E_local)) : 0u);
      if (lane < K) send_idx[(size_t)t * K + lane] = e >= 0 ? atomicAdd(&hist[e], 1) : -1;
      if (lane < R) {
        const bool in = (rm >> lane) & 1u;
        rank_slot[(size_t)t * R + lane] = in ? atomicAdd(&hist[E + lane], 1) : -1;
        in_rank[(size_t)t * R + lane] = in ? 1 : 0;
      }
      __syncwarp();
    }
    for (int i = lane; i < cols; i += 32) scratch[(size_t)c * cols + i] = hist[i];
    __syncwarp();
  }
  if (!grid_barrier(bar, gridDim.x)) {
    umdk_set_status(status, UMDK_ERR_TIMEOUT, UMDK_PH_BARRIER, 0, 0);
    return;
  }
  // Phase B: exclusive scan over chunks, one warp per column (32 chunk values per step, warp-level scan).
  for (int col = gwarp; col < cols; col += total_warps) {
    int carry = 0;
    for (int c0 = 0; c0 < num_chunks; c0 += 32) {
      const int c = c0 + lane;
      const int v = c < num_chunks ? scratch[(size_t)c * cols + col] : 0;
      int x = v;
#pragma unroll
      for (int d = 1; d < 32; d <<= 1) {
        const int y = __shfl_up_sync(0xffffffffu, x, d);
        if (lane >= d) x += y;
      }
      if (c < num_chunks) scratch[(size_t)c * cols + col] = x - v + carry;
      carry += __shfl_sync(0xffffffffu, x, 31);
    }
    if (lane == 0) {
      if (col < E) num_per_expert[col] = carry;
      else num_per_rank[col - E] = carry;
    }
  }
  if (!grid_barrier(bar, gridDim.x)) {
    umdk_set_status(status, UMDK_ERR_TIMEOUT, UMDK_PH_BARRIER, 1, 0);
    return;
  }
  // Phase C: add the chunk bases.
  for (int c = gwarp; c < num_chunks; c += total_warps) {
    const int t0 = c * 32;
    const int nt = min(32, T - t0);
    const int* base = scratch + (size_t)c * cols;
    for (int i = lane; i < nt * K; i += 32) {
      long long e = topk_idx[(size_t)t0 * K + i];
      if (e >= 0 && e < E) send_idx[(size_t)t0 * K + i] += base[e];
    }
    for (int i = lane; i < nt * R; i += 32) {
      const int v = rank_slot[(size_t)t0 * R + i];
      if (v >= 0) rank_slot[(size_t)t0 * R + i] = v + base[E + (i % R)];
    }
  }
}

// Layout in ONE CTA with every intermediate in shared memory (per-chunk histograms [chunks][E + R]): used whenever
// they fit, which covers decode batches and prefill batches of a few thousand tokens. Same outputs and the same
// (token-order) positions as ep_layout_kernel, but no global scratch, no grid barriers and no chains of dependent
// global-memory round trips: about 5 us for 128 tokens and 20 us for 4096 instead of 35-90 us.
constexpr int kSmallLayoutWarps = 32;
__global__ void __launch_bounds__(kSmallLayoutWarps * 32)
ep_layout_small_kernel(const int64_t* __restrict__ topk_idx, int T, int K, int E, int R,
                       int* __restrict__ num_per_expert, int* __restrict__ num_per_rank,
                       uint8_t* __restrict__ in_rank, int* __restrict__ send_idx, int* __restrict__ rank_slot) {
  extern __shared__ int sm_small[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int cols = E + R;
  const int E_local = E / R;
  const int num_chunks = (T + 31) / 32;
  int* hist_all = sm_small;                                  // [num_chunks][cols]
  int* stage = sm_small + num_chunks * cols + warp * 32 * K; // per warp: expert ids of the current chunk
  for (int i = threadIdx.x; i < num_chunks * cols; i += blockDim.x) hist_all[i] = 0;
  __syncthreads();
  for (int c = warp; c < num_chunks; c += kSmallLayoutWarps) {
    int* hist = hist_all + c * cols;
    const int t0 = c * 32;
    const int nt = min(32, T - t0);
    for (int i = lane; i < nt * K; i += 32) {
      long long e = topk_idx[(size_t)t0 * K + i];
      stage[i] = (e >= 0 && e < E) ? (int)e : -1;
    }
    __syncwarp();
    for (int i = 0; i < nt; ++i) {
      const int t = t0 + i;
      const int e = lane < K ? stage[i * K + lane] : -1;
      const uint32_t rm = __reduce_or_sync(0xffffffffu, e >= 0 ? (1u << (e / E_local)) : 0u);
      if (lane < K) send_idx[(size_t)t * K + lane] = e >= 0 ? atomicAdd(&hist[e], 1) : -1;   // position in the chunk
      if (lane < R) {
        const bool in = (rm >> lane) & 1u;
        rank_slot[(size_t)t * R + lane] = in ? atomicAdd(&hist[E + lane], 1) : -1;
        in_rank[(size_t)t * R + lane] = in ? 1 : 0;
      }
      __syncwarp();
    }
  }
  __syncthreads();
  // exclusive scan over the chunks, one thread per column
  for (int col = threadIdx.x; col < cols; col += blockDim.x) {
    int run = 0;
    for (int c = 0; c < num_chunks; ++c) {
      const int v = hist_all[c * cols + col];
      hist_all[c * cols + col] = run;
      run += v;
    }
    if (col < E) num_per_expert[col] = run;
    else num_per_rank[col - E] = run;
  }
  __syncthreads();
  // add the chunk bases (each warp revisits the chunks it wrote, so its own global writes are visible to it)
  for (int c = warp; c < num_chunks; c += kSmallLayoutWarps) {
    const int* base = hist_all + c * cols;
    const int t0 = c * 32;
    const int nt = min(32, T - t0);
    for (int i = lane; i < nt * K; i += 32) {
      long long e = topk_idx[(size_t)t0 * K + i];
      if (e >= 0 && e < E) send_idx[(size_t)t0 * K + i] += base[e];
    }
    for (int i = lane; i < nt * R; i += 32) {
      const int v = rank_slot[(size_t)t0 * R + i];
      if (v >= 0) rank_slot[(size_t)t0 * R + i] = v + base[E + (i % R)];
    }
  }
}

// ------------------------------------------------------------------------------------------------------------
// Dispatch
// ------------------------------------------------------------------------------------------------------------
struct DispatchArgs {
  EpGeom g;
  EpNormalOffsets off;
  PeerTable peers;
  long long meet_cycles;       // budget of the wait for the peers' counts (where the ranks meet)
  // inputs on this rank
  const __nv_bfloat16* x;      // [T, H]
  const int64_t* topk_idx;     // [T, K]
  const float* topk_w;         // [T, K] (may be null)
  const int* send_idx;         // [T, K] from layout
  const int* rank_slot;        // [T, R] from layout
  const int* num_per_expert;   // [E]
  const int* num_per_rank;     // [R]
  int T;
  // outputs on this rank
  uint8_t* recv_x;             // [n_cap, row_bytes] expert-major, then source rank
  float* recv_scales;          // [n_cap, nscale]
  int* expand_idx;             // [n_cap, 3] (srcRank, srcToken, k)
  int* recv_count;             // [E_local * R] inclusive prefix, index = le * R + src
  int64_t* recv_per_expert;    // [E_local]
  int* recv_meta;              // [a_cap, 2K+2] per arrival: src, srcToken, rows[K], weight bits[K]
  int* counts_dev;             // [4 + R]: expanded rows N, arrivals A, max tokens from one source, 0, then the
                               // index of the first arrival of every source
  volatile int* counts_host;   // same 4 ints in mapped pinned host memory + [4] = epoch stamp (may be null)
  int n_cap, a_cap;
  // control
  uint32_t* ctrl;              // [0] epoch, [2] recv-done counter, [10] staging gate (tag of the last staged call),
                               // [16 + i] done counter of send pass i
  int* status;
  int phase_mask;              // bit0: notify + send, bit1: receive + expand (both for normal use)
  long long* diag;             // optional [R]: nanoseconds CTA 0 waited for each source rank's data (diagnose mode)
};

__device__ __forceinline__ uint32_t pack_fp8x4(float a, float b, float c, float d) {
  const __nv_fp8x2_storage_t lo = __nv_cvt_float2_to_fp8x2(make_float2(a, b), __NV_SATFINITE, __NV_E4M3);
  const __nv_fp8x2_storage_t hi = __nv_cvt_float2_to_fp8x2(make_float2(c, d), __NV_SATFINITE, __NV_E4M3);
  return (uint32_t)lo | ((uint32_t)hi << 16);
}

__device__ __forceinline__ void bf16x8_to_float(const int4& v, float* f) {
  const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 t = __bfloat1622float2(p[i]);
    f[2 * i] = t.x;
    f[2 * i + 1] = t.y;
  }
}

// Barrier over the warps of one role (named barrier `id`, `nthreads` a multiple of 32).
__device__ __forceinline__ void role_sync(int id, int nthreads) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(nthreads) : "memory");
}

// One warp quantises token t (bf16 -> fp8 e4m3, fp32 scale per 1x128 block) and writes the row to up to two places.
__device__ __forceinline__ void quant_row_to(const int4* xrow, int H, int lane, uint8_t* px0, float* ps0, uint8_t* px1,
                                             float* ps1, uint8_t* px2 = nullptr, float* ps2 = nullptr) {
  const int nblk = H / 128;
  // each lane: 16 elements per step; 8 lanes share one 1x128 block; two groups of four blocks per iteration with all
  // four 16-byte loads of a lane issued first
  for (int b0 = 0; b0 < nblk; b0 += 8) {
    int4 raw[2][2];
    bool active[2];
#pragma unroll
    for (int u = 0; u < 2; ++u) {
      const int blk = b0 + 4 * u + (lane >> 3);
      active[u] = blk < nblk;
      if (active[u]) {
        raw[u][0] = __ldg(xrow + blk * 16 + (lane & 7) * 2);
        raw[u][1] = __ldg(xrow + blk * 16 + (lane & 7) * 2 + 1);
      } else {
        raw[u][0] = raw[u][1] = make_int4(0, 0, 0, 0);
      }
    }
#pragma unroll
    for (int u = 0; u < 2; ++u) {
      const int blk = b0 + 4 * u + (lane >> 3);
      float f[16];
      bf16x8_to_float(raw[u][0], f);
      bf16x8_to_float(raw[u][1], f + 8);
      float amax = 0.f;
#pragma unroll
      for (int i = 0; i < 16; ++i) amax = fmaxf(amax, fabsf(f[i]));
      amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
      amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
      amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 4));
      amax = fmaxf(amax, 1e-4f);
      const float scale = amax * (1.f / 448.f);
      const float inv = 448.f / amax;
      int4 q;
      q.x = pack_fp8x4(f[0] * inv, f[1] * inv, f[2] * inv, f[3] * inv);
      q.y = pack_fp8x4(f[4] * inv, f[5] * inv, f[6] * inv, f[7] * inv);
      q.z = pack_fp8x4(f[8] * inv, f[9] * inv, f[10] * inv, f[11] * inv);
      q.w = pack_fp8x4(f[12] * inv, f[13] * inv, f[14] * inv, f[15] * inv);
      if (active[u]) {
        const int o = blk * 128 + (lane & 7) * 16;
        if (px0) st_na_v4(px0 + o, q);
        if (px1) st_na_v4(px1 + o, q);
        if (px2) st_na_v4(px2 + o, q);
        if ((lane & 7) == 0) {
          if (ps0) ps0[blk] = scale;
          if (ps1) ps1[blk] = scale;
          if (ps2) ps2[blk] = scale;
        }
      }
    }
  }
}

// One warp copies `bytes` (a multiple of 16) with eight 16-byte loads per lane in flight before the first store.
template <bool kFromThisKernel>
__device__ __forceinline__ void warp_copy_row(uint8_t* dst, const uint8_t* src, int bytes, int lane) {
  const int nvec = bytes / 16;
  const int4* s = reinterpret_cast<const int4*>(src);
  int4* d = reinterpret_cast<int4*>(dst);
  for (int v0 = 0; v0 < nvec; v0 += 8 * 32) {
    int4 x[8];
#pragma unroll
    for (int u = 0; u < 8; ++u) {
      const int v = v0 + u * 32 + lane;
      if (v < nvec) x[u] = kFromThisKernel ? __ldcg(s + v) : __ldg(s + v);
    }
#pragma unroll
    for (int u = 0; u < 8; ++u) {
      const int v = v0 + u * 32 + lane;
      if (v < nvec) st_na_v4(d + v, x[u]);
    }
  }
}

// Dispatch = two roles that run side by side in every CTA (phase_mask 3: warps [0, 8) send, warps [8, 16) receive)
// or one at a time with all warps (phase_mask 1 or 2, which is how several ranks are emulated on one GPU).
//
// Sender. Pass 0 quantises every token once into a local staging area (and into this rank's own arrival slots for
// the tokens that stay here). Then one pass per peer, destination (rank + i) % R in pass i: the rows that go there
// are copied from the staging area into the peer's arrival slots, and the peer's data flag is raised as soon as the
// pass is complete on all CTAs. Every rank walks the ring in the same direction, so at any moment the ranks write to
// different destinations - a rotating permutation that keeps each inbound link busy with one writer - and a receiver
// gets its sources one after the other, in the order (rank, rank - 1, rank - 2, ...), which is the order in which
// its receiving warps expand them.
__global__ void __launch_bounds__(kEpThreads, 1) ep_dispatch_kernel(const DispatchArgs a) {
  const EpGeom& g = a.g;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  __shared__ uint32_t s_epoch;
  __shared__ int s_cnt[1024 + 64];   // counts [le][src] -> exclusive offsets; tail: per-source arrivals
  __shared__ int s_ok_send, s_ok_recv;
  __shared__ int s_row[kEpWarps][kMaxTopk];    // per-warp staging: expanded rows of the current arrival
  if (threadIdx.x == 0) {
    s_epoch = a.ctrl[0];
    s_ok_send = 1;
    s_ok_recv = 1;
  }
  __syncthreads();
  const uint32_t epoch = s_epoch;
  const int h = epoch & 1;
  const uint64_t tag = (uint64_t)epoch + 1;
  const int nw = ep_notify_words(g.E_local);
  const bool both = (a.phase_mask & 3) == 3;
  // Half of the warps send, half expand. Measured on 8 GPUs: 343 us; with 6 of 16 warps sending 353 us; with 4 of 16
  // (before the signalling warp existed) 414 us against 396 us.
  const int n_send_warps = both ? kEpWarps / 2 : kEpWarps;
  const bool is_sender = (a.phase_mask & 1) && (!both || warp < n_send_warps);
  const bool is_receiver = (a.phase_mask & 2) && (!both || warp >= n_send_warps);
  uint8_t* self = a.peers.base[g.rank];

  if (a.phase_mask & 1) {
    // Pass 0 (quantise everything once, keep what stays here) is done by ALL warps: nothing has arrived yet that the
    // receiving warps could work on. From pass 1 on only the sending warps continue.
    const int sw = warp;                       // sender warps are always the first ones
    const bool stage = g.quant && g.R > 2;    // two ranks: pass 0 reaches both destinations, nothing is read back
    uint8_t* stage_x = self + a.off.stage_x;
    float* stage_s = reinterpret_cast<float*>(self + a.off.stage_scale);
    // ---- notify: CTA 0, one warp per destination rank (looping) ----
    if (blockIdx.x == 0) {
      for (int d = sw; d < g.R; d += kEpWarps) {
        int* dst = reinterpret_cast<int*>(a.peers.base[d] + a.off.notify[h]) + (size_t)g.rank * nw;
        for (int i = lane; i < g.E_local; i += 32) dst[i] = a.num_per_expert[d * g.E_local + i];
        if (lane == 0) dst[g.E_local] = a.num_per_rank[d];
        __threadfence_system();
        __syncwarp();
        if (lane == 0) {
          st_release_sys(reinterpret_cast<uint64_t*>(a.peers.base[d] + a.off.notify_flag[h]) + g.rank, tag);
        }
      }
    }
    // With staging, pass 0 also serves the right-hand neighbour (the quantised row is in registers anyway), so the
    // first remote pass costs no extra read of the staging area and no extra end-of-pass round.
    const bool merged = g.quant && g.R > 1;
    const int d_next = (g.rank + 1) % g.R;
    for (int pass = 0; pass < g.R; ++pass) {
      if (pass > 0 && !is_sender) break;
      if (pass == 1 && merged) continue;
      const int nsw = pass == 0 ? kEpWarps : n_send_warps;   // warps working on this pass
      const int nthr = nsw * 32;
      const int bar_id = pass == 0 ? 3 : 1;
      const int d = (g.rank + pass) % g.R;
      uint8_t* peer = a.peers.base[d];
      // From pass 1 on the last sending warp copies nothing: it only publishes the end of each pass (a system-scope
      // fence that waits for the remote stores, a counter, the flag), so that the copying warps never sit behind
      // that fence and go straight on to the next destination.
      const bool have_signaller = pass > 0 && nsw >= 2;
      const bool signaller = have_signaller && sw == nsw - 1;
      const int ncopy = have_signaller ? nsw - 1 : nsw;
      for (int t = blockIdx.x * ncopy + sw; t < a.T && !signaller; t += gridDim.x * ncopy) {
        const int slot = a.rank_slot[(size_t)t * g.R + d];
        if (slot >= g.cap) {
          if (lane == 0) umdk_set_status(a.status, UMDK_ERR_OVERFLOW, UMDK_PH_DISPATCH_DATA, d, slot);
        }
        const bool goes = slot >= 0 && slot < g.cap;
        const int slot_next = (pass == 0 && merged) ? a.rank_slot[(size_t)t * g.R + d_next] : -1;
        if (!goes && !(pass == 0 && (stage || slot_next >= 0))) continue;
        const size_t rec = (size_t)g.rank * g.cap + (goes ? slot : 0);
        // metadata: lanes 0..K-1 hold (local expert << 16 | bucket position) or -1, then the weights, then the token
        auto put_meta = [&](int dd, size_t rr) {
          int* meta = reinterpret_cast<int*>(a.peers.base[dd] + a.off.arr_meta[h]) + rr * g.meta_words;
          if (lane < g.K) {
            const long long ee = a.topk_idx[(size_t)t * g.K + lane];
            const int e = (ee >= 0 && ee < g.E) ? (int)ee : -1;
            const bool mine = e >= 0 && (e / g.E_local) == dd;
            meta[lane] = mine ? (((e % g.E_local) << 16) | (a.send_idx[(size_t)t * g.K + lane] & 0xffff)) : -1;
            meta[g.K + lane] = __float_as_int(a.topk_w ? a.topk_w[(size_t)t * g.K + lane] : 1.f);
          }
          if (lane == 0) meta[2 * g.K] = t;
        };
        if (goes) put_meta(d, rec);
        uint8_t* px2 = nullptr;
        float* ps2 = nullptr;
        if (pass == 0 && merged) {
          const int slot1 = slot_next;
          if (slot1 >= g.cap) {
            if (lane == 0) umdk_set_status(a.status, UMDK_ERR_OVERFLOW, UMDK_PH_DISPATCH_DATA, d_next, slot1);
          } else if (slot1 >= 0) {
            const size_t rec1 = (size_t)g.rank * g.cap + slot1;
            put_meta(d_next, rec1);
            px2 = a.peers.base[d_next] + a.off.arr_x[h] + rec1 * g.row_bytes;
            ps2 = reinterpret_cast<float*>(a.peers.base[d_next] + a.off.arr_scale[h]) + rec1 * g.nscale;
          }
        }
        uint8_t* px = goes ? peer + a.off.arr_x[h] + rec * g.row_bytes : nullptr;
        float* ps = goes ? reinterpret_cast<float*>(peer + a.off.arr_scale[h]) + rec * g.nscale : nullptr;
        if (!g.quant) {
          warp_copy_row<false>(px, reinterpret_cast<const uint8_t*>(a.x + (size_t)t * g.H), g.row_bytes, lane);
        } else if (pass == 0) {
          quant_row_to(reinterpret_cast<const int4*>(a.x + (size_t)t * g.H), g.H, lane,
                       stage ? stage_x + (size_t)t * g.H : nullptr, stage ? stage_s + (size_t)t * g.nscale : nullptr,
                       px, ps, px2, ps2);
        } else {
          warp_copy_row<true>(px, stage_x + (size_t)t * g.H, g.row_bytes, lane);
          for (int v = lane; v < g.nscale; v += 32) ps[v] = __ldcg(stage_s + (size_t)t * g.nscale + v);
        }
      }
      // ---- end of the pass: the last CTA to finish it raises this rank's data flag on the destination ----
      role_sync(bar_id, nthr);
      if (have_signaller ? (signaller && lane == 0) : threadIdx.x == 0) {
        __threadfence_system();
        const uint32_t old = atomicAdd(&a.ctrl[16 + pass], 1u);
        if (old == gridDim.x - 1) {
          a.ctrl[16 + pass] = 0;
          __threadfence_system();
          st_release_sys(reinterpret_cast<uint64_t*>(peer + a.off.data_flag[h]) + g.rank, tag);
          if (pass == 0 && merged && d_next != g.rank) {
            st_release_sys(reinterpret_cast<uint64_t*>(a.peers.base[d_next] + a.off.data_flag[h]) + g.rank, tag);
          }
          if (pass == 0 && stage) {   // staging area complete: open the gate for this call
            __threadfence();
            atomicExch(&a.ctrl[10], epoch + 1);
          }
        }
        if (pass == 0 && stage) {
          // the later passes read rows that other CTAs quantised: wait until all of them are through pass 0
          const uint32_t want = epoch + 1;   // the gate holds the tag of the last call whose staging is complete
          const long long t0 = clock64();
          while ((int32_t)(ld_acquire_gpu(&a.ctrl[10]) - want) < 0) {
            if (clock64() - t0 > kSpinLimitCycles) {
              umdk_set_status(a.status, UMDK_ERR_TIMEOUT, UMDK_PH_BARRIER, blockIdx.x, (int)epoch);
              s_ok_send = 0;
              break;
            }
            __nanosleep(20);
          }
        }
      }
      if (pass == 0 && stage) {
        role_sync(bar_id, nthr);
        if (!s_ok_send) break;
      }
    }
  }

  if (!is_receiver) return;
  const int rw = both ? warp - n_send_warps : warp;   // index among the receiving warps
  const int n_recv_warps = both ? kEpWarps - n_send_warps : kEpWarps;
  const int rthr = n_recv_warps * 32;
  const int rtid = threadIdx.x - (both ? n_send_warps * 32 : 0);

  // ---- receive: wait for every source's counts, build offsets ----
  if (rtid < g.R) {
    const uint64_t* f = reinterpret_cast<const uint64_t*>(self + a.off.notify_flag[h]) + rtid;
    if (!wait_flag_ge_sys(f, tag, a.meet_cycles)) {
      umdk_set_status(a.status, UMDK_ERR_TIMEOUT, UMDK_PH_DISPATCH_COUNT, rtid, (int)epoch);
      s_ok_recv = 0;
    }
  }
  role_sync(2, rthr);
  if (!s_ok_recv) return;
  const int* notify = reinterpret_cast<const int*>(self + a.off.notify[h]);
  const int nle = g.E_local * g.R;
  int* s_arr = s_cnt + 1024;  // [R] arrivals per source, then [R] exclusive arrival base
  for (int i = rtid; i < nle; i += rthr) {
    const int le = i / g.R, src = i % g.R;
    s_cnt[i] = notify[(size_t)src * nw + le];
  }
  if (rtid < g.R) s_arr[rtid] = notify[(size_t)rtid * nw + g.E_local];
  role_sync(2, rthr);
  if (rtid == 0) {
    int run = 0, amax_src = 0, abase = 0;
    for (int i = 0; i < nle; ++i) {
      const int c = s_cnt[i];
      s_cnt[i] = run;  // exclusive offset of (le, src)
      run += c;
      if (blockIdx.x == 0) {
        a.recv_count[i] = run;  // inclusive prefix, as the reference returns it
        if ((i % g.R) == g.R - 1) {
          const int le = i / g.R;
          a.recv_per_expert[le] = (int64_t)(run - s_cnt[le * g.R]);
        }
      }
    }
    for (int r = 0; r < g.R; ++r) {
      const int c = s_arr[r];
      amax_src = max(amax_src, c);
      s_arr[g.R + r] = abase;
      abase += c;
    }
    s_cnt[1023] = run;
    if (blockIdx.x == 0) {
      a.counts_dev[0] = run;
      a.counts_dev[1] = abase;
      a.counts_dev[2] = amax_src;
      for (int r = 0; r < g.R; ++r) a.counts_dev[4 + r] = s_arr[g.R + r];  // first arrival of each source
      if (a.counts_host) {
        a.counts_host[0] = run;
        a.counts_host[1] = abase;
        a.counts_host[2] = amax_src;
        __threadfence_system();
        a.counts_host[4] = (int)tag;
      }
      if (run > a.n_cap || abase > a.a_cap) umdk_set_status(a.status, UMDK_ERR_OVERFLOW, UMDK_PH_DISPATCH_COUNT, run, abase);
    }
  }
  role_sync(2, rthr);

  // ---- expand: arrivals -> expert-major rows, sources in the order in which their passes reach this rank ----
  const int mw2 = 2 * g.K + 2;
  for (int i = 0; i < g.R; ++i) {
    const int src = (g.rank - i + g.R) % g.R;  // own tokens first (they are already here)
    if (rtid == 0) {
      const uint64_t* f = reinterpret_cast<const uint64_t*>(self + a.off.data_flag[h]) + src;
      const long long t0 = a.diag ? (long long)globaltimer_ns() : 0;
      if (!wait_flag_ge_sys(f, tag)) {
        umdk_set_status(a.status, UMDK_ERR_TIMEOUT, UMDK_PH_DISPATCH_DATA, src, (int)epoch);
        s_ok_recv = 0;
      }
      if (a.diag && blockIdx.x == 0) a.diag[src] = (long long)globaltimer_ns() - t0;
    }
    role_sync(2, rthr);
    if (!s_ok_recv) return;
    const int n_from = min(s_arr[src], g.cap);
    const int abase = s_arr[g.R + src];
    for (int p = blockIdx.x * n_recv_warps + rw; p < n_from; p += gridDim.x * n_recv_warps) {
      const size_t rec = (size_t)src * g.cap + p;
      const int* meta = reinterpret_cast<const int*>(self + a.off.arr_meta[h]) + rec * g.meta_words;
      int code = -1, wbits = 0;
      if (lane < g.K) {
        code = meta[lane];
        wbits = meta[g.K + lane];
      }
      const int src_tok = meta[2 * g.K];
      int row = -1;
      if (code >= 0) {
        const int le = code >> 16, pos = code & 0xffff;
        row = s_cnt[le * g.R + src] + pos;
        if (row >= a.n_cap) {
          umdk_set_status(a.status, UMDK_ERR_OVERFLOW, UMDK_PH_DISPATCH_DATA, src, row);
          row = -1;
        }
      }
      if (abase + p < a.a_cap) {
        int* rm = a.recv_meta + (size_t)(abase + p) * mw2;
        if (lane == 0) {
          rm[0] = src;
          rm[1] = src_tok;
        }
        if (lane < g.K) {
          rm[2 + lane] = row;
          rm[2 + g.K + lane] = wbits;
        }
      }
      if (row >= 0) {
        a.expand_idx[(size_t)row * 3 + 0] = src;
        a.expand_idx[(size_t)row * 3 + 1] = src_tok;
        a.expand_idx[(size_t)row * 3 + 2] = lane;
      }
      const uint32_t kmask = __ballot_sync(0xffffffffu, row >= 0);
      __syncwarp();
      if (lane < g.K) s_row[warp][lane] = row;
      __syncwarp();
      const int4* px = reinterpret_cast<const int4*>(self + a.off.arr_x[h] + rec * g.row_bytes);
      const int nvec = g.row_bytes / 16;
      // eight 512-byte loads per warp in flight before the first store
      for (int v0 = lane; v0 < nvec; v0 += 256) {
        int4 val[8];
#pragma unroll
        for (int u = 0; u < 8; ++u) {
          if (v0 + 32 * u < nvec) val[u] = px[v0 + 32 * u];
        }
        for (uint32_t m = kmask; m; m &= m - 1) {
          int4* drow = reinterpret_cast<int4*>(a.recv_x + (size_t)s_row[warp][__ffs(m) - 1] * g.row_bytes);
#pragma unroll
          for (int u = 0; u < 8; ++u) {
            if (v0 + 32 * u < nvec) drow[v0 + 32 * u] = val[u];
          }
        }
      }
      if (g.quant) {
        const float* ps = reinterpret_cast<const float*>(self + a.off.arr_scale[h]) + rec * g.nscale;
        for (int v = lane; v < g.nscale; v += 32) {
          const float val = ps[v];
          for (uint32_t m = kmask; m; m &= m - 1) {
            const int r2 = s_row[warp][__ffs(m) - 1];
            a.recv_scales[(size_t)r2 * g.nscale + v] = val;
          }
        }
      }
    }
  }
  // ---- epoch advance by the last CTA ----
  role_sync(2, rthr);
  if (rtid == 0) {
    __threadfence_system();
    const uint32_t old = atomicAdd(&a.ctrl[2], 1u);
    if (old == gridDim.x - 1) {
      a.ctrl[2] = 0;
      a.ctrl[0] = epoch + 1;
    }
  }
}

// ------------------------------------------------------------------------------------------------------------
// Combine
// ------------------------------------------------------------------------------------------------------------
struct CombineArgs {
  EpGeom g;
  EpNormalOffsets off;
  PeerTable peers;
  const __nv_bfloat16* y;     // [N, H] expert outputs in the dispatch row order
  // mode 0 (per-rank pre-reduction): arrival metadata from dispatch
  const int* recv_meta;       // [A, 2K+2]
  const int* counts_dev;      // [0] = N, [1] = A, [4 + r] = index of the first arrival from source r
  // mode 1 (row per (token,k), reference contract): (srcRank, srcToken, k) per row
  const int* src_idx;         // [N, 3]
  int n_rows;                 // mode 1: number of rows; mode 0: ignored
  // owner side
  const uint8_t* in_rank;     // [T, R] (mode 0)
  const int64_t* topk_idx;    // [T, K] (mode 1)
  const float* topk_w;        // [T, K] (mode 1)
  __nv_bfloat16* out;         // [T, H]
  int T;
  int mode;
  int apply_weights;          // mode 0: multiply rows by the weights shipped at dispatch time
  uint32_t* ctrl;             // [3] epoch, [4] send-done, [5] recv-done
  int* status;
  int phase_mask;
  long long* diag;            // optional [R]: nanoseconds CTA 0 waited for each source rank's rows
};

__global__ void __launch_bounds__(kEpThreads, 1) ep_combine_kernel(const CombineArgs a) {
  const EpGeom& g = a.g;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  __shared__ uint32_t s_epoch;
  __shared__ int s_ok;
  __shared__ int s_row[kEpWarps][kMaxRanks];
  __shared__ float s_coef[kEpWarps][kMaxRanks];
  if (threadIdx.x == 0) {
    s_epoch = a.ctrl[3];
    s_ok = 1;
  }
  __syncthreads();
  const uint32_t epoch = s_epoch;
  const int h = epoch & 1;
  const uint64_t tag = (uint64_t)epoch + 1;
  const int nvec = g.H / 8;
  const int mw2 = 2 * g.K + 2;

  if (a.phase_mask & 1) {
    const int items = a.mode == 0 ? a.counts_dev[1] : a.n_rows;
    // Arrivals are stored source by source. Every rank starts with the arrivals of its right-hand neighbour and goes
    // round from there, so that at any moment the ranks send to different destinations (a rotating permutation)
    // instead of all to the same one, whose inbound link would then be the bottleneck of the whole box.
    const int start = (a.mode == 0 && g.R > 1) ? min(max(a.counts_dev[4 + (g.rank + 1) % g.R], 0), items) : 0;
    for (int it0 = blockIdx.x * kEpWarps + warp; it0 < items; it0 += gridDim.x * kEpWarps) {
      const int it = it0 + start < items ? it0 + start : it0 + start - items;
      int dst_rank, dst_tok, slot_j;
      int row = -1;
      float w = 1.f;
      if (a.mode == 0) {
        const int* rm = a.recv_meta + (size_t)it * mw2;
        dst_rank = rm[0];
        dst_tok = rm[1];
        slot_j = g.rank;
        if (lane < g.K) {
          row = rm[2 + lane];
          if (a.apply_weights) w = __int_as_float(rm[2 + g.K + lane]);
        }
      } else {
        dst_rank = a.src_idx[(size_t)it * 3 + 0];
        dst_tok = a.src_idx[(size_t)it * 3 + 1];
        slot_j = a.src_idx[(size_t)it * 3 + 2];
        if (lane == 0) row = it;
      }
      if (dst_rank < 0 || dst_rank >= g.R || dst_tok < 0 || dst_tok >= g.cap || slot_j < 0 || slot_j >= g.J) {
        umdk_set_status(a.status, UMDK_ERR_OVERFLOW, UMDK_PH_COMBINE_DATA, dst_rank, dst_tok);
        continue;
      }
      // compact the valid rows so that the loads below can be issued as fixed-size batches (all in flight at once)
      const uint32_t kmask = __ballot_sync(0xffffffffu, row >= 0);
      const int n = __popc(kmask);
      __syncwarp();
      if (row >= 0) {
        const int pos = __popc(kmask & ((1u << lane) - 1u));
        s_row[warp][pos] = row;
        s_coef[warp][pos] = w;
      }
      __syncwarp();
      int4* dst = reinterpret_cast<int4*>(a.peers.base[dst_rank] + a.off.comb_buf[h] +
                                          ((size_t)dst_tok * g.J + slot_j) * g.H * 2);
      // four 512-byte chunks of the row per step and two source rows per batch: eight 16-byte loads per lane are in
      // flight before the first one is consumed (an arrival has 1.5 rows on average, so the parallelism has to come
      // from the chunks)
      for (int v0 = 0; v0 < nvec; v0 += 4 * 32) {
        float acc[4][8];
#pragma unroll
        for (int c = 0; c < 4; ++c)
#pragma unroll
          for (int i = 0; i < 8; ++i) acc[c][i] = 0.f;
        for (int base = 0; base < n; base += 2) {
          int4 vals[2][4];
#pragma unroll
          for (int u = 0; u < 2; ++u) {
            if (base + u < n) {
              const int4* rowp = reinterpret_cast<const int4*>(a.y + (size_t)s_row[warp][base + u] * g.H);
#pragma unroll
              for (int c = 0; c < 4; ++c) {
                const int v = v0 + c * 32 + lane;
                if (v < nvec) vals[u][c] = __ldg(rowp + v);
              }
            }
          }
#pragma unroll
          for (int u = 0; u < 2; ++u) {
            if (base + u < n) {
              const float w2 = s_coef[warp][base + u];
#pragma unroll
              for (int c = 0; c < 4; ++c) {
                if (v0 + c * 32 + lane < nvec) {
                  float f[8];
                  bf16x8_to_float(vals[u][c], f);
#pragma unroll
                  for (int i = 0; i < 8; ++i) acc[c][i] = fmaf(w2, f[i], acc[c][i]);
                }
              }
            }
          }
        }
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          const int v = v0 + c * 32 + lane;
          if (v < nvec) {
            int4 o;
            __nv_bfloat162* po = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
            for (int i = 0; i < 4; ++i) po[i] = __floats2bfloat162_rn(acc[c][2 * i], acc[c][2 * i + 1]);
            st_na_v4(dst + v, o);
          }
        }
      }
    }
    if (cta_done_is_last(&a.ctrl[4], gridDim.x)) {
      if (threadIdx.x < g.R) {
        st_release_sys(reinterpret_cast<uint64_t*>(a.peers.base[threadIdx.x] + a.off.comb_flag[h]) + g.rank, tag);
      }
    }
  }
  if (!(a.phase_mask & 2)) return;

  uint8_t* self = a.peers.base[g.rank];
  if (threadIdx.x < g.R) {
    const uint64_t* f = reinterpret_cast<const uint64_t*>(self + a.off.comb_flag[h]) + threadIdx.x;
    const long long t0 = a.diag ? (long long)globaltimer_ns() : 0;
    if (!wait_flag_ge_sys(f, tag)) {
      umdk_set_status(a.status, UMDK_ERR_TIMEOUT, UMDK_PH_COMBINE_DATA, threadIdx.x, (int)epoch);
      s_ok = 0;
    }
    if (a.diag && blockIdx.x == 0) a.diag[threadIdx.x] = (long long)globaltimer_ns() - t0;
  }
  __syncthreads();
  if (!s_ok) return;
  const int J = a.mode == 0 ? g.R : g.K;
  for (int t = blockIdx.x * kEpWarps + warp; t < a.T; t += gridDim.x * kEpWarps) {
    float coef = 0.f;
    if (lane < J) {
      if (a.mode == 0) coef = a.in_rank[(size_t)t * g.R + lane] ? 1.f : 0.f;
      else coef = a.topk_idx[(size_t)t * g.K + lane] >= 0 ? a.topk_w[(size_t)t * g.K + lane] : 0.f;
    }
    const bool used = lane < J && (a.mode == 0 ? coef != 0.f : a.topk_idx[(size_t)t * g.K + lane] >= 0);
    const uint32_t jmask = __ballot_sync(0xffffffffu, used);
    const int n = __popc(jmask);
    __syncwarp();
    if (used) {
      const int pos = __popc(jmask & ((1u << lane) - 1u));
      s_row[warp][pos] = lane;
      s_coef[warp][pos] = coef;
    }
    __syncwarp();
    const int4* src = reinterpret_cast<const int4*>(self + a.off.comb_buf[h] + (size_t)t * g.J * g.H * 2);
    for (int v0 = 0; v0 < nvec; v0 += 2 * 32) {
      float acc[2][8];
#pragma unroll
      for (int c = 0; c < 2; ++c)
#pragma unroll
        for (int i = 0; i < 8; ++i) acc[c][i] = 0.f;
      for (int base = 0; base < n; base += 4) {
        int4 vals[4][2];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          if (base + u < n) {
            const int4* rowp = src + (size_t)s_row[warp][base + u] * nvec;
#pragma unroll
            for (int c = 0; c < 2; ++c) {
              const int v = v0 + c * 32 + lane;
              if (v < nvec) vals[u][c] = rowp[v];
            }
          }
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          if (base + u < n) {
            const float cf = s_coef[warp][base + u];
#pragma unroll
            for (int c = 0; c < 2; ++c) {
              if (v0 + c * 32 + lane < nvec) {
                float f[8];
                bf16x8_to_float(vals[u][c], f);
#pragma unroll
                for (int i = 0; i < 8; ++i) acc[c][i] = fmaf(cf, f[i], acc[c][i]);
              }
            }
          }
        }
      }
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        const int v = v0 + c * 32 + lane;
        if (v < nvec) {
          int4 o;
          __nv_bfloat162* po = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
          for (int i = 0; i < 4; ++i) po[i] = __floats2bfloat162_rn(acc[c][2 * i], acc[c][2 * i + 1]);
          reinterpret_cast<int4*>(a.out + (size_t)t * g.H)[v] = o;
        }
      }
    }
  }
  if (cta_done_is_last(&a.ctrl[5], gridDim.x)) {
    if (threadIdx.x == 0) a.ctrl[3] = epoch + 1;
  }
}

}  // namespace
}  // namespace umdk

using namespace umdk;

static int fill_geom(EpGeom* g, int R, int rank, int E, int K, int H, int cap, int quant) {
  if (R < 1 || R > kMaxRanks || rank < 0 || rank >= R || E < R || (E % R) || K < 1 || K > kMaxTopk || H < 128 ||
      (H % 128) || cap < 1 || cap > 65535 || (E / R) * R > 1024 - 1)
    return -UMDK_ERR_BAD_ARG;
  g->R = R;
  g->rank = rank;
  g->E = E;
  g->E_local = E / R;
  g->K = K;
  g->H = H;
  g->cap = cap;
  g->quant = quant;
  g->row_bytes = quant ? H : 2 * H;
  g->nscale = quant ? H / 128 : 0;
  g->meta_words = ep_meta_words(K);
  g->J = R > K ? R : K;
  return 0;
}

// Bytes of symmetric heap each rank needs for normal-mode dispatch + combine with this geometry.
// Heap layout is sized for the larger payload format (bf16 rows, plus room for scales) so that quantised and
// unquantised calls share one heap.
static EpGeom layout_geom(EpGeom g) {
  g.quant = 0;
  g.row_bytes = 2 * g.H;
  g.nscale = g.H / 128;
  return g;
}

UMDK_API long long umdk_ep_normal_heap_bytes(int R, int E, int K, int H, int cap) {
  EpGeom g;
  if (fill_geom(&g, R, 0, E, K, H, cap, 0)) return -1;
  return (long long)ep_normal_offsets(layout_geom(g)).total;
}

// scratch: int32[(ceil(T/32)) * (E + R)]; bar: uint32[2], reset on the caller's stream at the start of every call
// that uses it (an earlier call cut short by a barrier time-out may have left a partial arrival count).
UMDK_API int umdk_ep_layout(const int64_t* topk_idx, int T, int K, int E, int R, int* num_per_expert,
                            int* num_per_rank, uint8_t* in_rank, int* send_idx, int* rank_slot, int* scratch,
                            uint32_t* bar, int* status, void* stream) {
  if (T < 0 || K < 1 || K > kMaxTopk || R < 1 || R > kMaxRanks || E < R || (E % R)) return -UMDK_ERR_BAD_ARG;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (T == 0) {
    UMDK_CUDA_CHECK(cudaMemsetAsync(num_per_expert, 0, sizeof(int) * E, s));
    UMDK_CUDA_CHECK(cudaMemsetAsync(num_per_rank, 0, sizeof(int) * R, s));
    return 0;
  }
  const int chunks = (T + 31) / 32;
  {
    // decode-sized inputs: one CTA with everything in shared memory (no grid barriers, no scratch); measured at
    // 4096 tokens the single CTA takes 96 us against 35-48 us for the multi-CTA kernel, so it is kept to small inputs
    const size_t small_smem = sizeof(int) * ((size_t)chunks * (E + R) + (size_t)kSmallLayoutWarps * 32 * K);
    if (T <= 1024 && small_smem <= 200 * 1024) {
      if (small_smem > 48 * 1024) {
        UMDK_CUDA_CHECK(cudaFuncSetAttribute(ep_layout_small_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             (int)small_smem));
      }
      ep_layout_small_kernel<<<1, kSmallLayoutWarps * 32, small_smem, s>>>(topk_idx, T, K, E, R, num_per_expert,
                                                                           num_per_rank, in_rank, send_idx, rank_slot);
      UMDK_CUDA_CHECK(cudaGetLastError());
      return 0;
    }
  }
  int grid = (chunks + kLayoutWarps - 1) / kLayoutWarps;
  if (grid > sm_count()) grid = sm_count();
  const size_t smem = sizeof(int) * (size_t)kLayoutWarps * ((E + R) + 32 * kMaxTopk);
  if (smem > 48 * 1024) {
    UMDK_CUDA_CHECK(cudaFuncSetAttribute(ep_layout_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  }
  UMDK_CUDA_CHECK(cudaMemsetAsync(bar, 0, 2 * sizeof(uint32_t), s));
  ep_layout_kernel<<<grid, kLayoutWarps * 32, smem, s>>>(topk_idx, T, K, E, R, num_per_expert, num_per_rank, in_rank,
                                                         send_idx, rank_slot, scratch, bar, status);
  UMDK_CUDA_CHECK(cudaGetLastError());
  return 0;
}

struct UmdkEpDispatchParams {
  int R, rank, E, K, H, cap, quant, T;
  int n_cap, a_cap, num_ctas, phase_mask;
  void* peers[kMaxRanks];
  const void* x;
  const int64_t* topk_idx;
  const float* topk_w;
  const int* send_idx;
  const int* rank_slot;
  const int* num_per_expert;
  const int* num_per_rank;
  void* recv_x;
  float* recv_scales;
  int* expand_idx;
  int* recv_count;
  int64_t* recv_per_expert;
  int* recv_meta;
  int* counts_dev;
  int* counts_host;
  uint32_t* ctrl;
  int* status;
  long long* diag;   // optional [R] per-source wait times in ns (diagnose mode), else null
};

UMDK_API int umdk_ep_dispatch(const UmdkEpDispatchParams* p, void* stream) {
  DispatchArgs a;
  a.meet_cycles = umdk_rendezvous_cycles();
  if (int rc = fill_geom(&a.g, p->R, p->rank, p->E, p->K, p->H, p->cap, p->quant)) return rc;
  if (p->T > p->cap) return -UMDK_ERR_BAD_ARG;
  a.off = ep_normal_offsets(layout_geom(a.g));
  for (int i = 0; i < p->R; ++i) a.peers.base[i] = static_cast<uint8_t*>(p->peers[i]);
  a.x = static_cast<const __nv_bfloat16*>(p->x);
  a.topk_idx = p->topk_idx;
  a.topk_w = p->topk_w;
  a.send_idx = p->send_idx;
  a.rank_slot = p->rank_slot;
  a.num_per_expert = p->num_per_expert;
  a.num_per_rank = p->num_per_rank;
  a.T = p->T;
  a.recv_x = static_cast<uint8_t*>(p->recv_x);
  a.recv_scales = p->recv_scales;
  a.expand_idx = p->expand_idx;
  a.recv_count = p->recv_count;
  a.recv_per_expert = p->recv_per_expert;
  a.recv_meta = p->recv_meta;
  a.counts_dev = p->counts_dev;
  a.counts_host = p->counts_host;
  a.n_cap = p->n_cap;
  a.a_cap = p->a_cap;
  a.ctrl = p->ctrl;
  a.status = p->status;
  a.diag = p->diag;
  a.phase_mask = p->phase_mask ? p->phase_mask : 3;
  int grid = p->num_ctas > 0 ? p->num_ctas : sm_count();
  if (grid > sm_count()) grid = sm_count();  // CTAs wait on peers: the whole grid must be resident
  ep_dispatch_kernel<<<grid, kEpThreads, 0, static_cast<cudaStream_t>(stream)>>>(a);
  UMDK_CUDA_CHECK(cudaGetLastError());
  return 0;
}

struct UmdkEpCombineParams {
  int R, rank, E, K, H, cap, T;
  int mode, apply_weights, n_rows, num_ctas, phase_mask;
  void* peers[kMaxRanks];
  const void* y;
  const int* recv_meta;
  const int* counts_dev;
  const int* src_idx;
  const uint8_t* in_rank;
  const int64_t* topk_idx;
  const float* topk_w;
  void* out;
  uint32_t* ctrl;
  int* status;
  long long* diag;   // optional [R] per-source wait times in ns (diagnose mode), else null
};

UMDK_API int umdk_ep_combine(const UmdkEpCombineParams* p, void* stream) {
  CombineArgs a;
  if (int rc = fill_geom(&a.g, p->R, p->rank, p->E, p->K, p->H, p->cap, 0)) return rc;
  a.off = ep_normal_offsets(layout_geom(a.g));
  for (int i = 0; i < p->R; ++i) a.peers.base[i] = static_cast<uint8_t*>(p->peers[i]);
  a.y = static_cast<const __nv_bfloat16*>(p->y);
  a.recv_meta = p->recv_meta;
  a.counts_dev = p->counts_dev;
  a.src_idx = p->src_idx;
  a.n_rows = p->n_rows;
  a.in_rank = p->in_rank;
  a.topk_idx = p->topk_idx;
  a.topk_w = p->topk_w;
  a.out = static_cast<__nv_bfloat16*>(p->out);
  a.T = p->T;
  a.mode = p->mode;
  a.apply_weights = p->apply_weights;
  a.ctrl = p->ctrl;
  a.status = p->status;
  a.diag = p->diag;
  a.phase_mask = p->phase_mask ? p->phase_mask : 3;
  if (p->T > p->cap) return -UMDK_ERR_BAD_ARG;
  int grid = p->num_ctas > 0 ? p->num_ctas : sm_count();
  if (grid > sm_count()) grid = sm_count();
  ep_combine_kernel<<<grid, kEpThreads, 0, static_cast<cudaStream_t>(stream)>>>(a);
  UMDK_CUDA_CHECK(cudaGetLastError());
  return 0;
}

// ------------------------------------------------------------------------------------------------------------
// Standalone notify: the count exchange of dispatch as an operator of its own
// ------------------------------------------------------------------------------------------------------------
// Every rank sends, to each peer, how many of its (token, k) pairs go to each of that peer's local experts and how
// many tokens it sends there at all; from what it receives it derives the totals and prefix tables a receiver needs
// to size and address its buffers. Same outputs as the reference's notify_dispatch
// (src/cam/comm_operator/ascend_kernels/notify_dispatch/op_kernel/notify_dispatch.h:91-160: totalRecvTokens, recvCount
// as inclusive prefix over [localExpert][srcRank], recvOffset, maxBs, recvTokensPerExpert). Dispatch does the same
// exchange internally; this entry exists for callers that want the numbers before they dispatch. Own flag region and
// epoch word (ctrl[8]), so it can be mixed freely with dispatch / combine calls.
struct NotifyArgs {
  EpGeom g;
  EpNormalOffsets off;
  PeerTable peers;
  long long meet_cycles;       // budget of the wait for the peers' counts
  const int* num_per_expert;   // [E]
  const int* num_per_rank;     // [R]
  int* recv_count;             // [E_local * R] inclusive prefix, index = le * R + src
  int* recv_offset;            // [E_local * R] exclusive prefix
  int64_t* recv_per_expert;    // [E_local]
  int* totals;                 // [4]: rows to receive, arrivals (tokens) to receive, max tokens from one source, 0
  uint32_t* ctrl;              // [8] epoch of this operator
  int* status;
  int phase_mask;              // 1 = send, 2 = receive
};

__global__ void __launch_bounds__(256, 1) ep_notify_kernel(const NotifyArgs a) {
  const EpGeom& g = a.g;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  __shared__ int s_cnt[1024];
  __shared__ int s_ok;
  const uint32_t epoch = a.ctrl[8];
  const int h = epoch & 1;
  const uint64_t tag = (uint64_t)epoch + 1;
  const int nw = ep_notify_words(g.E_local);
  if (threadIdx.x == 0) s_ok = 1;
  __syncthreads();
  if (a.phase_mask & 1) {
    for (int d = warp; d < g.R; d += 8) {
      int* dst = reinterpret_cast<int*>(a.peers.base[d] + a.off.snotify[h]) + (size_t)g.rank * nw;
      for (int i = lane; i < g.E_local; i += 32) dst[i] = a.num_per_expert[d * g.E_local + i];
      if (lane == 0) dst[g.E_local] = a.num_per_rank[d];
      __threadfence_system();
      __syncwarp();
      if (lane == 0) {
        st_release_sys(reinterpret_cast<uint64_t*>(a.peers.base[d] + a.off.snotify_flag[h]) + g.rank, tag);
      }
    }
  }
  if (!(a.phase_mask & 2)) return;
  uint8_t* self = a.peers.base[g.rank];
  if (threadIdx.x < g.R) {
    const uint64_t* f = reinterpret_cast<const uint64_t*>(self + a.off.snotify_flag[h]) + threadIdx.x;
    if (!wait_flag_ge_sys(f, tag, a.meet_cycles)) {
      umdk_set_status(a.status, UMDK_ERR_TIMEOUT, UMDK_PH_DISPATCH_COUNT, threadIdx.x, (int)epoch);
      s_ok = 0;
    }
  }
  __syncthreads();
  if (!s_ok) return;
  const int* notify = reinterpret_cast<const int*>(self + a.off.snotify[h]);
  const int nle = g.E_local * g.R;
  for (int i = threadIdx.x; i < nle; i += blockDim.x) s_cnt[i] = __ldcg(notify + (size_t)(i % g.R) * nw + i / g.R);
  __syncthreads();
  if (threadIdx.x == 0) {
    int run = 0, arrivals = 0, max_src = 0;
    for (int i = 0; i < nle; ++i) {
      a.recv_offset[i] = run;
      run += s_cnt[i];
      a.recv_count[i] = run;
      if ((i % g.R) == g.R - 1) {
        const int le = i / g.R;
        a.recv_per_expert[le] = (int64_t)(run - a.recv_offset[le * g.R]);
      }
    }
    for (int r = 0; r < g.R; ++r) {
      const int c = __ldcg(notify + (size_t)r * nw + g.E_local);
      arrivals += c;
      max_src = max(max_src, c);
    }
    a.totals[0] = run;
    a.totals[1] = arrivals;
    a.totals[2] = max_src;
    a.totals[3] = 0;
    a.ctrl[8] = epoch + 1;
  }
}

struct UmdkEpNotifyParams {
  int R, rank, E, K, H, cap, phase_mask;
  void* peers[kMaxRanks];
  const int* num_per_expert;
  const int* num_per_rank;
  int* recv_count;
  int* recv_offset;
  int64_t* recv_per_expert;
  int* totals;
  uint32_t* ctrl;
  int* status;
};

UMDK_API int umdk_ep_notify(const UmdkEpNotifyParams* p, void* stream) {
  NotifyArgs a;
  a.meet_cycles = umdk_rendezvous_cycles();
  if (int rc = fill_geom(&a.g, p->R, p->rank, p->E, p->K, p->H, p->cap, 0)) return rc;
  if (a.g.E_local * a.g.R > 1024) return -UMDK_ERR_BAD_ARG;
  a.off = ep_normal_offsets(layout_geom(a.g));
  for (int i = 0; i < p->R; ++i) a.peers.base[i] = static_cast<uint8_t*>(p->peers[i]);
  a.num_per_expert = p->num_per_expert;
  a.num_per_rank = p->num_per_rank;
  a.recv_count = p->recv_count;
  a.recv_offset = p->recv_offset;
  a.recv_per_expert = p->recv_per_expert;
  a.totals = p->totals;
  a.ctrl = p->ctrl;
  a.status = p->status;
  a.phase_mask = p->phase_mask ? p->phase_mask : 3;
  ep_notify_kernel<<<1, 256, 0, static_cast<cudaStream_t>(stream)>>>(a);
  UMDK_CUDA_CHECK(cudaGetLastError());
  return 0;
}

// ------------------------------------------------------------------------------------------------------------
// Allocation-free layout entry point (see ep_layout_noalloc.h for who needs it and the rules that come with it)
// ------------------------------------------------------------------------------------------------------------
#include "ep_layout_noalloc.h"

#include <mutex>

// Layout of the array: [0, 256) bytes = grid-barrier words (two uint32 used), then the per-chunk histogram.
// In host code this name is only a stand-in for the symbol; the device address comes from cudaGetSymbolAddress.
static __device__ __align__(256) unsigned char g_layout_noalloc_scratch[UMDK_EP_LAYOUT_NOALLOC_BYTES];

static int layout_noalloc_scratch_ptr(unsigned char** out) {
  static std::mutex mu;
  static unsigned char* per_device[64] = {nullptr};
  int dev = -1;
  UMDK_CUDA_CHECK(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64) return -UMDK_ERR_BAD_ARG;
  std::lock_guard<std::mutex> lock(mu);
  if (per_device[dev] == nullptr) {
    void* p = nullptr;
    UMDK_CUDA_CHECK(cudaGetSymbolAddress(&p, g_layout_noalloc_scratch));
    per_device[dev] = static_cast<unsigned char*>(p);
  }
  *out = per_device[dev];
  return 0;
}

UMDK_API int umdk_ep_layout_noalloc(const int64_t* topk_idx, int T, int K, int E, int R, int* num_per_expert,
                                    int* num_per_rank, uint8_t* in_rank, int* send_idx, int* rank_slot, int* status,
                                    void* stream) {
  if (T < 0 || K < 1 || K > kMaxTopk || R < 1 || R > kMaxRanks || E < R || (E % R)) return -UMDK_ERR_BAD_ARG;
  if (T > UMDK_EP_LAYOUT_NOALLOC_MAX_TOKENS || E + R > UMDK_EP_LAYOUT_NOALLOC_MAX_COLS) {
    fprintf(stderr,
            "[umdk] umdk_ep_layout_noalloc: T=%d (max %d) or num_experts+num_ranks=%d (max %d) exceeds the built-in "
            "scratch; use umdk_ep_layout with caller-provided scratch instead\n",
            T, UMDK_EP_LAYOUT_NOALLOC_MAX_TOKENS, E + R, UMDK_EP_LAYOUT_NOALLOC_MAX_COLS);
    return -UMDK_ERR_BAD_ARG;
  }
  unsigned char* base = nullptr;
  if (int rc = layout_noalloc_scratch_ptr(&base)) return rc;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (T == 0) {
    UMDK_CUDA_CHECK(cudaMemsetAsync(num_per_expert, 0, sizeof(int) * E, s));
    UMDK_CUDA_CHECK(cudaMemsetAsync(num_per_rank, 0, sizeof(int) * R, s));
    return 0;
  }
  uint32_t* bar = reinterpret_cast<uint32_t*>(base);
  int* scratch = reinterpret_cast<int*>(base + 256);
  // the barrier must start from a clean arrival count even if an earlier call was cut short
  UMDK_CUDA_CHECK(cudaMemsetAsync(bar, 0, 2 * sizeof(uint32_t), s));
  const int chunks = (T + 31) / 32;
  int grid = (chunks + kLayoutWarps - 1) / kLayoutWarps;
  if (grid > sm_count()) grid = sm_count();
  const size_t smem = sizeof(int) * (size_t)kLayoutWarps * ((E + R) + 32 * kMaxTopk);
  if (smem > 48 * 1024) {
    UMDK_CUDA_CHECK(cudaFuncSetAttribute(ep_layout_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  }
  ep_layout_kernel<<<grid, kLayoutWarps * 32, smem, s>>>(topk_idx, T, K, E, R, num_per_expert, num_per_rank, in_rank,
                                                         send_idx, rank_slot, scratch, bar, status);
  UMDK_CUDA_CHECK(cudaGetLastError());
  return 0;
}
