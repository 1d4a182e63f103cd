// Pieces shared by the tensor-parallel fused GEMM kernels (tp_gemm.cu: one CTA per tile; tp_gemm_2sm.cu: one CTA
// pair per tile): the argument block, the copy role of all-gather -> GEMM and the owner-side reduction of
// GEMM -> reduce-scatter.
#pragma once
#include "common.h"
#include "ep_common.cuh"
#include "ptx.cuh"
#include "sync.cuh"

namespace umdk {

constexpr int kTpThreads = 256;

struct TpArgs {
  int mode;
  int R, rank;
  int Ts;          // rows per rank shard (multiple of 128)
  int N, K;        // GEMM N and K seen by this rank
  int n_copy;      // MODE 0: number of copy CTAs (the first n_copy CTAs of the grid)
  PeerTable peers;
  // MODE 0
  uint64_t x_slot_off[2];   // [Ts, K] bf16 shard of each rank (ping-pong)
  uint64_t ready_off[2];    // [R] uint64: peer r's shard for this epoch is in place
  const __nv_bfloat16* x_local;  // this rank's shard [Ts, K]; the copy CTAs place it into the heap slot themselves
  __nv_bfloat16* xg;        // local gathered activations [R*Ts, K]
  uint32_t* chunk_done;     // [R] local counters, advanced by n_copy per call and source
  // MODE 1
  uint64_t recv_off[2];     // [R src][Ts][N] bf16 on every rank, one per epoch parity (a source may start call
                            // n+1 while the owner still reduces call n; call n+2 cannot start before that ended)
  uint64_t arrive_off;      // [R] uint32 counters on every rank, advanced by tiles*4 per call and source
  __nv_bfloat16* out;       // [Ts, N]
  uint32_t* ctrl;           // [0] epoch, [1] done counter, [2] copy-CTA counter
  int* status;
  // Normal use: 3. Splitting lets several ranks be emulated on one GPU by running each phase for every rank in turn:
  // MODE 0: 4 = only publish this rank's "shard ready" flags (one CTA), 3 = everything;
  // MODE 1: 1 = GEMM + push, 2 = wait + reduce. The epoch advances only when bit 1 (value 2) is set.
  int phase_mask;
};


// Copy role of MODE 0, run by the first n_copy CTAs of the grid (no tensor cores, no TMEM): place the own shard in
// its heap slot, tell the peers, then pull every peer's shard chunk by chunk into the gathered buffer and advance
// the chunk counters the GEMM CTAs wait on. `s_ok` is a shared-memory flag of the calling CTA.
__device__ __forceinline__ void tp_copy_role(const TpArgs& a, int n_copy, int slot, uint64_t tag, uint32_t epoch,
                                             int* s_ok) {
  const size_t shard_vec = (size_t)a.Ts * a.K * 2 / 16;
  const size_t per_cta = (shard_vec + n_copy - 1) / n_copy;
  const size_t v0 = (size_t)blockIdx.x * per_cta;
  const size_t v1 = v0 + per_cta < shard_vec ? v0 + per_cta : shard_vec;
  {
    // place this rank's shard into its heap slot; the last copy CTA to finish tells every peer it is in place
    const int4* from = reinterpret_cast<const int4*>(a.x_local);
    int4* to = reinterpret_cast<int4*>(a.peers.base[a.rank] + a.x_slot_off[slot]);
    for (size_t v = v0 + threadIdx.x; v < v1; v += kTpThreads) to[v] = from[v];
    if (cta_done_is_last(&a.ctrl[2], n_copy)) {
      if (threadIdx.x < a.R) {
        st_release_sys(reinterpret_cast<uint64_t*>(a.peers.base[threadIdx.x] + a.ready_off[slot]) + a.rank, tag);
      }
    }
  }
  for (int i = 0; i < a.R; ++i) {
    const int src = (a.rank + i) % a.R;
    if (threadIdx.x == 0) {
      const uint64_t* f = reinterpret_cast<const uint64_t*>(a.peers.base[a.rank] + a.ready_off[slot]) + src;
      if (!wait_flag_ge_sys(f, tag)) {
        umdk_set_status(a.status, UMDK_ERR_TIMEOUT, UMDK_PH_AG_CHUNK, src, (int)epoch);
        *s_ok = 0;
      }
    }
    __syncthreads();
    if (!*s_ok) break;
    const int4* from = reinterpret_cast<const int4*>(a.peers.base[src] + a.x_slot_off[slot]);
    int4* to = reinterpret_cast<int4*>(a.xg + (size_t)src * a.Ts * a.K);
    for (size_t v = v0 + threadIdx.x; v < v1; v += 4 * kTpThreads) {
      // four independent 16-byte loads in flight per thread
      int4 r0 = ld_relaxed_sys_v4(from + v), r1, r2, r3;
      const bool h1 = v + kTpThreads < v1, h2 = v + 2 * kTpThreads < v1, h3 = v + 3 * kTpThreads < v1;
      if (h1) r1 = ld_relaxed_sys_v4(from + v + kTpThreads);
      if (h2) r2 = ld_relaxed_sys_v4(from + v + 2 * kTpThreads);
      if (h3) r3 = ld_relaxed_sys_v4(from + v + 3 * kTpThreads);
      to[v] = r0;
      if (h1) to[v + kTpThreads] = r1;
      if (h2) to[v + 2 * kTpThreads] = r2;
      if (h3) to[v + 3 * kTpThreads] = r3;
    }
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) red_add_release_gpu(&a.chunk_done[src], 1u);
  }
}

// Copy role on the bulk-copy engine of the SM (for CTAs that ONLY copy): one thread streams 32 KB pieces
// peer memory -> shared memory -> local memory with untiled bulk copies, two half-rings of `kCopyHalf` pieces so that
// the loads of one half are in flight while the other half drains. A handful of CTAs keeps hundreds of KB in flight
// on NVLink without spending registers or issue slots, so few SMs are taken from the GEMM.
// `ring`: >= 2 * kCopyHalf * kCopyPiece bytes of shared memory (1024-aligned); `bars`: 2 * kCopyHalf mbarriers.
constexpr int kCopyPiece = 32768;
constexpr int kCopyHalf = 3;

struct BulkCopier {
  uint8_t* ring;
  uint64_t* bars;
  uint32_t use[2 * kCopyHalf];   // how often each slot's barrier has completed (parity = use & 1)
  int* status;

  __device__ __forceinline__ void init(uint8_t* r, uint64_t* b, int* st) {
    ring = r;
    bars = b;
    status = st;
    for (int i = 0; i < 2 * kCopyHalf; ++i) {
      use[i] = 0;
      mbar_init(&bars[i], 1);
    }
    mbar_fence_init();
  }
  // Copies bytes [b0, b1) of `src` to the same offsets of `dst` (one thread). Returns false on a barrier timeout.
  __device__ __forceinline__ bool copy(uint8_t* dst, const uint8_t* src, size_t b0, size_t b1) {
    size_t next = b0;          // next byte to load
    size_t drain_pos[2] = {0, 0};
    int drain_cnt[2] = {0, 0};
    auto issue_half = [&](int h) {
      drain_pos[h] = next;
      drain_cnt[h] = 0;
      for (int i = 0; i < kCopyHalf && next < b1; ++i) {
        const int s = h * kCopyHalf + i;
        const uint32_t n = (uint32_t)((b1 - next) < (size_t)kCopyPiece ? (b1 - next) : (size_t)kCopyPiece);
        mbar_expect_tx(&bars[s], n);
        bulk_load_1d(ring + (size_t)s * kCopyPiece, src + next, n, &bars[s]);
        next += n;
        ++drain_cnt[h];
      }
    };
    issue_half(0);
    for (int h = 0; drain_cnt[h] > 0; h ^= 1) {
      issue_half(h ^ 1);   // the other half's earlier stores were waited for at the end of the previous round
      size_t pos = drain_pos[h];
      for (int i = 0; i < drain_cnt[h]; ++i) {
        const int s = h * kCopyHalf + i;
        if (!mbar_wait(&bars[s], use[s] & 1)) {
          umdk_set_status(status, UMDK_ERR_TIMEOUT, UMDK_PH_AG_CHUNK, s, (int)(pos >> 10));
          tma_store_wait<0>();
          return false;
        }
        ++use[s];
        const uint32_t n = (uint32_t)((b1 - pos) < (size_t)kCopyPiece ? (b1 - pos) : (size_t)kCopyPiece);
        bulk_store_1d(dst + pos, ring + (size_t)s * kCopyPiece, n);
        tma_store_commit();
        pos += n;
      }
      tma_store_wait_read<0>();   // this half's shared memory may be overwritten by the next loads
    }
    tma_store_wait<0>();          // everything written
    return true;
  }
};

__device__ __forceinline__ void tp_copy_role_bulk(const TpArgs& a, int n_copy, int slot, uint64_t tag, uint32_t epoch,
                                                  int* s_ok, uint8_t* ring, uint64_t* bars) {
  const size_t shard_bytes = (size_t)a.Ts * a.K * 2;
  const size_t npieces = (shard_bytes + kCopyPiece - 1) / kCopyPiece;
  const size_t per = (npieces + n_copy - 1) / n_copy;
  size_t b0 = (size_t)blockIdx.x * per * kCopyPiece, b1 = b0 + per * kCopyPiece;
  if (b0 > shard_bytes) b0 = shard_bytes;
  if (b1 > shard_bytes) b1 = shard_bytes;
  __shared__ BulkCopier bc;
  if (threadIdx.x == 0) {
    bc.init(ring, bars, a.status);
    // own shard into its heap slot; the last copy CTA to finish tells every peer that it is in place
    if (!bc.copy(a.peers.base[a.rank] + a.x_slot_off[slot], reinterpret_cast<const uint8_t*>(a.x_local), b0, b1))
      *s_ok = 0;
    fence_proxy_async_all();
  }
  if (cta_done_is_last(&a.ctrl[2], n_copy)) {
    if (threadIdx.x < a.R) {
      st_release_sys(reinterpret_cast<uint64_t*>(a.peers.base[threadIdx.x] + a.ready_off[slot]) + a.rank, tag);
    }
  }
  for (int i = 0; i < a.R; ++i) {
    const int src = (a.rank + i) % a.R;
    if (threadIdx.x == 0) {
      const uint64_t* f = reinterpret_cast<const uint64_t*>(a.peers.base[a.rank] + a.ready_off[slot]) + src;
      if (!wait_flag_ge_sys(f, tag)) {
        umdk_set_status(a.status, UMDK_ERR_TIMEOUT, UMDK_PH_AG_CHUNK, src, (int)epoch);
        *s_ok = 0;
      }
      if (*s_ok) {
        fence_proxy_async_all();   // the flag was read by the generic proxy, the data is read by the bulk engine
        if (!bc.copy(reinterpret_cast<uint8_t*>(a.xg + (size_t)src * a.Ts * a.K),
                     a.peers.base[src] + a.x_slot_off[slot], b0, b1))
          *s_ok = 0;
        fence_proxy_async_all();
        __threadfence();
      }
    }
    __syncthreads();
    if (!*s_ok) break;
    if (threadIdx.x == 0) red_add_release_gpu(&a.chunk_done[src], 1u);
  }
}

// Owner side of MODE 1, run by every CTA after its tiles: wait (bounded) until every source rank has delivered
// `per_src` epilogue arrivals for this call, then sum the R partial results of the owned rows in fp32.
__device__ __forceinline__ void tp_owner_reduce(const TpArgs& a, uint32_t per_src, int slot, uint64_t tag,
                                                uint32_t epoch, int* s_ok) {
  // ---- owner-side reduction of the R partial results of this rank's rows ----
  if (threadIdx.x < a.R) {
    const uint32_t* f = reinterpret_cast<const uint32_t*>(a.peers.base[a.rank] + a.arrive_off) + threadIdx.x;
    if (!wait_flag_ge_sys(f, (uint32_t)tag * per_src)) {
      umdk_set_status(a.status, UMDK_ERR_TIMEOUT, UMDK_PH_RS_CHUNK, threadIdx.x, (int)epoch);
      *s_ok = 0;
    }
  }
  __syncthreads();
  if (*s_ok) {
    const size_t nvec = (size_t)a.Ts * a.N / 8;
    const int4* base = reinterpret_cast<const int4*>(a.peers.base[a.rank] + a.recv_off[slot]);
    for (size_t v = (size_t)blockIdx.x * kTpThreads + threadIdx.x; v < nvec; v += (size_t)gridDim.x * kTpThreads) {
      float acc[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) acc[i] = 0.f;
      for (int s0 = 0; s0 < a.R; s0 += 8) {   // up to eight sources' loads in flight before the first add
        int4 vals[8];
#pragma unroll
        for (int u = 0; u < 8; ++u) {
          if (s0 + u < a.R) vals[u] = ld_relaxed_sys_v4(base + (size_t)(s0 + u) * nvec + v);
        }
#pragma unroll
        for (int u = 0; u < 8; ++u) {
          if (s0 + u < a.R) {
            const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&vals[u]);
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              const float2 f = __bfloat1622float2(p[i]);
              acc[2 * i] += f.x;
              acc[2 * i + 1] += f.y;
            }
          }
        }
      }
      int4 o;
      __nv_bfloat162* po = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
      for (int i = 0; i < 4; ++i) po[i] = __floats2bfloat162_rn(acc[2 * i], acc[2 * i + 1]);
      reinterpret_cast<int4*>(a.out)[v] = o;
    }
  }
}

}  // namespace umdk
