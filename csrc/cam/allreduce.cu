// All-reduce over NVLink peer memory: one-shot (every rank reads all peers and reduces; latency-optimal for small
// messages) and two-shot (reduce-scatter then all-gather through peer loads; bandwidth-optimal for large ones).
// Data lives in a double-buffered region of the symmetric heap; barriers are epoch-tagged flags with bounded waits.
// There is no all-reduce in the reference (its operators only use point-to-point window traffic); this implements
// the all-reduce part of the tensor-parallel configuration.
#include "common.h"
#include "ep_common.cuh"
#include "ptx.cuh"
#include "sync.cuh"

namespace umdk {
namespace {

constexpr int kArThreads = 512;

struct ArArgs {
  int R, rank, algo;       // algo 0 = one-shot, 1 = two-shot (peer loads), 2 = NVLS (multimem reduce + broadcast in
                           // NVSwitch), 3 = two-shot with peer STORES only (reduce-scatter push, all-gather push),
                           // 4 = one-shot with peer stores only (every rank sends its vector to all peers)
  uint8_t* mc_base;        // multicast alias of the heap (algo 2)
  int in_place;            // input already sits in the heap buffer and the result stays there (no copies)
  PeerTable peers;
  uint64_t buf_off[2];     // [max_bytes] per epoch parity
  uint64_t flag_off;       // [3][R] uint64: start / middle / end barriers
  uint64_t cta_flag_off;   // [kMaxArCtas][R] uint64: per-CTA "slice in place" flags of the multi-CTA one-shot path
  const __nv_bfloat16* in; // local input (copied into the heap buffer by the kernel)
  __nv_bfloat16* out;
  size_t n;                // elements, multiple of 8 * R
  uint32_t* ctrl;          // [0] epoch, [1] done counter, [2..3] grid barrier
  int* status;
  int phase_mask;          // 1 = copy-in + publish, 2 = reduce (+ gather) ; 3 = both
};

__device__ __forceinline__ void acc8(float* acc, const int4& v) {
  const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 f = __bfloat1622float2(p[i]);
    acc[2 * i] += f.x;
    acc[2 * i + 1] += f.y;
  }
}
// Sum over all ranks of vector `v` of their buffers: the loads of up to eight peers are issued back to back, so one
// NVLink round trip covers them all instead of one round trip per peer.
__device__ __forceinline__ void reduce_over_ranks(float* acc, const PeerTable& peers, uint64_t off, int R, int rank,
                                                  size_t v) {
  for (int i0 = 0; i0 < R; i0 += 8) {
    int4 vals[8];
#pragma unroll
    for (int u = 0; u < 8; ++u) {
      if (i0 + u < R) {
        const int p = (rank + i0 + u) % R;
        vals[u] = ld_relaxed_sys_v4(reinterpret_cast<const int4*>(peers.base[p] + off) + v);
      }
    }
#pragma unroll
    for (int u = 0; u < 8; ++u) {
      if (i0 + u < R) {
        const __nv_bfloat162* p2 = reinterpret_cast<const __nv_bfloat162*>(&vals[u]);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const float2 f = __bfloat1622float2(p2[i]);
          acc[2 * i] += f.x;
          acc[2 * i + 1] += f.y;
        }
      }
    }
  }
}
__device__ __forceinline__ int4 pack8(const float* acc) {
  int4 o;
  __nv_bfloat162* po = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
  for (int i = 0; i < 4; ++i) po[i] = __floats2bfloat162_rn(acc[2 * i], acc[2 * i + 1]);
  return o;
}

// Barrier across ranks: the last CTA of this grid to arrive publishes `tag` to every peer; everyone then waits for
// all peers' flags. `which` selects one of the three flag rows.
__device__ bool rank_barrier(const ArArgs& a, int which, uint64_t tag, uint32_t* grid_cnt, bool publish, bool wait) {
  __shared__ int s_ok_b;
  if (threadIdx.x == 0) s_ok_b = 1;
  if (publish) {
    bool last;
    if (gridDim.x == 1) {  // latency path for small messages: no inter-CTA counting needed
      __syncthreads();
      if (threadIdx.x < a.R) __threadfence_system();
      last = true;
    } else {
      last = cta_done_is_last(grid_cnt, gridDim.x);
    }
    if (last && threadIdx.x < a.R) {
      st_release_sys(reinterpret_cast<uint64_t*>(a.peers.base[threadIdx.x] + a.flag_off) + which * a.R + a.rank, tag);
    }
  }
  __syncthreads();
  if (wait) {
    if (threadIdx.x < a.R) {
      const uint64_t* f = reinterpret_cast<const uint64_t*>(a.peers.base[a.rank] + a.flag_off) + which * a.R + threadIdx.x;
      if (!wait_flag_ge_sys(f, tag)) {
        umdk_set_status(a.status, UMDK_ERR_TIMEOUT, UMDK_PH_ALLREDUCE, which, threadIdx.x);
        s_ok_b = 0;
      }
    }
    __syncthreads();
  }
  return s_ok_b != 0;
}

// End of a call: the last CTA of the grid to get here tells every peer that this rank has finished reading their
// buffers of this parity (flag row 2; the buffers are reused two calls later) and advances the epoch. Being last to
// arrive also proves that every CTA has read the epoch at kernel start, so one counter serves both purposes.
__device__ __forceinline__ void finish_call(const ArArgs& a, uint64_t tag, uint32_t epoch) {
  bool last;
  if (gridDim.x == 1) {
    __syncthreads();
    if (threadIdx.x < a.R) __threadfence_system();
    last = true;
  } else {
    last = cta_done_is_last(&a.ctrl[1], gridDim.x);
  }
  if (last) {
    if (threadIdx.x < a.R) {
      st_release_sys(reinterpret_cast<uint64_t*>(a.peers.base[threadIdx.x] + a.flag_off) + 2 * a.R + a.rank, tag);
    }
    if (threadIdx.x == 0) a.ctrl[0] = epoch + 1;
  }
}

__global__ void __launch_bounds__(kArThreads, 1) allreduce_kernel(const ArArgs a) {
  __shared__ uint32_t s_epoch;
  if (threadIdx.x == 0) s_epoch = a.ctrl[0];
  __syncthreads();
  const uint32_t epoch = s_epoch;
  const int slot = epoch & 1;
  const uint64_t tag = (uint64_t)epoch + 1;
  const size_t nvec = a.n / 8;
  const size_t tid = (size_t)blockIdx.x * kArThreads + threadIdx.x;
  const size_t nthreads = (size_t)gridDim.x * kArThreads;
  int4* mine = reinterpret_cast<int4*>(a.peers.base[a.rank] + a.buf_off[slot]);

  if (a.algo == 3) {
    // Push variant: every byte that crosses NVLink is a store (posted, no round trip), the way ring / tree
    // libraries move data. Buffer of this parity on every rank: [0, n) gathered result, [n, 2n) staging with one
    // slot of n / R elements per source rank.
    const size_t per = nvec / a.R;
    const size_t lo = per * a.rank;
    const int4* src = reinterpret_cast<const int4*>(a.in);
    __shared__ int s_ok3;
    if (threadIdx.x == 0) s_ok3 = 1;
    __syncthreads();
    // phase bits: 1 = push contributions, 2 = reduce own slice + push result, 4 = copy out + finish (normal: all)
    const int pm = a.phase_mask;
    if (pm & 1) {
      if (epoch >= 2) {   // peers wrote nothing here since call e-2; they must also have finished READING it
        if (threadIdx.x < a.R) {
          const uint64_t* f =
              reinterpret_cast<const uint64_t*>(a.peers.base[a.rank] + a.flag_off) + 2 * a.R + threadIdx.x;
          if (!wait_flag_ge_sys(f, (uint64_t)epoch - 1)) {
            umdk_set_status(a.status, UMDK_ERR_TIMEOUT, UMDK_PH_ALLREDUCE, 3, threadIdx.x);
            s_ok3 = 0;
          }
        }
        __syncthreads();
        if (!s_ok3) return;
      }
      // reduce-scatter push: my contribution to slice p goes into peer p's staging slot [rank]
      for (int i = 1; i < a.R; ++i) {
        const int p = (a.rank + i) % a.R;
        int4* dst = reinterpret_cast<int4*>(a.peers.base[p] + a.buf_off[slot]) + nvec + per * a.rank;
        const int4* from = src + per * p;
        for (size_t v0 = tid; v0 < per; v0 += 4 * nthreads) {
          int4 r[4];
#pragma unroll
          for (int u = 0; u < 4; ++u)
            if (v0 + u * nthreads < per) r[u] = __ldg(from + v0 + u * nthreads);
#pragma unroll
          for (int u = 0; u < 4; ++u)
            if (v0 + u * nthreads < per) st_na_v4(dst + v0 + u * nthreads, r[u]);
        }
      }
    }
    if ((pm & 3) && !rank_barrier(a, 0, tag, &a.ctrl[1], pm & 1, pm & 2)) return;
    // reduce my slice (own input + R-1 staged contributions), keep it, and push it to every peer's result area
    if (pm & 2) {
      const int4* stage = mine + nvec;
      int4* out4 = reinterpret_cast<int4*>(a.out);
      for (size_t v = tid; v < per; v += nthreads) {
        float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
        int4 vals[8];
        vals[0] = __ldg(src + lo + v);
        acc8(acc, vals[0]);
        for (int i0 = 1; i0 < a.R; i0 += 8) {
#pragma unroll
          for (int u = 0; u < 8; ++u) {
            if (i0 + u < a.R) vals[u] = stage[per * ((a.rank + i0 + u) % a.R) + v];
          }
#pragma unroll
          for (int u = 0; u < 8; ++u) {
            if (i0 + u < a.R) acc8(acc, vals[u]);
          }
        }
        const int4 r = pack8(acc);
        out4[lo + v] = r;
        for (int i = 1; i < a.R; ++i) {
          const int p = (a.rank + i) % a.R;
          st_na_v4(reinterpret_cast<int4*>(a.peers.base[p] + a.buf_off[slot]) + lo + v, r);
        }
      }
    }
    if ((pm & 6) && !rank_barrier(a, 1, tag, &a.ctrl[1], pm & 2, pm & 4)) return;
    if (!(pm & 4)) return;
    // the other ranks' slices have landed in my result area: local copy into the output
    {
      int4* out4 = reinterpret_cast<int4*>(a.out);
      for (int i = 1; i < a.R; ++i) {
        const size_t off = per * ((a.rank + i) % a.R);
        for (size_t v0 = tid; v0 < per; v0 += 4 * nthreads) {
          int4 r[4];
#pragma unroll
          for (int u = 0; u < 4; ++u)
            if (v0 + u * nthreads < per) r[u] = mine[off + v0 + u * nthreads];
#pragma unroll
          for (int u = 0; u < 4; ++u)
            if (v0 + u * nthreads < per) out4[off + v0 + u * nthreads] = r[u];
        }
      }
    }
    finish_call(a, tag, epoch);
    return;
  }
  if (a.algo == 4) {
    // One-shot with stores only: CTA c sends its slice of the input to slot [rank] of every peer's buffer (posted
    // writes, no round trip), raises its per-CTA flag there, waits for the peers' slice-c flags and sums the slots
    // out of LOCAL memory. Buffer of this parity: R slots of n elements. Latency = one NVLink store + one flag.
    const size_t per_cta = (nvec + gridDim.x - 1) / gridDim.x;
    const size_t v_lo = per_cta * blockIdx.x;
    const size_t v_hi = v_lo + per_cta < nvec ? v_lo + per_cta : nvec;
    uint64_t* cta_flags = reinterpret_cast<uint64_t*>(a.peers.base[a.rank] + a.cta_flag_off);
    const int4* src = reinterpret_cast<const int4*>(a.in);
    __shared__ int s_okp;
    if (threadIdx.x == 0) s_okp = 1;
    __syncthreads();
    if (a.phase_mask & 1) {
      if (epoch >= 2 && threadIdx.x < a.R) {
        const uint64_t* f =
            reinterpret_cast<const uint64_t*>(a.peers.base[a.rank] + a.flag_off) + 2 * a.R + threadIdx.x;
        if (!wait_flag_ge_sys(f, (uint64_t)epoch - 1)) {
          umdk_set_status(a.status, UMDK_ERR_TIMEOUT, UMDK_PH_ALLREDUCE, 3, threadIdx.x);
          s_okp = 0;
        }
      }
      __syncthreads();
      if (!s_okp) return;
      for (size_t v = v_lo + threadIdx.x; v < v_hi; v += kArThreads) {
        const int4 val = __ldg(src + v);
        for (int i = 1; i < a.R; ++i) {
          const int p = (a.rank + i) % a.R;
          st_na_v4(reinterpret_cast<int4*>(a.peers.base[p] + a.buf_off[slot]) + nvec * a.rank + v, val);
        }
      }
      __syncthreads();
      if (threadIdx.x < a.R) {
        __threadfence_system();
        st_release_sys(reinterpret_cast<uint64_t*>(a.peers.base[threadIdx.x] + a.cta_flag_off) +
                           (size_t)blockIdx.x * a.R + a.rank,
                       tag);
      }
    }
    if (!(a.phase_mask & 2)) return;
    if (threadIdx.x < a.R) {
      if (!wait_flag_ge_sys(cta_flags + (size_t)blockIdx.x * a.R + threadIdx.x, tag)) {
        umdk_set_status(a.status, UMDK_ERR_TIMEOUT, UMDK_PH_ALLREDUCE, 0, threadIdx.x);
        s_okp = 0;
      }
    }
    __syncthreads();
    if (!s_okp) return;
    int4* dst = reinterpret_cast<int4*>(a.out);
    for (size_t v = v_lo + threadIdx.x; v < v_hi; v += kArThreads) {
      float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
      acc8(acc, __ldg(src + v));
      for (int i0 = 1; i0 < a.R; i0 += 8) {
        int4 vals[8];
#pragma unroll
        for (int u = 0; u < 8; ++u) {
          if (i0 + u < a.R) vals[u] = mine[nvec * ((a.rank + i0 + u) % a.R) + v];
        }
#pragma unroll
        for (int u = 0; u < 8; ++u) {
          if (i0 + u < a.R) acc8(acc, vals[u]);
        }
      }
      dst[v] = pack8(acc);
    }
    finish_call(a, tag, epoch);
    return;
  }
  if (a.algo == 0 && gridDim.x > 1 && !a.in_place) {
    // One-shot with several CTAs and NO grid-wide step on the critical path: CTA c owns the contiguous slice c of the
    // vector on every rank, announces "my slice c is in place" to CTA c of every peer through its own flag word and
    // waits only for the peers' slice-c flags. (All ranks launch the same grid for the same size.)
    const size_t per_cta = (nvec + gridDim.x - 1) / gridDim.x;
    const size_t v_lo = per_cta * blockIdx.x;
    const size_t v_hi = v_lo + per_cta < nvec ? v_lo + per_cta : nvec;
    uint64_t* cta_flags = reinterpret_cast<uint64_t*>(a.peers.base[a.rank] + a.cta_flag_off);
    __shared__ int s_okf;
    if (threadIdx.x == 0) s_okf = 1;
    __syncthreads();
    if (a.phase_mask & 1) {
      if (epoch >= 2 && threadIdx.x < a.R) {   // buffer reuse: the peers' call e-2 has ended (flag row 2)
        const uint64_t* f =
            reinterpret_cast<const uint64_t*>(a.peers.base[a.rank] + a.flag_off) + 2 * a.R + threadIdx.x;
        if (!wait_flag_ge_sys(f, (uint64_t)epoch - 1)) {
          umdk_set_status(a.status, UMDK_ERR_TIMEOUT, UMDK_PH_ALLREDUCE, 3, threadIdx.x);
          s_okf = 0;
        }
      }
      __syncthreads();
      if (!s_okf) return;
      const int4* src = reinterpret_cast<const int4*>(a.in);
      for (size_t v = v_lo + threadIdx.x; v < v_hi; v += kArThreads) mine[v] = src[v];
      __syncthreads();
      if (threadIdx.x < a.R) {
        __threadfence_system();
        st_release_sys(reinterpret_cast<uint64_t*>(a.peers.base[threadIdx.x] + a.cta_flag_off) +
                           (size_t)blockIdx.x * a.R + a.rank,
                       tag);
      }
    }
    if (!(a.phase_mask & 2)) return;
    if (threadIdx.x < a.R) {
      if (!wait_flag_ge_sys(cta_flags + (size_t)blockIdx.x * a.R + threadIdx.x, tag)) {
        umdk_set_status(a.status, UMDK_ERR_TIMEOUT, UMDK_PH_ALLREDUCE, 0, threadIdx.x);
        s_okf = 0;
      }
    }
    __syncthreads();
    if (!s_okf) return;
    int4* dst = reinterpret_cast<int4*>(a.out);
    for (size_t v = v_lo + threadIdx.x; v < v_hi; v += kArThreads) {
      float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
      reduce_over_ranks(acc, a.peers, a.buf_off[slot], a.R, a.rank, v);
      dst[v] = pack8(acc);
    }
    finish_call(a, tag, epoch);
    return;
  }
  if ((a.phase_mask & 1) && !a.in_place) {
    // this buffer parity was last used two calls ago: every peer must have finished reading it
    if (epoch >= 2) {
      __shared__ int s_ok0;
      if (threadIdx.x == 0) s_ok0 = 1;
      __syncthreads();
      if (threadIdx.x < a.R) {
        const uint64_t* f = reinterpret_cast<const uint64_t*>(a.peers.base[a.rank] + a.flag_off) + 2 * a.R + threadIdx.x;
        if (!wait_flag_ge_sys(f, (uint64_t)epoch - 1)) {
          umdk_set_status(a.status, UMDK_ERR_TIMEOUT, UMDK_PH_ALLREDUCE, 3, threadIdx.x);
          s_ok0 = 0;
        }
      }
      __syncthreads();
      if (!s_ok0) return;
    }
    const int4* src = reinterpret_cast<const int4*>(a.in);
    for (size_t v = tid; v < nvec; v += nthreads) mine[v] = src[v];
  }
  if (!rank_barrier(a, 0, tag, &a.ctrl[1], a.phase_mask & 1, a.phase_mask & 2)) return;
  if (!(a.phase_mask & 2)) return;

  if (a.algo == 0) {
    int4* dst = reinterpret_cast<int4*>(a.out);
    for (size_t v = tid; v < nvec; v += nthreads) {
      float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
      reduce_over_ranks(acc, a.peers, a.buf_off[slot], a.R, a.rank, v);
      dst[v] = pack8(acc);
    }
  } else if (a.algo == 2) {
    // NVLS: this rank owns slice `rank`; one multimem load reduces the slice over all ranks inside the switch and one
    // multimem store broadcasts the result into every rank's buffer (in place, nobody else touches this slice)
    const size_t per = nvec / a.R;
    const size_t lo = per * a.rank;
    uint8_t* mc = a.mc_base + a.buf_off[slot];
    // four switch reductions in flight per thread before the first broadcast store
    for (size_t v0 = tid; v0 < per; v0 += 4 * nthreads) {
      int4 r[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        if (v0 + u * nthreads < per) r[u] = multimem_ld_reduce_bf16x8(mc + (lo + v0 + u * nthreads) * 16);
      }
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        if (v0 + u * nthreads < per) multimem_st_v4(mc + (lo + v0 + u * nthreads) * 16, r[u]);
      }
    }
    if (!rank_barrier(a, 1, tag, &a.ctrl[1], true, true)) return;
    if (!a.in_place) {
      int4* dst = reinterpret_cast<int4*>(a.out);
      for (size_t v = tid; v < nvec; v += nthreads) dst[v] = mine[v];
    }
  } else {
    // stage 1: reduce my 1/R slice from all peers into my own buffer (in place: only I write my slice)
    const size_t per = nvec / a.R;
    const size_t lo = per * a.rank;
    for (size_t v = tid; v < per; v += nthreads) {
      float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
      reduce_over_ranks(acc, a.peers, a.buf_off[slot], a.R, a.rank, lo + v);
      mine[lo + v] = pack8(acc);
    }
    if (!rank_barrier(a, 1, tag, &a.ctrl[1], true, true)) return;
    // stage 2: gather every rank's reduced slice
    int4* dst = reinterpret_cast<int4*>(a.out);
    for (int i = 0; i < a.R; ++i) {
      const int p = (a.rank + i) % a.R;
      const int4* from = reinterpret_cast<const int4*>(a.peers.base[p] + a.buf_off[slot]) + per * p;
      for (size_t v0 = tid; v0 < per; v0 += 4 * nthreads) {
        int4 r[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          if (v0 + u * nthreads < per) r[u] = ld_relaxed_sys_v4(from + v0 + u * nthreads);
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          if (v0 + u * nthreads < per) dst[per * p + v0 + u * nthreads] = r[u];
        }
      }
    }
  }
  finish_call(a, tag, epoch);
}

}  // namespace
}  // namespace umdk

using namespace umdk;

struct UmdkAllreduceParams {
  int R, rank, algo, num_ctas, phase_mask;
  void* peers[kMaxRanks];
  uint64_t buf_off[2];
  uint64_t flag_off;
  const void* in;
  void* out;
  unsigned long long n;
  uint32_t* ctrl;
  int* status;
  void* mc_base;
  int in_place;
  unsigned long long buf_bytes;   // size of each parity buffer (algo 3 needs 2 * n * 2 bytes of it)
};

constexpr int kMaxArCtas = 160;

UMDK_API long long umdk_allreduce_heap_bytes(unsigned long long max_bytes, int R) {
  return (long long)(2 * align_up_u64(max_bytes, 1024) + align_up_u64(3ull * R * 8, 256) +
                     align_up_u64((uint64_t)kMaxArCtas * R * 8, 256));
}

UMDK_API int umdk_allreduce(const UmdkAllreduceParams* p, void* stream) {
  if (p->R < 1 || p->R > kMaxRanks || p->n == 0 || (p->n % (8ull * p->R))) return -UMDK_ERR_BAD_ARG;
  ArArgs a;
  a.R = p->R;
  a.rank = p->rank;
  a.algo = p->algo;
  for (int i = 0; i < kMaxRanks; ++i) a.peers.base[i] = i < p->R ? static_cast<uint8_t*>(p->peers[i]) : nullptr;
  a.buf_off[0] = p->buf_off[0];
  a.buf_off[1] = p->buf_off[1];
  a.flag_off = p->flag_off;
  a.cta_flag_off = p->flag_off + align_up_u64(3ull * p->R * 8, 256);
  a.in = static_cast<const __nv_bfloat16*>(p->in);
  a.out = static_cast<__nv_bfloat16*>(p->out);
  a.n = p->n;
  a.ctrl = p->ctrl;
  a.status = p->status;
  a.phase_mask = p->phase_mask ? p->phase_mask : (p->algo == 3 ? 7 : 3);
  a.mc_base = static_cast<uint8_t*>(p->mc_base);
  a.in_place = p->in_place;
  if (a.algo == 2 && a.mc_base == nullptr) return -UMDK_ERR_BAD_ARG;
  if (a.algo == 3 && p->buf_bytes < 4ull * p->n) return -UMDK_ERR_BAD_ARG;
  if (a.algo == 4 && p->buf_bytes < 2ull * p->n * p->R) return -UMDK_ERR_BAD_ARG;
  if (a.algo < 0 || a.algo > 4) return -UMDK_ERR_BAD_ARG;
  int grid = p->num_ctas;
  if (grid <= 0) {
    const size_t nvec = p->n / 8;
    grid = nvec <= 2048 ? 1 : (int)((nvec + kArThreads * 2 - 1) / (kArThreads * 2));
    if (grid < 1) grid = 1;
  }
  if (grid > sm_count()) grid = sm_count();
  if (grid > kMaxArCtas) grid = kMaxArCtas;
  allreduce_kernel<<<grid, kArThreads, 0, static_cast<cudaStream_t>(stream)>>>(a);
  UMDK_CUDA_CHECK(cudaGetLastError());
  return 0;
}
