// Device-side body of the low-latency (decode) expert-parallel dispatch, shared by the stand-alone dispatch kernel
// (ep_ll.cu) and by the fused MoE kernel (moe_fused.cu), which runs it as its prologue so that a decode layer is ONE
// launch: per-expert counts are all-gathered through peer memory, then every (token, k) is quantised to fp8 e4m3
// (fp32 scale per 1x128 block) and stored straight into its final row of the destination rank's expert-major slab.
// All scratch lives in a caller-provided shared-memory area (the fused kernel lends its operand ring).
#pragma once
#include "ep_common.cuh"
#include "ptx.cuh"
#include "sync.cuh"

namespace umdk {

struct LLDispatchIO {
  const __nv_bfloat16* x;     // [T, H]
  const int64_t* topk_idx;    // [T, K] (-1 = skip)
  const int* send_idx;        // [T, K] position inside the expert bucket on this rank (layout kernel), or null:
                              // then every CTA derives both tables from topk_idx itself, in shared memory
  const int* num_per_expert;  // [E] (null together with send_idx)
  int T;
  int* group_off;             // out [E_local + 1]: row offsets of this rank's experts inside its slab
  int64_t* recv_per_expert;   // out [E_local]
  uint32_t* ctrl;             // [0] epoch (read), [3] send-done counter
  int* status;
  int phase_mask;             // bit0: publish counts; bit1: wait counts, push rows, raise data flags
  long long meet_cycles;      // budget of the wait for the peers' counts (where the ranks meet); 0 = the usual budget
};

// Shared-memory bytes the body needs: four int tables over the experts, destination pointers per warp, and (layout
// inside the kernel) 16-bit histogram / position / expert-id tables.
__host__ __device__ inline size_t ll_dispatch_smem_bytes(int T, int E, int K, int nwarps, bool own_layout) {
  size_t n = 16 + 4 * (size_t)E * 4 + 2 * (size_t)nwarps * kMaxTopk * 8;
  if (own_layout) n += 2 * ((size_t)((T + 31) / 32) * E + 2 * (size_t)T * K);
  return (n + 15) / 16 * 16;
}

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

// Quantises 16 consecutive elements held by this lane; 8 lanes share a 1x128 block. Returns the packed fp8 and
// writes the block scale to *scale (same value on the 8 lanes).
__device__ __forceinline__ int4 quant16(const float* f, float* scale) {
  float amax = 0.f;
#pragma unroll
  for (int i = 0; i < 16; ++i) amax = fmaxf(amax, fabsf(f[i]));
  amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
  amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
  amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 4));
  amax = fmaxf(amax, 1e-4f);
  *scale = amax * (1.f / 448.f);
  const float inv = 448.f / amax;
  int4 q;
  q.x = pack_fp8x4(f[0] * inv, f[1] * inv, f[2] * inv, f[3] * inv);
  q.y = pack_fp8x4(f[4] * inv, f[5] * inv, f[6] * inv, f[7] * inv);
  q.z = pack_fp8x4(f[8] * inv, f[9] * inv, f[10] * inv, f[11] * inv);
  q.w = pack_fp8x4(f[12] * inv, f[13] * inv, f[14] * inv, f[15] * inv);
  return q;
}


// Runs the dispatch for the calling CTA (all `kThreads` threads of it must call). Returns false when a bounded wait
// ran out (the status record says which). `goff_sm` (optional, shared memory, [E_local + 1]) receives this rank's
// group offsets in every CTA. `scratch` must hold ll_dispatch_smem_bytes(...) bytes, 16-byte aligned.
template <int kThreads>
__device__ __forceinline__ bool ll_dispatch_body(const EpLLGeom& g, const EpLLOffsets& off, const PeerTable& peers,
                                                 const LLDispatchIO& a, uint8_t* scratch, int* goff_sm) {
  constexpr int kLLWarps = kThreads / 32;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  uint32_t* s_epoch_p = reinterpret_cast<uint32_t*>(scratch);
  int* s_ok_p = reinterpret_cast<int*>(scratch + 4);
  int* s_base = reinterpret_cast<int*>(scratch + 16);       // destination row base of my tokens, per global expert
  int* s_npe = s_base + g.E;
  int* s_tot = s_npe + g.E;
  int* s_before = s_tot + g.E;
  uint8_t** s_dx = reinterpret_cast<uint8_t**>(s_before + g.E);          // [kLLWarps][kMaxTopk]
  float** s_ds = reinterpret_cast<float**>(s_dx + kLLWarps * kMaxTopk);   // [kLLWarps][kMaxTopk]
  uint8_t* ll_dyn = reinterpret_cast<uint8_t*>(s_ds + kLLWarps * kMaxTopk);
#define s_epoch (*s_epoch_p)
#define s_ok (*s_ok_p)
  if (threadIdx.x == 0) {
    s_epoch = a.ctrl[0];
    s_ok = 1;
  }
  // ---- layout inside the kernel (decode-sized inputs) ----
  // Every CTA computes, for all T x K entries, the position of the entry inside its expert's bucket (token-major
  // order) and the bucket sizes: per 32-token chunk a warp walks its tokens in order with shared-memory counters,
  // then the chunks are scanned per expert. A few microseconds of redundant work per CTA instead of a kernel launch
  // and a pass through global memory.
  const bool own_layout = a.send_idx == nullptr;
  const int n_chunks = (a.T + 31) / 32;
  uint16_t* s_hist = reinterpret_cast<uint16_t*>(ll_dyn);              // [n_chunks][E] counts, then exclusive bases
  uint16_t* s_sidx = s_hist + (size_t)n_chunks * g.E;                  // [T * K] positions
  int16_t* s_eid = reinterpret_cast<int16_t*>(s_sidx + (size_t)a.T * g.K);   // [T * K] expert ids (-1 = none)
  if (own_layout) {
    // all indices first, in one round of loads: the walk below must not wait on global memory at every step
    for (int i = threadIdx.x; i < a.T * g.K; i += blockDim.x) {
      const long long ee = a.topk_idx[i];
      s_eid[i] = (ee >= 0 && ee < g.E) ? (int16_t)ee : (int16_t)-1;
    }
    for (int i = threadIdx.x; i < n_chunks * g.E; i += blockDim.x) s_hist[i] = 0;
    __syncthreads();
    for (int c = warp; c < n_chunks; c += kLLWarps) {
      uint16_t* hist = s_hist + (size_t)c * g.E;
      const int t_end = min(a.T, (c + 1) * 32);
      for (int t = c * 32; t < t_end; ++t) {
        if (lane < g.K) {
          const int ee = s_eid[(size_t)t * g.K + lane];
          uint16_t pos = 0xffff;
          if (ee >= 0) {
            // the K experts of one token are distinct, so the lanes touch different counters; a repeated expert in
            // one row would only make the two entries share a position, which the bounds checks below reject
            pos = hist[ee];
            hist[ee] = pos + 1;
          }
          s_sidx[(size_t)t * g.K + lane] = pos;
        }
        __syncwarp();
      }
    }
    __syncthreads();
    for (int e = threadIdx.x; e < g.E; e += blockDim.x) {
      int run = 0;
      for (int c = 0; c < n_chunks; ++c) {
        const int v = s_hist[(size_t)c * g.E + e];
        s_hist[(size_t)c * g.E + e] = (uint16_t)run;
        run += v;
      }
      s_npe[e] = run;
    }
    __syncthreads();
    for (int i = threadIdx.x; i < a.T * g.K; i += blockDim.x) {
      const int ee = s_eid[i];
      if (ee >= 0) s_sidx[i] += s_hist[(size_t)((i / g.K) / 32) * g.E + ee];
    }
  }
  __syncthreads();
  const uint32_t epoch = s_epoch;
  const uint64_t tag = (uint64_t)epoch + 1;
  uint8_t* self = peers.base[g.rank];

  if ((a.phase_mask & 1) && blockIdx.x == 0) {
    for (int d = warp; d < g.R; d += kLLWarps) {
      int* dst = reinterpret_cast<int*>(peers.base[d] + off.cnt[0]) + (size_t)g.rank * g.E;
      for (int i = lane; i < g.E; i += 32) dst[i] = own_layout ? s_npe[i] : a.num_per_expert[i];
      __threadfence_system();
      __syncwarp();
      if (lane == 0) st_release_sys(reinterpret_cast<uint64_t*>(peers.base[d] + off.cnt_flag[0]) + g.rank, tag);
    }
  }
  if (!(a.phase_mask & 2)) return true;

  if (threadIdx.x < g.R) {
    const uint64_t* f = reinterpret_cast<const uint64_t*>(self + off.cnt_flag[0]) + threadIdx.x;
    if (!wait_flag_ge_sys(f, tag, a.meet_cycles > 0 ? a.meet_cycles : kSpinLimitCycles)) {
      umdk_set_status(a.status, UMDK_ERR_TIMEOUT, UMDK_PH_DISPATCH_COUNT, threadIdx.x, (int)epoch);
      s_ok = 0;
    }
  }
  __syncthreads();
  if (!s_ok) return false;
  const int* cnt = reinterpret_cast<const int*>(self + off.cnt[0]);  // [src][E]
  // per-expert totals over sources, then exclusive prefix inside each destination rank
  // totals over sources and the part that comes from lower-numbered sources (my rows start after theirs); the
  // loads of eight sources are issued together
  for (int e = threadIdx.x; e < g.E; e += blockDim.x) {
    int tot = 0, before = 0;
    for (int s0 = 0; s0 < g.R; s0 += 8) {
      int v[8];
#pragma unroll
      for (int u = 0; u < 8; ++u) v[u] = s0 + u < g.R ? __ldcg(cnt + (size_t)(s0 + u) * g.E + e) : 0;
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        tot += v[u];
        if (s0 + u < g.rank) before += v[u];
      }
    }
    s_tot[e] = tot;
    s_before[e] = before;
  }
  __syncthreads();
  // one thread per destination rank walks its experts (E_local steps)
  if (threadIdx.x < g.R) {
    const int d = threadIdx.x;
    int run = 0;
    for (int le = 0; le < g.E_local; ++le) {
      const int e = d * g.E_local + le;
      s_base[e] = run;
      run += s_tot[e];
      if (d == g.rank) {
        if (goff_sm != nullptr) {
          goff_sm[le] = s_base[e];
          if (le == g.E_local - 1) goff_sm[g.E_local] = run;
        }
        if (blockIdx.x == 0) {
          a.group_off[le] = s_base[e];
          a.recv_per_expert[le] = (int64_t)s_tot[e];
          if (le == g.E_local - 1) {
            a.group_off[g.E_local] = run;
            if (run > g.n_cap) umdk_set_status(a.status, UMDK_ERR_OVERFLOW, UMDK_PH_DISPATCH_COUNT, run, g.n_cap);
          }
        }
      }
    }
  }
  __syncthreads();
  for (int e = threadIdx.x; e < g.E; e += blockDim.x) s_base[e] += s_before[e];
  __syncthreads();

  const int nblk = g.H / 128;
  // One work item = 16 consecutive 1x128 blocks (2 KiB of fp8) of one token: a warp has all its eight 16-byte loads
  // in flight at once, and a decode-sized batch still spreads over every warp of the grid.
  const int nparts = (nblk + 15) / 16;
  for (int item = blockIdx.x * kLLWarps + warp; item < a.T * nparts; item += gridDim.x * kLLWarps) {
    const int t = item / nparts, part = item - t * nparts;
    __syncwarp();
    if (lane < g.K) {
      const long long ee = own_layout ? (long long)s_eid[(size_t)t * g.K + lane] : a.topk_idx[(size_t)t * g.K + lane];
      uint8_t* dx = nullptr;
      float* ds = nullptr;
      if (ee >= 0 && ee < g.E) {
        const int e = (int)ee, d = e / g.E_local;
        const int row = s_base[e] + (own_layout ? (int)s_sidx[(size_t)t * g.K + lane]
                                               : a.send_idx[(size_t)t * g.K + lane]);
        if (row < 0 || row >= g.n_cap) {
          umdk_set_status(a.status, UMDK_ERR_OVERFLOW, UMDK_PH_DISPATCH_DATA, e, row);
        } else {
          dx = peers.base[d] + off.slab_x[0] + (size_t)row * g.H;
          ds = reinterpret_cast<float*>(peers.base[d] + off.slab_s[0]) + (size_t)row * nblk;
          if (part == 0) {
            int* meta = reinterpret_cast<int*>(peers.base[d] + off.slab_meta[0]) + (size_t)row * 2;
            meta[0] = g.rank;
            meta[1] = t * g.K + lane;
          }
        }
      }
      s_dx[warp * kMaxTopk + lane] = dx;
      s_ds[warp * kMaxTopk + lane] = ds;
    }
    __syncwarp();
    const int4* xrow = reinterpret_cast<const int4*>(a.x + (size_t)t * g.H);
    const int b0 = part * 16;
    int4 raw[4][2];
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int blk = b0 + 4 * u + (lane >> 3);
      if (blk < nblk) {
        raw[u][0] = __ldg(xrow + blk * 16 + (lane & 7) * 2);
        raw[u][1] = __ldg(xrow + blk * 16 + (lane & 7) * 2 + 1);
      } else {
        raw[u][0] = raw[u][1] = make_int4(0, 0, 0, 0);
      }
    }
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int blk = b0 + 4 * u + (lane >> 3);
      float f[16];
      bf16x8_to_float(raw[u][0], f);
      bf16x8_to_float(raw[u][1], f + 8);
      float scale;
      const int4 q = quant16(f, &scale);   // shuffles inside: executed by all lanes
      if (blk < nblk) {
        for (int k = 0; k < g.K; ++k) {
          uint8_t* dx = s_dx[warp * kMaxTopk + k];
          if (dx == nullptr) continue;
          st_na_v4(dx + blk * 128 + (lane & 7) * 16, q);
          if ((lane & 7) == 0) s_ds[warp * kMaxTopk + k][blk] = scale;
        }
      }
    }
    // This part of the row has been stored at every destination: count it on each destination expert's arrival
    // word (the warp's stores are ordered before the release by the warp barrier). An expert's rows are complete
    // when its word has reached rows x parts-per-row; the fused kernel starts that expert's GEMM tiles then,
    // without waiting for the rest of the slab. Every lane fences its own stores at system scope first: the counting
    // lanes' release alone does not wait for stores that OTHER lanes still have in flight to the peer.
    __threadfence_system();
    __syncwarp();
    if (lane < g.K && s_dx[warp * kMaxTopk + lane] != nullptr) {
      const long long ee = own_layout ? (long long)s_eid[(size_t)t * g.K + lane] : a.topk_idx[(size_t)t * g.K + lane];
      const int e = (int)ee, d = e / g.E_local;
      red_add_release_sys(reinterpret_cast<uint32_t*>(peers.base[d] + off.exp_cnt[0]) + (e - d * g.E_local), 1u);
    }
  }
  if (cta_done_is_last(&a.ctrl[3], gridDim.x)) {
    if (threadIdx.x < g.R) {
      st_release_sys(reinterpret_cast<uint64_t*>(peers.base[threadIdx.x] + off.data_flag[0]) + g.rank, tag);
    }
  }
  return true;
#undef s_epoch
#undef s_ok
}

// Owner-side tail of the combine: out[t] = sum_k w[t, k] * row(t, k) over the rows that the expert ranks stored into
// this rank's combine buffer ([T][Kt][H] bf16), accumulated in fp32 and rounded once. With `share_out` the row of the
// LAST slot is copied there unweighted instead of being summed (the folded shared expert). The caller has already
// waited for every peer's completion flag.
template <int kThreads>
__device__ __forceinline__ void ll_weighted_reduce(const uint8_t* comb_buf, const int64_t* topk_idx,
                                                   const float* topk_w, __nv_bfloat16* out, __nv_bfloat16* share_out,
                                                   int T, int Kt, int H) {
  const int warp = threadIdx.x >> 5;
  // One work item = 512 bytes of one token's output (32 lanes x 16 bytes), spread over every warp of the grid: with
  // decode-sized batches a warp per token would leave most of the GPU idle while a few warps walk whole rows.
  // All K rows of an item are loaded before the first is used.
  const int lane = threadIdx.x & 31;
  const int nvec = H / 8;
  const int nchunk = (nvec + 31) / 32;
  const int nwarps = kThreads / 32;
  const int k_sum = share_out ? Kt - 1 : Kt;
  constexpr int kMaxK = 8;
  for (int item = blockIdx.x * nwarps + warp; item < T * nchunk; item += gridDim.x * nwarps) {
    const int t = item / nchunk;
    const int v = (item % nchunk) * 32 + lane;
    if (v >= nvec) continue;
    const int4* src = reinterpret_cast<const int4*>(comb_buf + (size_t)t * Kt * H * 2);
    if (share_out) {
      const bool have = topk_idx[(size_t)t * Kt + k_sum] >= 0;
      const int4 val = have ? ld_relaxed_sys_v4(src + (size_t)k_sum * nvec + v) : make_int4(0, 0, 0, 0);
      reinterpret_cast<int4*>(share_out + (size_t)t * H)[v] = val;
    }
    float acc[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[i] = 0.f;
    for (int k0 = 0; k0 < k_sum; k0 += kMaxK) {
      int4 vals[kMaxK];
      float wk[kMaxK];
#pragma unroll
      for (int u = 0; u < kMaxK; ++u) {
        const int k = k0 + u;
        const bool on = k < k_sum && topk_idx[(size_t)t * Kt + k] >= 0;
        wk[u] = on ? topk_w[(size_t)t * Kt + k] : 0.f;
        vals[u] = on ? ld_relaxed_sys_v4(src + (size_t)k * nvec + v) : make_int4(0, 0, 0, 0);
      }
#pragma unroll
      for (int u = 0; u < kMaxK; ++u) {
        const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&vals[u]);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const float2 f = __bfloat1622float2(p[i]);
          acc[2 * i] = fmaf(wk[u], f.x, acc[2 * i]);
          acc[2 * i + 1] = fmaf(wk[u], f.y, acc[2 * i + 1]);
        }
      }
    }
    int4 o;
    __nv_bfloat162* po = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
    for (int i = 0; i < 4; ++i) po[i] = __floats2bfloat162_rn(acc[2 * i], acc[2 * i + 1]);
    reinterpret_cast<int4*>(out + (size_t)t * H)[v] = o;
  }
}

}  // namespace umdk
