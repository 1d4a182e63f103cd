// Low-latency (decode) expert-parallel dispatch: per-expert counts are all-gathered through peer memory, then every
// (token, k) is quantised to fp8 e4m3 (fp32 scale per 1x128 block) and stored straight into its final row of the
// destination rank's expert-major slab, which the grouped GEMM reads with TMA without any repacking.
//
// The reference's decode path pushes int8 tokens into fixed [srcRank][localExpert] window slots and compacts them
// on the receiver before the GEMM (src/cam/comm_operator/ascend_kernels/fused_deep_moe/op_kernel/fused_deep_moe/
// raw_distributed/cam_moe_distribute_dispatch.h:433-488 SendToMoeExpert, :781-861 LocalWindowCopy). Here the counts
// travel first (one small NVLink round), so senders know the exact destination rows and the compaction pass
// disappears; rows of one expert are ordered by source rank, then by (token, k) - the same order as the reference's
// compacted expandX (status index = localExpert * R + srcRank, :625-633).
#include "ep_common.cuh"
#include "ptx.cuh"
#include "sync.cuh"

namespace umdk {
namespace {

constexpr int kLLThreads = 512;
constexpr int kLLWarps = kLLThreads / 32;

struct LLDispatchArgs {
  EpLLGeom g;
  EpLLOffsets off;
  PeerTable peers;
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

__global__ void __launch_bounds__(kLLThreads, 1) ep_ll_dispatch_kernel(const LLDispatchArgs a) {
  const EpLLGeom& g = a.g;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  __shared__ uint32_t s_epoch;
  __shared__ int s_ok;
  __shared__ int s_base[1024];                        // destination row base of my tokens, per global expert
  __shared__ uint8_t* s_dx[kLLWarps][kMaxTopk];
  __shared__ float* s_ds[kLLWarps][kMaxTopk];
  if (threadIdx.x == 0) {
    s_epoch = a.ctrl[0];
    s_ok = 1;
  }
  // ---- layout inside the kernel (decode-sized inputs) ----
  // Every CTA computes, for all T x K entries, the position of the entry inside its expert's bucket (token-major
  // order) and the bucket sizes: per 32-token chunk a warp walks its tokens in order with shared-memory counters,
  // then the chunks are scanned per expert. A few microseconds of redundant work per CTA instead of a kernel launch
  // and a pass through global memory.
  extern __shared__ __align__(16) uint8_t ll_dyn[];
  const bool own_layout = a.send_idx == nullptr;
  const int n_chunks = (a.T + 31) / 32;
  uint16_t* s_hist = reinterpret_cast<uint16_t*>(ll_dyn);              // [n_chunks][E] counts, then exclusive bases
  uint16_t* s_sidx = s_hist + (size_t)n_chunks * g.E;                  // [T * K] positions
  int16_t* s_eid = reinterpret_cast<int16_t*>(s_sidx + (size_t)a.T * g.K);   // [T * K] expert ids (-1 = none)
  __shared__ int s_npe[1024];
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
  uint8_t* self = a.peers.base[g.rank];

  if ((a.phase_mask & 1) && blockIdx.x == 0) {
    for (int d = warp; d < g.R; d += kLLWarps) {
      int* dst = reinterpret_cast<int*>(a.peers.base[d] + a.off.cnt[0]) + (size_t)g.rank * g.E;
      for (int i = lane; i < g.E; i += 32) dst[i] = own_layout ? s_npe[i] : a.num_per_expert[i];
      __threadfence_system();
      __syncwarp();
      if (lane == 0) st_release_sys(reinterpret_cast<uint64_t*>(a.peers.base[d] + a.off.cnt_flag[0]) + g.rank, tag);
    }
  }
  if (!(a.phase_mask & 2)) return;

  if (threadIdx.x < g.R) {
    const uint64_t* f = reinterpret_cast<const uint64_t*>(self + a.off.cnt_flag[0]) + threadIdx.x;
    if (!wait_flag_ge_sys(f, tag)) {
      umdk_set_status(a.status, UMDK_ERR_TIMEOUT, UMDK_PH_DISPATCH_COUNT, threadIdx.x, (int)epoch);
      s_ok = 0;
    }
  }
  __syncthreads();
  if (!s_ok) return;
  const int* cnt = reinterpret_cast<const int*>(self + a.off.cnt[0]);  // [src][E]
  // per-expert totals over sources, then exclusive prefix inside each destination rank
  __shared__ int s_tot[1024];
  // totals over sources and the part that comes from lower-numbered sources (my rows start after theirs); the
  // loads of eight sources are issued together
  __shared__ int s_before[1024];
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
      if (d == g.rank && blockIdx.x == 0) {
        a.group_off[le] = s_base[e];
        a.recv_per_expert[le] = (int64_t)s_tot[e];
        if (le == g.E_local - 1) {
          a.group_off[g.E_local] = run;
          if (run > g.n_cap) umdk_set_status(a.status, UMDK_ERR_OVERFLOW, UMDK_PH_DISPATCH_COUNT, run, g.n_cap);
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
          dx = a.peers.base[d] + a.off.slab_x[0] + (size_t)row * g.H;
          ds = reinterpret_cast<float*>(a.peers.base[d] + a.off.slab_s[0]) + (size_t)row * nblk;
          if (part == 0) {
            int* meta = reinterpret_cast<int*>(a.peers.base[d] + a.off.slab_meta[0]) + (size_t)row * 2;
            meta[0] = g.rank;
            meta[1] = t * g.K + lane;
          }
        }
      }
      s_dx[warp][lane] = dx;
      s_ds[warp][lane] = ds;
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
          uint8_t* dx = s_dx[warp][k];
          if (dx == nullptr) continue;
          st_na_v4(dx + blk * 128 + (lane & 7) * 16, q);
          if ((lane & 7) == 0) s_ds[warp][k][blk] = scale;
        }
      }
    }
  }
  if (cta_done_is_last(&a.ctrl[3], gridDim.x)) {
    if (threadIdx.x < g.R) {
      st_release_sys(reinterpret_cast<uint64_t*>(a.peers.base[threadIdx.x] + a.off.data_flag[0]) + g.rank, tag);
    }
  }
}

// Stand-alone fp8 e4m3 1x128 quantisation of local rows (shared expert input, tests).
__global__ void __launch_bounds__(256) quant_fp8_kernel(const __nv_bfloat16* __restrict__ x, int T, int H,
                                                        uint8_t* __restrict__ q, float* __restrict__ s) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nblk = H / 128;
  for (int t = blockIdx.x * 8 + warp; t < T; t += gridDim.x * 8) {
    const int4* xrow = reinterpret_cast<const int4*>(x + (size_t)t * H);
    for (int b0 = 0; b0 < nblk; b0 += 4) {
      const int blk = b0 + (lane >> 3);
      const bool active = blk < nblk;
      float f[16];
      if (active) {
        bf16x8_to_float(__ldg(xrow + blk * 16 + (lane & 7) * 2), f);
        bf16x8_to_float(__ldg(xrow + blk * 16 + (lane & 7) * 2 + 1), f + 8);
      } else {
#pragma unroll
        for (int i = 0; i < 16; ++i) f[i] = 0.f;
      }
      float scale;
      const int4 v = quant16(f, &scale);
      if (active) {
        *reinterpret_cast<int4*>(q + (size_t)t * H + blk * 128 + (lane & 7) * 16) = v;
        if ((lane & 7) == 0) s[(size_t)t * nblk + blk] = scale;
      }
    }
  }
}

}  // namespace
}  // namespace umdk

using namespace umdk;

static int fill_ll_geom(EpLLGeom* g, int R, int rank, int E, int K, int H, int T_cap) {
  if (R < 1 || R > kMaxRanks || rank < 0 || rank >= R || E < R || (E % R) || E > 1024 || K < 1 || K > kMaxTopk ||
      H < 128 || (H % 128) || T_cap < 1)
    return -UMDK_ERR_BAD_ARG;
  g->R = R;
  g->rank = rank;
  g->E = E;
  g->E_local = E / R;
  g->K = K;
  g->H = H;
  g->T_cap = T_cap;
  g->n_cap = ep_ll_n_cap(R, T_cap, K, E / R);
  return 0;
}

struct UmdkEpLLLayout {
  uint64_t cnt, cnt_flag, data_flag, comb_flag, slab_x, slab_s, slab_meta, comb_buf, total;
  int n_cap;
};

// Offsets of the low-latency regions inside each rank's symmetric heap, and the heap size needed.
UMDK_API int umdk_ep_ll_layout(int R, int E, int K, int H, int T_cap, UmdkEpLLLayout* out) {
  EpLLGeom g;
  if (int rc = fill_ll_geom(&g, R, 0, E, K, H, T_cap)) return rc;
  const EpLLOffsets o = ep_ll_offsets(g);
  out->cnt = o.cnt[0];
  out->cnt_flag = o.cnt_flag[0];
  out->data_flag = o.data_flag[0];
  out->comb_flag = o.comb_flag[0];
  out->slab_x = o.slab_x[0];
  out->slab_s = o.slab_s[0];
  out->slab_meta = o.slab_meta[0];
  out->comb_buf = o.comb_buf[0];
  out->total = o.total;
  out->n_cap = g.n_cap;
  return 0;
}

struct UmdkEpLLDispatchParams {
  int R, rank, E, K, H, T_cap, T, num_ctas, phase_mask;
  void* peers[kMaxRanks];
  const void* x;
  const int64_t* topk_idx;
  const int* send_idx;
  const int* num_per_expert;
  int* group_off;
  int64_t* recv_per_expert;
  uint32_t* ctrl;
  int* status;
};

UMDK_API int umdk_ep_ll_dispatch(const UmdkEpLLDispatchParams* p, void* stream) {
  LLDispatchArgs a;
  if (int rc = fill_ll_geom(&a.g, p->R, p->rank, p->E, p->K, p->H, p->T_cap)) return rc;
  if (p->T > p->T_cap) return -UMDK_ERR_BAD_ARG;
  a.off = ep_ll_offsets(a.g);
  for (int i = 0; i < kMaxRanks; ++i) a.peers.base[i] = i < p->R ? static_cast<uint8_t*>(p->peers[i]) : nullptr;
  a.x = static_cast<const __nv_bfloat16*>(p->x);
  a.topk_idx = p->topk_idx;
  a.send_idx = p->send_idx;
  a.num_per_expert = p->num_per_expert;
  a.T = p->T;
  a.group_off = p->group_off;
  a.recv_per_expert = p->recv_per_expert;
  a.ctrl = p->ctrl;
  a.status = p->status;
  a.phase_mask = p->phase_mask ? p->phase_mask : 3;
  int grid = p->num_ctas > 0 ? p->num_ctas : 32;
  if (grid > sm_count()) grid = sm_count();
  size_t dyn = 0;
  if (!p->send_idx) {
    // layout inside the kernel: 16-bit counters and positions, so at most 65535 entries per expert and a table that
    // fits in shared memory
    if (p->num_per_expert || p->T > 2048 || p->E > 1024) return -UMDK_ERR_BAD_ARG;
    dyn = sizeof(uint16_t) * ((size_t)((p->T + 31) / 32) * p->E + 2 * (size_t)p->T * p->K);
    if (dyn > 160 * 1024) return -UMDK_ERR_BAD_ARG;
    if (dyn > 16 * 1024) {
      UMDK_CUDA_CHECK(cudaFuncSetAttribute(ep_ll_dispatch_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)dyn));
    }
  } else if (!p->num_per_expert) {
    return -UMDK_ERR_BAD_ARG;
  }
  ep_ll_dispatch_kernel<<<grid, kLLThreads, dyn, static_cast<cudaStream_t>(stream)>>>(a);
  UMDK_CUDA_CHECK(cudaGetLastError());
  return 0;
}

UMDK_API int umdk_quant_fp8_1x128(const void* x, int T, int H, void* q, float* s, void* stream) {
  if (T < 0 || H < 128 || (H % 128)) return -UMDK_ERR_BAD_ARG;
  if (T == 0) return 0;
  int grid = (T + 7) / 8;
  if (grid > 4 * sm_count()) grid = 4 * sm_count();
  quant_fp8_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(static_cast<const __nv_bfloat16*>(x), T, H,
                                                                      static_cast<uint8_t*>(q), s);
  UMDK_CUDA_CHECK(cudaGetLastError());
  return 0;
}
