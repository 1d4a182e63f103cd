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
#include "ep_ll_dispatch.cuh"

namespace umdk {
namespace {

constexpr int kLLThreads = 512;
constexpr int kLLWarps = kLLThreads / 32;

struct LLDispatchArgs {
  EpLLGeom g;
  EpLLOffsets off;
  PeerTable peers;
  LLDispatchIO io;
};

__global__ void __launch_bounds__(kLLThreads, 1) ep_ll_dispatch_kernel(const LLDispatchArgs a) {
  extern __shared__ __align__(16) uint8_t ll_scratch[];
  ll_dispatch_body<kLLThreads>(a.g, a.off, a.peers, a.io, ll_scratch, nullptr);
}

// Low-latency combine as an operator of its own (the counterpart of the fused kernel's tail for callers that ran
// their own expert computation between low_latency_dispatch and low_latency_combine): every bf16 row of the slab goes
// back to its token's owner over NVLink into the owner's combine buffer (the slot comes from the row metadata the
// dispatch left beside the slab), completion flags go to every peer, and after all peers' flags have arrived the owner
// sums its rows with the routing weights. No host synchronisation: the row count is read from group_off on the
// device. Reference: cam_moe_distribute_combine.h:238-320 (status set / wait), :627-717 (weighted sum).
struct LLCombineArgs {
  EpLLGeom g;
  EpLLOffsets off;
  PeerTable peers;
  const __nv_bfloat16* y;     // [>= n, H] expert outputs in slab row order
  const int* group_off;       // [E_local + 1]; n = group_off[E_local]
  const int64_t* topk_idx;    // [T, K]
  const float* topk_w;        // [T, K]
  __nv_bfloat16* out;         // [T, H]
  int T;
  uint32_t* ctrl;             // [0] epoch (advanced here), [1] send-done, [2] reduce-done
  int* status;
  int phase_mask;             // bit0: send rows + flags; bit1: wait flags + weighted sum + epoch advance
};

__global__ void __launch_bounds__(kLLThreads, 1) ep_ll_combine_kernel(const LLCombineArgs a) {
  const EpLLGeom& g = a.g;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  __shared__ uint32_t s_epoch;
  __shared__ int s_ok;
  if (threadIdx.x == 0) {
    s_epoch = a.ctrl[0];
    s_ok = 1;
  }
  __syncthreads();
  const uint32_t epoch = s_epoch;
  const uint64_t tag = (uint64_t)epoch + 1;
  uint8_t* self = a.peers.base[g.rank];
  if (a.phase_mask & 1) {
    const int n = min(a.group_off[g.E_local], g.n_cap);
    const int* meta = reinterpret_cast<const int*>(self + a.off.slab_meta[0]);
    // one work item = 4 KiB of one row (32 lanes x 8 x 16 bytes): all loads of an item are in flight together
    const int nvec = g.H / 8;
    const int nparts = (nvec + 255) / 256;
    for (int item = blockIdx.x * kLLWarps + warp; item < n * nparts; item += gridDim.x * kLLWarps) {
      const int row = item / nparts, part = item - row * nparts;
      const int owner = meta[2 * row], slot = meta[2 * row + 1];
      if (owner < 0 || owner >= g.R || slot < 0 || slot >= g.T_cap * g.K) {
        if (lane == 0) umdk_set_status(a.status, UMDK_ERR_OVERFLOW, UMDK_PH_COMBINE_DATA, owner, slot);
        continue;
      }
      const int4* src = reinterpret_cast<const int4*>(a.y + (size_t)row * g.H);
      uint8_t* dst = a.peers.base[owner] + a.off.comb_buf[0] + (size_t)slot * g.H * 2;
      int4 v[8];
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        const int i = part * 256 + u * 32 + lane;
        v[u] = i < nvec ? __ldg(src + i) : make_int4(0, 0, 0, 0);
      }
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        const int i = part * 256 + u * 32 + lane;
        if (i < nvec) st_na_v4(dst + (size_t)i * 16, v[u]);
      }
    }
    if (cta_done_is_last(&a.ctrl[1], gridDim.x)) {
      // the call ends here for this rank's slab: its arrival words go back to zero before the flags that let the
      // peers start their next dispatch
      uint32_t* exp_cnt = reinterpret_cast<uint32_t*>(self + a.off.exp_cnt[0]);
      for (int i = threadIdx.x; i < g.E_local; i += blockDim.x) exp_cnt[i] = 0;
      __threadfence_system();
      __syncthreads();
      if (threadIdx.x < g.R) {
        st_release_sys(reinterpret_cast<uint64_t*>(a.peers.base[threadIdx.x] + a.off.comb_flag[0]) + g.rank, tag);
      }
    }
  }
  if (!(a.phase_mask & 2)) return;
  if (threadIdx.x < g.R) {
    const uint64_t* f = reinterpret_cast<const uint64_t*>(self + a.off.comb_flag[0]) + threadIdx.x;
    if (!wait_flag_ge_sys(f, tag)) {
      umdk_set_status(a.status, UMDK_ERR_TIMEOUT, UMDK_PH_COMBINE_DATA, threadIdx.x, (int)epoch);
      s_ok = 0;
    }
  }
  __syncthreads();
  if (s_ok) {
    ll_weighted_reduce<kLLThreads>(self + a.off.comb_buf[0], a.topk_idx, a.topk_w, a.out, nullptr, a.T, g.K, g.H);
  }
  if (cta_done_is_last(&a.ctrl[2], gridDim.x)) {
    if (threadIdx.x == 0) a.ctrl[0] = epoch + 1;
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


struct UmdkEpLLLayout {
  uint64_t cnt, cnt_flag, data_flag, comb_flag, slab_x, slab_s, slab_meta, comb_buf, total;
  int n_cap;
  uint64_t exp_cnt;   // arrival words per local expert
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
  out->exp_cnt = o.exp_cnt[0];
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
  a.io.x = static_cast<const __nv_bfloat16*>(p->x);
  a.io.topk_idx = p->topk_idx;
  a.io.send_idx = p->send_idx;
  a.io.num_per_expert = p->num_per_expert;
  a.io.T = p->T;
  a.io.group_off = p->group_off;
  a.io.recv_per_expert = p->recv_per_expert;
  a.io.ctrl = p->ctrl;
  a.io.status = p->status;
  a.io.meet_cycles = umdk_rendezvous_cycles();
  a.io.phase_mask = p->phase_mask ? p->phase_mask : 3;
  int grid = p->num_ctas > 0 ? p->num_ctas : 32;
  if (grid > sm_count()) grid = sm_count();
  if (!p->send_idx) {
    // layout inside the kernel: 16-bit counters and positions, so at most 65535 entries per expert and a table that
    // fits in shared memory
    if (p->num_per_expert || p->T > 2048 || p->E > 1024) return -UMDK_ERR_BAD_ARG;
  } else if (!p->num_per_expert) {
    return -UMDK_ERR_BAD_ARG;
  }
  const size_t dyn = ll_dispatch_smem_bytes(p->T, p->E, p->K, kLLWarps, p->send_idx == nullptr);
  if (dyn > 200 * 1024) return -UMDK_ERR_BAD_ARG;
  if (dyn > 40 * 1024) {
    UMDK_CUDA_CHECK(cudaFuncSetAttribute(ep_ll_dispatch_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)dyn));
  }
  ep_ll_dispatch_kernel<<<grid, kLLThreads, dyn, static_cast<cudaStream_t>(stream)>>>(a);
  UMDK_CUDA_CHECK(cudaGetLastError());
  return 0;
}

struct UmdkEpLLCombineParams {
  int R, rank, E, K, H, T_cap, T, num_ctas, phase_mask;
  void* peers[kMaxRanks];
  const void* y;
  const int* group_off;
  const int64_t* topk_idx;
  const float* topk_w;
  void* out;
  uint32_t* ctrl;
  int* status;
};

UMDK_API int umdk_ep_ll_combine(const UmdkEpLLCombineParams* p, void* stream) {
  LLCombineArgs a;
  if (int rc = fill_ll_geom(&a.g, p->R, p->rank, p->E, p->K, p->H, p->T_cap)) return rc;
  if (p->T > p->T_cap || p->T < 0) return -UMDK_ERR_BAD_ARG;
  a.off = ep_ll_offsets(a.g);
  for (int i = 0; i < kMaxRanks; ++i) a.peers.base[i] = i < p->R ? static_cast<uint8_t*>(p->peers[i]) : nullptr;
  a.y = static_cast<const __nv_bfloat16*>(p->y);
  a.group_off = p->group_off;
  a.topk_idx = p->topk_idx;
  a.topk_w = p->topk_w;
  a.out = static_cast<__nv_bfloat16*>(p->out);
  a.T = p->T;
  a.ctrl = p->ctrl;
  a.status = p->status;
  a.phase_mask = p->phase_mask ? p->phase_mask : 3;
  int grid = p->num_ctas > 0 ? p->num_ctas : 64;
  if (grid > sm_count()) grid = sm_count();
  ep_ll_combine_kernel<<<grid, kLLThreads, 0, static_cast<cudaStream_t>(stream)>>>(a);
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
