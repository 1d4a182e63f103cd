// One persistent kernel for the whole low-latency MoE layer: dispatch, expert FFN and combine in ONE launch.
//
//   dispatch (optional prologue, ep_ll_dispatch.cuh) every CTA derives the routing layout in shared memory, the
//          per-expert counts are all-gathered through peer memory, and all warps of the grid quantise this rank's
//          tokens to fp8 1x128 and store them into their final slab rows on the destination ranks over NVLink;
//          TMEM allocation, barrier set-up and descriptor prefetch of the GEMM pipeline are already done by then
//   gate   wait (bounded) until the dispatched fp8 rows of every source rank have landed in this rank's slab
//   phase 1  grouped gate/up GEMM (tcgen05, fp8 e4m3, TMEM) + block-scale promotion + SwiGLU + fp8 1x128 re-quant
//   phase 2  grouped down GEMM whose epilogue stores each bf16 row straight into the token owner's combine buffer
//            over NVLink; a phase-2 tile starts as soon as the phase-1 tiles of ITS token tile are done (per-tile
//            counters), so the small phase-2 tiles fill the tail of the last phase-1 wave instead of a second launch
//   tail   completion flags to every peer, bounded wait for all peers, top-k weighted reduction of this rank's tokens
//
// Work split: phase-1 items are dealt round-robin; phase-2 items (about 1/7 of the cost each) are dealt in
// contiguous ranges sized so that every CTA ends at the same time, the CTAs with fewer phase-1 items taking the
// earliest (first ready) phase-2 items. Roles per CTA as in moe_gemm.cu: TMA producer warp, single-thread MMA issuer,
// TMEM allocator warp, eight promotion/epilogue warps (two per scheduler, so one hides the other's TMEM-load latency). Same math and operand formats as moe_gemm.cu modes 0 and 2.
// Reference counterpart: the fused_deep_moe operator (src/cam/comm_operator/ascend_kernels/fused_deep_moe/op_kernel/
// fused_deep_moe.h:354-448), whose cube cores likewise wait per expert group for arrived tokens
// (gemm/kernel/grouped_matmul_slice_m_per_token_dequant_swiglu_quant_multistage_workspace.h:271-280) - there with an
// unbounded spin, here with a cycle budget and a status record.
#include "ep_ll_dispatch.cuh"

namespace umdk {
namespace {

constexpr int TT = 64;
constexpr int BMW = 128;
constexpr int BKB = 128;
constexpr int kThreads = 384;      // TMA, MMA, TMEM-allocator and one spare warp + 8 promotion / epilogue warps
constexpr int kEpiThreads = 256;
constexpr int kTransStride = 129;
constexpr int kRingBytes = 4 * (2 * BMW * BKB + TT * BKB);  // 160 KB: 4 x 40 KB (phase 1) or 6 x 24 KB (phase 2)
constexpr int kTmemCols = 256;

struct FusedArgs {
  int G, F, H;             // local experts, FFN width, hidden size
  int n_rows_cap;
  const int* group_off;    // [G + 1]
  const float* xs;         // [n_rows_cap, H/128] scales of the dispatched rows
  const float* w1s;        // [G, 2F/128, H/128]
  const float* w2s;        // [G, H/128, F/128]
  uint8_t* hq;             // [n_rows_cap, F] intermediate (fp8)
  float* hs;               // [n_rows_cap, F/128]
  uint32_t* tile_done;     // [>= n_rows_cap/64 + G] zero between calls (reset by this kernel)
  const uint64_t* wait_flags;
  uint32_t* exp_cnt;       // [G] arrival words of this rank's experts (row parts landed in the running call)
  int exp_parts;           // parts per row (ep_ll_row_parts)
  int exp_gate;            // 1: a phase-1 item waits for ITS expert's rows only; 0: the whole slab is awaited first
  int wait_n;
  PeerTable peers;
  int R, rank;
  uint64_t comb_buf_off, comb_flag_off;
  const int* row_meta;     // [n_rows_cap][2] owner rank, owner slot
  const int64_t* topk_idx;
  const float* topk_w;
  __nv_bfloat16* out;
  __nv_bfloat16* share_out;  // optional [T, H]: the row of the LAST top-k slot goes here unweighted instead of into `out`
  int T, Kt, T_cap;
  uint32_t* ctrl;          // [0] epoch (advanced here), [1] send-done, [2] reduce-done
  int w_tiled;             // weights are stored tile by tile (see umdk_moe_fused)
  int phase_mask;          // bit0: gate + both GEMM phases + combine-send + flags; bit1: wait + reduce + epoch advance;
                           // bit2: dispatch prologue, publish counts; bit3: dispatch prologue, push rows + data flags
  int fuse_dispatch;       // the dispatch runs inside this kernel (disp / ll_geom / ll_off are valid)
  EpLLGeom ll_geom;
  EpLLOffsets ll_off;
  LLDispatchIO disp;
  int* status;
  // optional [6] global-timer stamps (ns): [0] earliest CTA start, then the latest CTA to pass: [1] the wait for the
  // dispatched rows, [2] phase 1, [3] phase 2, [4] the wait for the peers' combine flags, [5] the end of the kernel
  unsigned long long* diag;
};

template <int PH>
struct P {
  static constexpr int kATiles = PH == 1 ? 2 : 1;
  static constexpr int kABytes = kATiles * BMW * BKB;
  static constexpr int kStageBytes = kABytes + TT * BKB;
  static constexpr int kStages = PH == 1 ? 4 : 6;
  static constexpr int kTmemStageCols = kATiles * TT;
};

struct Shared {
  float* trans;
  float* xs_sm;
  float* ws_sm;
  float* amax_sm;
  int* tile_pref;
  int* goff;
  int* epi_flag;
  int* meta_sm;    // [TT][2] owner rank and slot of the rows of the current token tile (phase 2)
  uint64_t* bars;  // per phase: full[6], empty[6], tfull[2], tempty[2] = 16 barriers
  uint8_t* ring;
};

__device__ __forceinline__ void bar_epi() { asm volatile("bar.sync 1, 256;" ::: "memory"); }
__device__ __forceinline__ uint32_t pack_fp8x4(float a, float b, float c, float d) {
  const __nv_fp8x2_storage_t lo = __nv_cvt_float2_to_fp8x2(make_float2(a, b), __NV_SATFINITE, __NV_E4M3);
  const __nv_fp8x2_storage_t hi = __nv_cvt_float2_to_fp8x2(make_float2(c, d), __NV_SATFINITE, __NV_E4M3);
  return (uint32_t)lo | ((uint32_t)hi << 16);
}
__device__ __forceinline__ void locate_tile(const int* tile_pref, const int* goff, int G, int tile, int* e, int* row0,
                                            int* m) {
  int lo = 0, hi = G;
  while (hi - lo > 1) {
    const int mid = (lo + hi) >> 1;
    if (tile_pref[mid] <= tile) lo = mid;
    else hi = mid;
  }
  *e = lo;
  *row0 = goff[lo] + (tile - tile_pref[lo]) * TT;
  *m = min(TT, goff[lo + 1] - *row0);
}

// One phase of the pipeline for the items first, first + step, ... < last of this CTA.
template <int PH>
__device__ __forceinline__ void run_phase(const CUtensorMap* tmW, const CUtensorMap* tmX, const FusedArgs& a,
                                          const Shared& sh, uint32_t tmem_base, int first, int last, int step) {
  using C = P<PH>;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int K = PH == 1 ? a.H : a.F;
  const int Nout = PH == 1 ? a.F : a.H;
  const int w_rows = PH == 1 ? 2 * a.F : a.H;
  const int NT = Nout / BMW;
  const int kb_total = K / BKB;
  uint64_t* full = sh.bars + (PH - 1) * 16;
  uint64_t* empty = full + 6;
  uint64_t* tfull = full + 12;
  uint64_t* tempty = full + 14;
  const int NT1 = a.F / BMW;

  if (warp == 0) {
    if (elect_one()) {
      const uint64_t pol_w = policy_evict_first();
      const uint64_t pol_x = policy_evict_last();
      int s = 0;
      uint32_t ph = 0;
      bool ok = true;
      int ready_tile = -1, ready_e = -1;
      for (int w = first; w < last && ok; w += step) {
        int e, row0, m;
        const int tile = w / NT;
        locate_tile(sh.tile_pref, sh.goff, a.G, tile, &e, &row0, &m);
        const int j = w % NT;
        if (PH == 1 && a.exp_gate && e != ready_e) {
          // per-expert gate: this expert's rows (all parts of all its rows, from every source) have landed; other
          // experts' rows may still be in flight while this item computes
          const uint32_t need = (uint32_t)(sh.goff[e + 1] - sh.goff[e]) * (uint32_t)a.exp_parts;
          if (!wait_flag_ge_sys(a.exp_cnt + e, need)) {
            umdk_set_status(a.status, UMDK_ERR_TIMEOUT, UMDK_PH_GROUP_READY, e, (int)need);
            break;
          }
          ready_e = e;
          fence_proxy_async_all();   // the rows were written with ordinary stores and are read by TMA
        }
        if (PH == 2 && tile != ready_tile) {
          // the intermediate rows of this token tile are complete when all its phase-1 items have finished
          if (!wait_flag_ge_gpu(&a.tile_done[tile], (uint32_t)NT1)) {
            umdk_set_status(a.status, UMDK_ERR_TIMEOUT, UMDK_PH_GROUP_READY, tile, w);
            break;
          }
          ready_tile = tile;
          fence_proxy_async_all();
        }
        for (int kb = 0; kb < kb_total; ++kb) {
          if (!mbar_wait(&empty[s], ph ^ 1)) {
            umdk_set_status(a.status, UMDK_ERR_TIMEOUT, UMDK_PH_TMA_EMPTY, w, kb);
            ok = false;
            break;
          }
          mbar_expect_tx(&full[s], C::kStageBytes);
          uint8_t* st = sh.ring + s * C::kStageBytes;
          if (a.w_tiled) {
            // one contiguous chunk per k-block: 128 x 128 B (phase 2) or gate + up = 256 x 128 B (phase 1)
            tma_load_2d_hint(st, tmW, &full[s], 0, ((e * NT + j) * kb_total + kb) * (C::kATiles * BMW), pol_w);
          } else {
            tma_load_2d_hint(st, tmW, &full[s], kb * BKB, e * w_rows + j * BMW, pol_w);
            if (PH == 1) tma_load_2d_hint(st + BMW * BKB, tmW, &full[s], kb * BKB, e * w_rows + a.F + j * BMW, pol_w);
          }
          tma_load_2d_hint(st + C::kABytes, tmX, &full[s], kb * BKB, row0, pol_x);
          if (++s == C::kStages) {
            s = 0;
            ph ^= 1;
          }
        }
      }
    }
  } else if (warp == 1) {
    if (elect_one()) {
      constexpr uint32_t idesc = umma_idesc(kFmtE4M3, kFmtE4M3, BMW, TT);
      int s = 0;
      uint32_t ph = 0, kbc = 0;
      bool ok = true;
      for (int w = first; w < last && ok; w += step) {
        for (int kb = 0; kb < kb_total; ++kb, ++kbc) {
          const int ts = kbc & 1;
          const uint32_t tph = (kbc >> 1) & 1;
          if (!mbar_wait(&tempty[ts], tph ^ 1)) {
            umdk_set_status(a.status, UMDK_ERR_TIMEOUT, UMDK_PH_TMEM_EMPTY, w, kb);
            ok = false;
            break;
          }
          if (!mbar_wait(&full[s], ph)) {
            umdk_set_status(a.status, UMDK_ERR_TIMEOUT, UMDK_PH_TMA_FULL, w, kb);
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t sa = smem_u32(sh.ring + s * C::kStageBytes);
          const uint64_t adesc = umma_desc_k_sw128(sa);
          const uint64_t adesc_u = umma_desc_k_sw128(sa + BMW * BKB);
          const uint64_t bdesc = umma_desc_k_sw128(sa + C::kABytes);
          const uint32_t d = tmem_base + ts * C::kTmemStageCols;
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            umma_f8(d, adesc + 2 * k, bdesc + 2 * k, idesc, k > 0 ? 1u : 0u);
            if (PH == 1) umma_f8(d + TT, adesc_u + 2 * k, bdesc + 2 * k, idesc, k > 0 ? 1u : 0u);
          }
          umma_commit(&empty[s]);
          umma_commit(&tfull[ts]);
          if (++s == C::kStages) {
            s = 0;
            ph ^= 1;
          }
        }
      }
    }
  } else if (warp >= 4) {
    // Eight promotion / epilogue warps. TMEM lane = weight row of the tile; a warp may only touch the 32 lanes
    // selected by (warp index mod 4), so warps 4..7 and 8..11 cover the same rows and split the 64 token columns.
    const int ew = warp - 4;
    const int q = warp & 3, hh = ew >> 2;
    const int tid = ew * 32 + lane;         // 0..255 inside the epilogue group
    const int wrow = q * 32 + lane;         // weight row of this thread inside the 128-row tile
    constexpr int HC = TT / 2;              // token columns per thread
    const int nsb = K / 128;
    const int wsb = w_rows / 128;
    const float* xs = PH == 1 ? a.xs : a.hs;
    const float* ws = PH == 1 ? a.w1s : a.w2s;
    uint32_t kbc = 0;
    bool ok = true;
    int ready_tile = -1, loaded_tile = -1;
    float ws_next = 0.f;
    bool have_ws_next = false;
    for (int w = first; w < last && ok; w += step) {
      int e, row0, m;
      const int tile = w / NT;
      locate_tile(sh.tile_pref, sh.goff, a.G, tile, &e, &row0, &m);
      const int j = w % NT;
      if (PH == 2 && tile != ready_tile) {
        // the scales of the intermediate rows are read with plain loads below: order them after the phase-1 writers
        if (tid == 0) *sh.epi_flag = wait_flag_ge_gpu(&a.tile_done[tile], (uint32_t)NT1) ? 1 : 0;
        bar_epi();
        if (!*sh.epi_flag) break;  // the producer records the timeout
        ready_tile = tile;
      }
      if (PH == 1 || tile != loaded_tile) {
        // activation scales (and, in phase 2, the owner / slot of every row) depend on the token tile only; a CTA's
        // phase-2 items walk the weight tiles of one token tile back to back, so they are fetched once per tile
        for (int i = tid; i < TT * kb_total; i += kEpiThreads) {
          const int t = i / kb_total, kb = i - t * kb_total;
          // phase 2 reads scales written by other SMs during this launch: bypass L1
          sh.xs_sm[kb * TT + t] = t < m ? __ldcg(xs + (size_t)(row0 + t) * nsb + kb) : 0.f;
        }
        if (PH == 2 && tid < 2 * TT) sh.meta_sm[tid] = (tid >> 1) < m ? a.row_meta[2 * row0 + tid] : -1;
        loaded_tile = tile;
      }
      if (!have_ws_next) {
        for (int i = tid; i < C::kATiles * kb_total; i += kEpiThreads) {
          const int which = i / kb_total, kb = i - which * kb_total;
          const int brow = which == 0 ? j : (a.F / 128 + j);
          sh.ws_sm[which * kb_total + kb] = ws[((size_t)e * wsb + brow) * nsb + kb];
        }
      } else if (tid < C::kATiles * kb_total) {
        sh.ws_sm[tid] = ws_next;   // fetched while the previous item was in its k-loop
      }
      have_ws_next = false;
      if (w + step < last && C::kATiles * kb_total <= kEpiThreads) {
        // weight scales of the NEXT item: the load is in flight during this item's k-loop
        int e2, r2, m2;
        const int w2 = w + step;
        locate_tile(sh.tile_pref, sh.goff, a.G, w2 / NT, &e2, &r2, &m2);
        if (tid < C::kATiles * kb_total) {
          const int which = tid / kb_total, kb = tid - which * kb_total;
          const int brow = which == 0 ? (w2 % NT) : (a.F / 128 + (w2 % NT));
          ws_next = ws[((size_t)e2 * wsb + brow) * nsb + kb];
        }
        have_ws_next = true;
      }
      bar_epi();
      float acc_g[HC];
      float acc_u[PH == 1 ? HC : 1];
#pragma unroll
      for (int c = 0; c < HC; ++c) acc_g[c] = 0.f;
      if (PH == 1) {
#pragma unroll
        for (int c = 0; c < HC; ++c) acc_u[c] = 0.f;
      }
      for (int kb = 0; kb < kb_total; ++kb, ++kbc) {
        const int ts = kbc & 1;
        const uint32_t tph = (kbc >> 1) & 1;
        if (!mbar_wait(&tfull[ts], tph)) {
          umdk_set_status(a.status, UMDK_ERR_TIMEOUT, UMDK_PH_TMEM_FULL, w, kb);
          ok = false;
          break;
        }
        tc_fence_after();
        const uint32_t taddr = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + ts * C::kTmemStageCols + hh * HC;
        uint32_t rg[HC];
        uint32_t ru[PH == 1 ? HC : 1];
        tmem_ld_x32(taddr, rg);
        if constexpr (PH == 1) tmem_ld_x32(taddr + TT, ru);
        const float wg = sh.ws_sm[kb];
        const float wu = PH == 1 ? sh.ws_sm[kb_total + kb] : 0.f;
        const float4* xsk = reinterpret_cast<const float4*>(sh.xs_sm + kb * TT + hh * HC);
        tmem_ld_wait();
        // the accumulator stage is free as soon as its values are in registers
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&tempty[ts]);
#pragma unroll
        for (int c4 = 0; c4 < HC / 4; ++c4) {
          const float4 x4 = xsk[c4];
          acc_g[4 * c4 + 0] = fmaf(__uint_as_float(rg[4 * c4 + 0]), x4.x * wg, acc_g[4 * c4 + 0]);
          acc_g[4 * c4 + 1] = fmaf(__uint_as_float(rg[4 * c4 + 1]), x4.y * wg, acc_g[4 * c4 + 1]);
          acc_g[4 * c4 + 2] = fmaf(__uint_as_float(rg[4 * c4 + 2]), x4.z * wg, acc_g[4 * c4 + 2]);
          acc_g[4 * c4 + 3] = fmaf(__uint_as_float(rg[4 * c4 + 3]), x4.w * wg, acc_g[4 * c4 + 3]);
          if constexpr (PH == 1) {
            acc_u[4 * c4 + 0] = fmaf(__uint_as_float(ru[4 * c4 + 0]), x4.x * wu, acc_u[4 * c4 + 0]);
            acc_u[4 * c4 + 1] = fmaf(__uint_as_float(ru[4 * c4 + 1]), x4.y * wu, acc_u[4 * c4 + 1]);
            acc_u[4 * c4 + 2] = fmaf(__uint_as_float(ru[4 * c4 + 2]), x4.z * wu, acc_u[4 * c4 + 2]);
            acc_u[4 * c4 + 3] = fmaf(__uint_as_float(ru[4 * c4 + 3]), x4.w * wu, acc_u[4 * c4 + 3]);
          }
        }
      }
      if (!ok) break;
      // transpose through shared memory: trans[token][weight row]
#pragma unroll
      for (int c = 0; c < HC; ++c) {
        float v = acc_g[c];
        if constexpr (PH == 1) v = (v / (1.f + __expf(-v))) * acc_u[c];
        sh.trans[(hh * HC + c) * kTransStride + wrow] = v;
      }
      bar_epi();
      const int t = tid & 63, qtr = tid >> 6;     // token, 32-column quarter of the 128 output columns
      const float* src = sh.trans + t * kTransStride + qtr * 32;
      const int row = row0 + t;
      if (PH == 1) {
        float amax = 0.f;
#pragma unroll 8
        for (int i = 0; i < 32; ++i) amax = fmaxf(amax, fabsf(src[i]));
        sh.amax_sm[tid] = amax;
        bar_epi();
        amax = fmaxf(fmaxf(fmaxf(sh.amax_sm[t], sh.amax_sm[t + 64]), fmaxf(sh.amax_sm[t + 128], sh.amax_sm[t + 192])),
                     1e-4f);
        const float inv = 448.f / amax;
        if (t < m) {
          uint8_t* dst = a.hq + (size_t)row * a.F + j * BMW + qtr * 32;
#pragma unroll
          for (int qq = 0; qq < 2; ++qq) {
            int4 o;
            const float* s4 = src + qq * 16;
            o.x = pack_fp8x4(s4[0] * inv, s4[1] * inv, s4[2] * inv, s4[3] * inv);
            o.y = pack_fp8x4(s4[4] * inv, s4[5] * inv, s4[6] * inv, s4[7] * inv);
            o.z = pack_fp8x4(s4[8] * inv, s4[9] * inv, s4[10] * inv, s4[11] * inv);
            o.w = pack_fp8x4(s4[12] * inv, s4[13] * inv, s4[14] * inv, s4[15] * inv);
            reinterpret_cast<int4*>(dst)[qq] = o;
          }
          if (qtr == 0) a.hs[(size_t)row * (a.F / 128) + j] = amax * (1.f / 448.f);
        }
        // publish: the rows of this item are in global memory -> one more phase-1 item of this token tile is done
        __threadfence();
        bar_epi();
        if (tid == 0) red_add_release_gpu(&a.tile_done[tile], 1u);
      } else {
        if (t < m) {
          const int owner = sh.meta_sm[2 * t], slot = sh.meta_sm[2 * t + 1];
          if (owner < 0 || owner >= a.R || slot < 0 || slot >= a.T_cap * a.Kt) {
            umdk_set_status(a.status, UMDK_ERR_OVERFLOW, UMDK_PH_COMBINE_DATA, owner, slot);
          } else {
            uint8_t* dst = a.peers.base[owner] + a.comb_buf_off + ((size_t)slot * a.H + j * BMW + qtr * 32) * 2;
#pragma unroll
            for (int qq = 0; qq < 4; ++qq) {
              int4 o;
              __nv_bfloat162* po = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
              for (int i = 0; i < 4; ++i) po[i] = __floats2bfloat162_rn(src[qq * 8 + 2 * i], src[qq * 8 + 2 * i + 1]);
              st_na_v4(dst + qq * 16, o);
            }
          }
        }
        bar_epi();
      }
    }
  }
}

__global__ void __launch_bounds__(kThreads, 1)
moe_fused_kernel(const __grid_constant__ CUtensorMap tmW1, const __grid_constant__ CUtensorMap tmX,
                 const __grid_constant__ CUtensorMap tmW2, const __grid_constant__ CUtensorMap tmH, const FusedArgs a) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const int kb_max = (a.H > a.F ? a.H : a.F) / BKB;
  Shared sh;
  sh.ring = smem;
  sh.trans = reinterpret_cast<float*>(smem + kRingBytes);
  sh.xs_sm = sh.trans + TT * kTransStride;
  sh.ws_sm = sh.xs_sm + kb_max * TT;
  sh.amax_sm = sh.ws_sm + 2 * kb_max;
  sh.tile_pref = reinterpret_cast<int*>(sh.amax_sm + kEpiThreads);
  sh.goff = sh.tile_pref + (a.G + 1);
  sh.epi_flag = sh.goff + (a.G + 1);
  sh.meta_sm = sh.epi_flag + 1;
  sh.bars = reinterpret_cast<uint64_t*>((reinterpret_cast<uintptr_t>(sh.meta_sm + 2 * TT) + 15) & ~uintptr_t(15));
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(sh.bars + 32);
  __shared__ int s_ok;
  __shared__ uint32_t s_epoch;
  const int warp = threadIdx.x >> 5;

  if (threadIdx.x == 0) {
    for (int p = 0; p < 2; ++p) {
      uint64_t* b = sh.bars + p * 16;
      for (int s = 0; s < 6; ++s) {
        mbar_init(&b[s], 1);
        mbar_init(&b[6 + s], 1);
      }
      for (int i = 0; i < 2; ++i) {
        mbar_init(&b[12 + i], 1);
        mbar_init(&b[14 + i], 8);
      }
    }
    mbar_fence_init();
    tma_prefetch_desc(&tmW1);
    tma_prefetch_desc(&tmX);
    tma_prefetch_desc(&tmW2);
    tma_prefetch_desc(&tmH);
    s_ok = 1;
    s_epoch = a.ctrl[0];
  }
  if (warp == 2) {
    tmem_alloc(tmem_slot, kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t epoch = s_epoch;
  const uint64_t tag = (uint64_t)epoch + 1;
  auto stamp = [&](int i) {
    if (a.diag && threadIdx.x == 0) {
      if (i == 0) atomicMin(&a.diag[0], globaltimer_ns());
      else atomicMax(&a.diag[i], globaltimer_ns());
    }
  };
  stamp(0);

  bool goff_local = false;
  if (a.fuse_dispatch && (a.phase_mask & 8) && (a.phase_mask & 1) && a.w_tiled && threadIdx.x == 0) {
    // While the dispatch is in flight HBM is idle: bring the first weight tiles this CTA will stream into L2.
    // Which expert a phase-1 item belongs to is only known once the counts have arrived, so this is a guess - in a
    // decode batch every local expert has rows and fewer than 64 of them, which makes token tile i = expert i.
    // A wrong guess costs bandwidth nobody else wanted. About 100 MB over the grid, to stay inside L2.
    const int NT1g = a.F / BMW, kbt = a.H / BKB;
    const int w = blockIdx.x;
    const int e = w / NT1g, j = w % NT1g;
    if (e < a.G) {
      int n = (100 << 20) / (int)gridDim.x / (2 * BMW * BKB);
      if (n > kbt) n = kbt;
      for (int kb = 0; kb < n; ++kb) tma_prefetch_l2_2d(&tmW1, 0, ((e * NT1g + j) * kbt + kb) * (2 * BMW));
    }
  }
  if (a.fuse_dispatch && (a.phase_mask & 12)) {
    // dispatch prologue: the operand ring is free until phase 1 and serves as its scratch
    LLDispatchIO io = a.disp;
    io.phase_mask = (a.phase_mask >> 2) & 3;
    const bool sent = ll_dispatch_body<kThreads>(a.ll_geom, a.ll_off, a.peers, io, sh.ring, sh.goff);
    goff_local = (io.phase_mask & 2) != 0 && sent;
    fence_proxy_async_smem();   // the ring is written by TMA next
    __syncthreads();
    if (!sent && threadIdx.x == 0) s_ok = 0;
    __syncthreads();
  }

  if (a.wait_n > 0 && (a.phase_mask & 1) && !a.exp_gate) {
    if (threadIdx.x < a.wait_n) {
      if (!wait_flag_ge_sys(a.wait_flags + threadIdx.x, tag)) {
        umdk_set_status(a.status, UMDK_ERR_TIMEOUT, UMDK_PH_GROUP_READY, threadIdx.x, (int)epoch);
        s_ok = 0;
      }
    }
    __syncthreads();
  }
  stamp(1);
  // group offsets: from the prologue of this launch (every CTA computed them) or from an earlier dispatch launch
  if (!goff_local) {
    for (int i = threadIdx.x; i <= a.G; i += blockDim.x) sh.goff[i] = a.group_off[i];
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int run = 0;
    for (int e = 0; e < a.G; ++e) {
      sh.tile_pref[e] = run;
      int m = sh.goff[e + 1] - sh.goff[e];
      if (m < 0 || sh.goff[e + 1] > a.n_rows_cap) {
        umdk_set_status(a.status, UMDK_ERR_OVERFLOW, UMDK_PH_GROUP_READY, e, sh.goff[e + 1]);
        m = 0;
        s_ok = 0;
      }
      run += (m + TT - 1) / TT;
    }
    sh.tile_pref[a.G] = run;
  }
  __syncthreads();
  const int tiles = (s_ok && (a.phase_mask & 1)) ? sh.tile_pref[a.G] : 0;
  const int NT1 = a.F / BMW, NT2 = a.H / BMW;
  const int items1 = tiles * NT1, items2 = tiles * NT2;
  const int grid = gridDim.x, c = blockIdx.x;

  // ---- phase 1: items dealt round-robin ----
  run_phase<1>(&tmW1, &tmX, a, sh, tmem_base, c, items1, grid);
  tc_fence_before();
  __syncthreads();  // the ring and the TMEM stages change their layout
  stamp(2);
  tc_fence_after();

  // ---- phase 2: contiguous ranges sized so that all CTAs finish together ----
  // Costs in weight bytes / 128: a phase-1 item streams two 128 x H tiles, a phase-2 item one 128 x F tile.
  // CTAs [0, extra) hold one more phase-1 item than the others ("heavy"); the light CTAs come first in the order of
  // ranges, so they take the phase-2 items whose token tiles were finished in the early phase-1 waves.
  {
    const long long c1 = 2LL * a.H, c2 = a.F;
    const int n1_lo = items1 / grid, extra = items1 % grid, n_light = grid - extra;
    const long long total = (long long)items1 * c1 + (long long)items2 * c2;
    const long long target = (total + grid - 1) / grid;
    long long bl = target - (long long)n1_lo * c1, bh = target - (long long)(n1_lo + 1) * c1;
    if (bl < 0) bl = 0;
    if (bh < 0) bh = 0;
    const int pos = c >= extra ? c - extra : n_light + c;
    auto start_cost = [&](int p) -> long long {
      return p <= n_light ? (long long)p * bl : (long long)n_light * bl + (long long)(p - n_light) * bh;
    };
    long long lo = (start_cost(pos) + c2 - 1) / c2;
    long long hi = pos == grid - 1 ? (long long)items2 : (start_cost(pos + 1) + c2 - 1) / c2;
    if (lo > items2) lo = items2;
    if (hi > items2) hi = items2;
    run_phase<2>(&tmW2, &tmH, a, sh, tmem_base, (int)lo, (int)hi, 1);
  }

  tc_fence_before();
  __syncthreads();
  stamp(3);
  if (warp == 2) {
    tc_fence_after();
    tmem_dealloc(tmem_base, kTmemCols);
  }

  // ---- combine tail ----
  if (a.phase_mask & 1) {
    if (cta_done_is_last(&a.ctrl[1], gridDim.x)) {
      // Every CTA is through with the slab: the arrival words go back to zero BEFORE the combine flags go out - a
      // peer starts its next call (and adds to these words again) only after it has seen this rank's flag.
      if (a.exp_cnt != nullptr)
        for (int i = threadIdx.x; i < a.G; i += blockDim.x) a.exp_cnt[i] = 0;
      for (int i = threadIdx.x; i < tiles; i += blockDim.x) a.tile_done[i] = 0;  // counters start from zero next call
      __threadfence_system();
      __syncthreads();
      if (threadIdx.x < a.R) {
        st_release_sys(reinterpret_cast<uint64_t*>(a.peers.base[threadIdx.x] + a.comb_flag_off) + a.rank, tag);
      }
    }
  }
  if (!(a.phase_mask & 2)) return;
  uint8_t* self = a.peers.base[a.rank];
  if (threadIdx.x < a.R) {
    const uint64_t* f = reinterpret_cast<const uint64_t*>(self + a.comb_flag_off) + threadIdx.x;
    if (!wait_flag_ge_sys(f, tag)) {
      umdk_set_status(a.status, UMDK_ERR_TIMEOUT, UMDK_PH_COMBINE_DATA, threadIdx.x, (int)epoch);
      s_ok = 0;
    }
  }
  __syncthreads();
  stamp(4);
  if (s_ok) {
    ll_weighted_reduce<kThreads>(self + a.comb_buf_off, a.topk_idx, a.topk_w, a.out, a.share_out, a.T, a.Kt, a.H);
  }
  stamp(5);
  if (cta_done_is_last(&a.ctrl[2], gridDim.x)) {
    if (threadIdx.x == 0) a.ctrl[0] = epoch + 1;
  }
}

}  // namespace
}  // namespace umdk

using namespace umdk;

struct UmdkMoeFusedParams {
  int G, F, H, n_rows_cap, max_ctas;
  int w_tiled;             // 0: w1 [G, 2F, H], w2 [G, H, F] row-major; 1: tile-major, see below
  const void* w1;          // fp8 [G, 2F, H]
  const float* w1s;
  const void* w2;          // fp8 [G, H, F]
  const float* w2s;
  const void* x;           // fp8 slab [n_rows_cap, H]
  const float* xs;
  const int* group_off;
  void* hq;
  float* hs;
  uint32_t* tile_done;
  const void* wait_flags;
  int wait_n;
  int R, rank, T, Kt, T_cap;
  void* peers[kMaxRanks];
  uint64_t comb_buf_off, comb_flag_off;
  const int* row_meta;
  const int64_t* topk_idx;
  const float* topk_w;
  void* out;
  void* share_out;
  uint32_t* ctrl;
  int phase_mask;
  int* status;
  unsigned long long* diag;   // optional timeline, see FusedArgs::diag
  // dispatch inside the kernel (disp_x != null): this rank's tokens and the routed geometry; phase_mask bits 2 / 3
  const void* disp_x;         // bf16 [T, H]
  int E;                      // experts over all ranks (G * R)
  int64_t* recv_per_expert;   // out [G]
  int* group_off_out;         // out [G + 1] (may be the same array as group_off)
};

// Weight layouts. Row-major (w_tiled = 0): every 128 x 128-byte weight tile that a k-block needs is 128 separate
// 128-byte pieces H (or F) bytes apart. Tile-major (w_tiled = 1): the same bytes repacked once at load time so that
// the tile of (expert e, weight tile j, k-block kb) is one contiguous chunk -
//   w1: [G][F/128][H/128][256][128]  rows 0..127 = gate rows j*128.., rows 128..255 = up rows F + j*128..
//   w2: [G][H/128][F/128][128][128]
// - which turns the weight stream into 32 KB / 16 KB sequential DRAM reads. Scales are unchanged.
UMDK_API int umdk_moe_fused(const UmdkMoeFusedParams* p, void* stream) {
  if (p->G < 1 || p->F < 128 || (p->F % 128) || p->H < 128 || (p->H % 128) || p->n_rows_cap < 1 || p->R < 1 ||
      p->R > kMaxRanks)
    return -UMDK_ERR_BAD_ARG;
  FusedArgs a;
  a.G = p->G;
  a.F = p->F;
  a.H = p->H;
  a.n_rows_cap = p->n_rows_cap;
  a.group_off = p->group_off;
  a.xs = p->xs;
  a.w1s = p->w1s;
  a.w2s = p->w2s;
  a.hq = static_cast<uint8_t*>(p->hq);
  a.hs = p->hs;
  a.tile_done = p->tile_done;
  a.wait_flags = static_cast<const uint64_t*>(p->wait_flags);
  a.wait_n = p->wait_n;
  for (int i = 0; i < kMaxRanks; ++i) a.peers.base[i] = i < p->R ? static_cast<uint8_t*>(p->peers[i]) : nullptr;
  a.R = p->R;
  a.rank = p->rank;
  a.comb_buf_off = p->comb_buf_off;
  a.comb_flag_off = p->comb_flag_off;
  a.row_meta = p->row_meta;
  a.topk_idx = p->topk_idx;
  a.topk_w = p->topk_w;
  a.out = static_cast<__nv_bfloat16*>(p->out);
  a.share_out = static_cast<__nv_bfloat16*>(p->share_out);
  a.T = p->T;
  a.Kt = p->Kt;
  a.T_cap = p->T_cap;
  a.ctrl = p->ctrl;
  a.phase_mask = p->phase_mask ? p->phase_mask : 3;
  a.w_tiled = p->w_tiled;
  a.status = p->status;
  a.diag = p->diag;
  a.fuse_dispatch = p->disp_x != nullptr ? 1 : 0;
  {
    // the arrival words live in the low-latency region of this rank's heap (the dispatch, fused or not, adds to them)
    EpLLGeom lg;
    if (fill_ll_geom(&lg, p->R, p->rank, p->G * p->R, p->Kt, p->H, p->T_cap) == 0 && a.peers.base[p->rank] != nullptr) {
      a.exp_cnt = reinterpret_cast<uint32_t*>(a.peers.base[p->rank] + ep_ll_offsets(lg).exp_cnt[0]);
      a.exp_parts = ep_ll_row_parts(p->H);
      static const int gate = [] {
        const char* e = getenv("UMDK_LL_EXPERT_GATE");
        return (e && e[0] == '0') ? 0 : 1;
      }();
      a.exp_gate = (gate && p->wait_n > 0) ? 1 : 0;   // callers that pass no flags to wait for gate nothing
    } else {
      a.exp_cnt = nullptr;
      a.exp_parts = 0;
      a.exp_gate = 0;
    }
  }
  if (a.fuse_dispatch) {
    if (p->E != p->G * p->R || p->T > 2048 || p->T > p->T_cap || !p->recv_per_expert || !p->group_off_out)
      return -UMDK_ERR_BAD_ARG;
    if (int rc = fill_ll_geom(&a.ll_geom, p->R, p->rank, p->E, p->Kt, p->H, p->T_cap)) return rc;
    if (a.ll_geom.n_cap != p->n_rows_cap) return -UMDK_ERR_BAD_ARG;
    a.ll_off = ep_ll_offsets(a.ll_geom);
    if (ll_dispatch_smem_bytes(p->T, p->E, p->Kt, kThreads / 32, true) > (size_t)kRingBytes) return -UMDK_ERR_BAD_ARG;
    a.disp.x = static_cast<const __nv_bfloat16*>(p->disp_x);
    a.disp.topk_idx = p->topk_idx;
    a.disp.send_idx = nullptr;
    a.disp.num_per_expert = nullptr;
    a.disp.T = p->T;
    a.disp.group_off = p->group_off_out;
    a.disp.recv_per_expert = p->recv_per_expert;
    a.disp.ctrl = p->ctrl;
    a.disp.status = p->status;
    a.disp.phase_mask = 3;
    a.disp.meet_cycles = umdk_rendezvous_cycles();
  } else {
    if (a.phase_mask & 12) return -UMDK_ERR_BAD_ARG;
    a.ll_geom = EpLLGeom{};
    a.ll_off = EpLLOffsets{};
    a.disp = LLDispatchIO{};
  }
  CUtensorMap tmW1, tmX, tmW2, tmH;
  int bad;
  if (p->w_tiled) {
    bad = make_tmap_2d(&tmW1, TMAP_U8, p->w1, BKB, (uint64_t)p->G * 2 * p->F * (p->H / BKB), BKB, BKB, 2 * BMW,
                       TMAP_SW_128B) ||
          make_tmap_2d(&tmW2, TMAP_U8, p->w2, BKB, (uint64_t)p->G * p->H * (p->F / BKB), BKB, BKB, BMW, TMAP_SW_128B);
  } else {
    bad = make_tmap_2d(&tmW1, TMAP_U8, p->w1, p->H, (uint64_t)p->G * 2 * p->F, p->H, BKB, BMW, TMAP_SW_128B) ||
          make_tmap_2d(&tmW2, TMAP_U8, p->w2, p->F, (uint64_t)p->G * p->H, p->F, BKB, BMW, TMAP_SW_128B);
  }
  if (bad ||
      make_tmap_2d(&tmX, TMAP_U8, p->x, p->H, p->n_rows_cap, p->H, BKB, TT, TMAP_SW_128B) ||
      make_tmap_2d(&tmH, TMAP_U8, p->hq, p->F, p->n_rows_cap, p->F, BKB, TT, TMAP_SW_128B))
    return -UMDK_ERR_BAD_ARG;
  const int kb_max = (p->H > p->F ? p->H : p->F) / BKB;
  const size_t smem = 1024 + (size_t)kRingBytes + TT * kTransStride * 4 + (size_t)kb_max * TT * 4 + 2 * kb_max * 4 +
                      256 * 4 + 2 * (size_t)(p->G + 1) * 4 + 4 + 2 * TT * 4 + 16 + 32 * 8 + 16;
  if (smem > 227 * 1024) return -UMDK_ERR_BAD_ARG;
  UMDK_CUDA_CHECK(cudaFuncSetAttribute(moe_fused_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  int grid = sm_count();
  if (p->max_ctas > 0 && p->max_ctas < grid) grid = p->max_ctas;
  moe_fused_kernel<<<grid, kThreads, smem, static_cast<cudaStream_t>(stream)>>>(tmW1, tmX, tmW2, tmH, a);
  UMDK_CUDA_CHECK(cudaGetLastError());
  return 0;
}
