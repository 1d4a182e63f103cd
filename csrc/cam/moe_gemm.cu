// Grouped (per-expert) fp8 GEMMs of the MoE FFN on tcgen05 tensor cores, with the block-scale promotion and the
// FFN epilogues fused in, written for decode-sized expert batches ("swap-AB": weights are the MMA's M operand).
//
//   MODE 0  h = SwiGLU(x @ W1^T)  -> fp8 e4m3 with one fp32 scale per 1x128 block   (gate/up projection)
//   MODE 1  y = h @ W2^T          -> bf16 rows in local memory                      (down projection)
//   MODE 2  y = h @ W2^T          -> bf16 rows stored straight into the token owner's combine buffer over NVLink,
//                                    then completion flags and the owner's top-k weighted reduction in the same
//                                    kernel (down projection fused with combine)
//
// Operand formats: activations fp8 e4m3 [rows, K] with fp32 scales [rows, K/128]; weights fp8 e4m3 [G, N, K] with
// fp32 scales per 128x128 block [G, N/128, K/128]. Per 128-wide K block the tensor core produces a fresh partial
// product in TMEM (128 weight rows x 64 tokens); epilogue warps read it back with tcgen05.ld and accumulate
// partial * w_scale * x_scale in fp32 registers while the next block's MMAs run into the other TMEM stage.
//
// Role split per CTA (persistent, one CTA per SM): warp 0 TMA producer, warp 1 MMA issuer, warp 2 TMEM allocator,
// warps 4-7 promotion + epilogue. The reference fuses the same chain on Ascend cube/vector cores with int8
// operands and per-token scales (src/cam/comm_operator/ascend_kernels/fused_deep_moe/op_kernel/fused_deep_moe.h:354-448,
// epilogue/block/block_epilogue_per_token_dequant_swiglu.h:255-283, gemm/kernel/post_swiglu_dynamic_quant.h:30-60,
// epilogue/block/block_epilogue_per_token_dequant.hpp:199-250 for the combine-send epilogue).
#include "ep_common.cuh"
#include "ptx.cuh"
#include "sync.cuh"

namespace umdk {
namespace {

constexpr int TT = 64;     // tokens per tile (MMA N)
constexpr int BMW = 128;   // weight rows per tile (MMA M)
constexpr int BKB = 128;   // K bytes per block (= 128 fp8 elements = one scale block = one swizzle atom)
constexpr int kThreads = 256;
constexpr int kTransStride = 129;

struct MoeGemmArgs {
  int G;                   // groups (experts)
  int Nout;                // output features per group (MODE 0: F, MODE 1/2: H)
  int K;                   // reduction size (elements)
  int w_rows;              // weight rows per group (MODE 0: 2F, gate rows first; otherwise Nout)
  int n_rows_cap;          // rows allocated in the activation slab
  const int* group_off;    // [G + 1] row offsets of each group inside the slab
  const float* xs;         // [n_rows_cap, K/128]
  const float* ws;         // [G, w_rows/128, K/128]
  uint8_t* hq;             // MODE 0 out: [n_rows_cap, Nout] fp8
  float* hs;               // MODE 0 out: [n_rows_cap, Nout/128]
  __nv_bfloat16* y;        // MODE 1 out: [n_rows_cap, Nout]
  // start gate: wait until flags[i] >= *epoch + 1 for i < wait_n (arrival of the dispatched rows)
  const uint64_t* wait_flags[2];
  int wait_n;
  const uint32_t* epoch_ptr;
  // MODE 2: combine-send + reduce
  PeerTable peers;
  int R, rank;
  uint64_t comb_buf_off[2];   // [T_cap][Kt][Nout] bf16 on every rank
  uint64_t comb_flag_off[2];  // [R] uint64 on every rank
  uint32_t* exp_cnt;          // [G] arrival words of the low-latency dispatch (zeroed here when the call ends)
  const int* row_meta;        // [n_rows_cap][2]: owner rank, owner slot (token * Kt + k)
  const int64_t* topk_idx;    // [T, Kt] on the owner
  const float* topk_w;        // [T, Kt]
  __nv_bfloat16* out;         // [T, Nout]
  int T, Kt, T_cap;
  uint32_t* ctrl;             // [0] epoch (advanced here), [1] send-done counter, [2] reduce-done counter
  int phase_mask;             // MODE 2: bit0 GEMM + combine-send + flags, bit1 wait + reduce + epoch advance
  int* status;
};

template <int MODE>
struct Cfg {
  static constexpr int kATiles = MODE == 0 ? 2 : 1;
  static constexpr int kABytes = kATiles * BMW * BKB;
  static constexpr int kBBytes = TT * BKB;
  static constexpr int kStageBytes = kABytes + kBBytes;
  static constexpr int kStages = MODE == 0 ? 4 : 6;
  static constexpr int kTmemStageCols = kATiles * TT;
  static constexpr int kTmemCols = 256;
  static constexpr int kTransBytes = TT * kTransStride * 4;
};

__device__ __forceinline__ void bar_epi() { asm volatile("bar.sync 1, 128;" ::: "memory"); }

__device__ __forceinline__ uint32_t pack_fp8x4(float a, float b, float c, float d) {
  const __nv_fp8x2_storage_t lo = __nv_cvt_float2_to_fp8x2(make_float2(a, b), __NV_SATFINITE, __NV_E4M3);
  const __nv_fp8x2_storage_t hi = __nv_cvt_float2_to_fp8x2(make_float2(c, d), __NV_SATFINITE, __NV_E4M3);
  return (uint32_t)lo | ((uint32_t)hi << 16);
}

// Maps a tile index to (group, first row, rows in tile) using the prefix table built at kernel start.
__device__ __forceinline__ void locate_tile(const int* tile_pref, const int* goff, int G, int tile, int* e, int* row0,
                                            int* m) {
  int lo = 0, hi = G;  // largest lo with tile_pref[lo] <= tile
  while (hi - lo > 1) {
    const int mid = (lo + hi) >> 1;
    if (tile_pref[mid] <= tile) lo = mid;
    else hi = mid;
  }
  *e = lo;
  const int tt = tile - tile_pref[lo];
  *row0 = goff[lo] + tt * TT;
  *m = min(TT, goff[lo + 1] - *row0);
}

template <int MODE>
__global__ void __launch_bounds__(kThreads, 1)
moe_gemm_kernel(const __grid_constant__ CUtensorMap tmW, const __grid_constant__ CUtensorMap tmX,
                const MoeGemmArgs a) {
  using C = Cfg<MODE>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const int kb_total = a.K / BKB;
  float* trans = reinterpret_cast<float*>(smem + C::kStages * C::kStageBytes);
  float* xs_sm = trans + TT * kTransStride;            // [kb_total][TT]
  float* ws_sm = xs_sm + kb_total * TT;                // [kATiles][kb_total]
  float* amax_sm = ws_sm + 2 * kb_total;               // [128]
  int* tile_pref = reinterpret_cast<int*>(amax_sm + 128);  // [G + 1]
  int* goff_sm = tile_pref + (a.G + 1);                // [G + 1]
  uint64_t* bars = reinterpret_cast<uint64_t*>((reinterpret_cast<uintptr_t>(goff_sm + a.G + 1) + 15) & ~uintptr_t(15));
  uint64_t* full = bars;
  uint64_t* empty = bars + C::kStages;
  uint64_t* tfull = bars + 2 * C::kStages;
  uint64_t* tempty = tfull + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty + 2);
  __shared__ int s_ok;
  __shared__ uint32_t s_epoch;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int NT = a.Nout / BMW;

  if (threadIdx.x == 0) {
    for (int s = 0; s < C::kStages; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&tfull[i], 1);
      mbar_init(&tempty[i], 4);
    }
    mbar_fence_init();
    tma_prefetch_desc(&tmW);
    tma_prefetch_desc(&tmX);
    s_ok = 1;
    s_epoch = a.epoch_ptr ? *a.epoch_ptr : 0u;
  }
  if (warp == 2) {
    tmem_alloc(tmem_slot, C::kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t epoch = s_epoch;
  const int h = epoch & 1;
  const uint64_t tag = (uint64_t)epoch + 1;

  // ---- start gate: dispatched rows have arrived ----
  if (a.wait_n > 0) {
    if (threadIdx.x < a.wait_n) {
      if (!wait_flag_ge_sys(a.wait_flags[h] + threadIdx.x, tag)) {
        umdk_set_status(a.status, UMDK_ERR_TIMEOUT, UMDK_PH_GROUP_READY, threadIdx.x, (int)epoch);
        s_ok = 0;
      }
    }
    __syncthreads();
  }
  // ---- tile table ----
  for (int i = threadIdx.x; i <= a.G; i += blockDim.x) goff_sm[i] = a.group_off[i];
  __syncthreads();
  if (threadIdx.x == 0) {
    int run = 0;
    for (int e = 0; e < a.G; ++e) {
      tile_pref[e] = run;
      int m = goff_sm[e + 1] - goff_sm[e];
      if (m < 0 || goff_sm[e + 1] > a.n_rows_cap) {
        umdk_set_status(a.status, UMDK_ERR_OVERFLOW, UMDK_PH_GROUP_READY, e, goff_sm[e + 1]);
        m = 0;
        s_ok = 0;
      }
      run += (m + TT - 1) / TT;
    }
    tile_pref[a.G] = run;
  }
  __syncthreads();
  const int num_items = (s_ok && (MODE != 2 || (a.phase_mask & 1))) ? tile_pref[a.G] * NT : 0;

  if (warp == 0) {
    if (elect_one()) {
      const uint64_t pol_w = policy_evict_first();
      const uint64_t pol_x = policy_evict_last();
      int s = 0;
      uint32_t ph = 0;
      bool ok = true;
      for (int w = blockIdx.x; w < num_items && ok; w += gridDim.x) {
        int e, row0, m;
        locate_tile(tile_pref, goff_sm, a.G, w / NT, &e, &row0, &m);
        const int j = w % NT;
        for (int kb = 0; kb < kb_total; ++kb) {
          if (!mbar_wait(&empty[s], ph ^ 1)) {
            umdk_set_status(a.status, UMDK_ERR_TIMEOUT, UMDK_PH_TMA_EMPTY, w, kb);
            ok = false;
            break;
          }
          mbar_expect_tx(&full[s], C::kStageBytes);
          uint8_t* st = smem + s * C::kStageBytes;
          tma_load_2d_hint(st, &tmW, &full[s], kb * BKB, e * a.w_rows + j * BMW, pol_w);
          if (MODE == 0) {
            tma_load_2d_hint(st + BMW * BKB, &tmW, &full[s], kb * BKB, e * a.w_rows + a.Nout + j * BMW, pol_w);
          }
          tma_load_2d_hint(st + C::kABytes, &tmX, &full[s], kb * BKB, row0, pol_x);
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
      uint32_t ph = 0;
      uint32_t kbc = 0;  // running K-block counter selects the TMEM stage
      bool ok = true;
      for (int w = blockIdx.x; w < num_items && ok; w += gridDim.x) {
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
          const uint32_t sa = smem_u32(smem + s * C::kStageBytes);
          const uint64_t adesc = umma_desc_k_sw128(sa);
          const uint64_t bdesc = umma_desc_k_sw128(sa + C::kABytes);
          const uint32_t d = tmem_base + ts * C::kTmemStageCols;
#pragma unroll
          for (int k = 0; k < 4; ++k) {  // 32 fp8 elements = 32 bytes per MMA K step
            umma_f8(d, adesc + 2 * k, bdesc + 2 * k, idesc, k > 0 ? 1u : 0u);
            if (MODE == 0) {
              const uint64_t adesc_u = umma_desc_k_sw128(sa + BMW * BKB);
              umma_f8(d + TT, adesc_u + 2 * k, bdesc + 2 * k, idesc, k > 0 ? 1u : 0u);
            }
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
    const int ew = warp - 4;
    const int tid = ew * 32 + lane;  // 0..127 == weight row inside the tile == TMEM lane
    const int nsb = a.K / 128;       // activation scale blocks per row
    const int wsb = a.w_rows / 128;  // weight scale block rows per group
    uint32_t kbc = 0;
    bool ok = true;
    for (int w = blockIdx.x; w < num_items && ok; w += gridDim.x) {
      int e, row0, m;
      locate_tile(tile_pref, goff_sm, a.G, w / NT, &e, &row0, &m);
      const int j = w % NT;
      // stage this tile's scales: xs_sm[kb][t], ws_sm[tile][kb]
      for (int i = tid; i < TT * kb_total; i += 128) {
        const int t = i / kb_total, kb = i - t * kb_total;
        xs_sm[kb * TT + t] = t < m ? a.xs[(size_t)(row0 + t) * nsb + kb] : 0.f;
      }
      for (int i = tid; i < C::kATiles * kb_total; i += 128) {
        const int which = i / kb_total, kb = i - which * kb_total;
        const int brow = (which == 0 ? j : (a.Nout / 128 + j));
        ws_sm[which * kb_total + kb] = a.ws[((size_t)e * wsb + brow) * nsb + kb];
      }
      bar_epi();
      float acc_g[TT];
      float acc_u[MODE == 0 ? TT : 1];
#pragma unroll
      for (int c = 0; c < TT; ++c) acc_g[c] = 0.f;
      if (MODE == 0) {
#pragma unroll
        for (int c = 0; c < TT; ++c) acc_u[c] = 0.f;
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
        const float wg = ws_sm[kb];
        const float wu = MODE == 0 ? ws_sm[kb_total + kb] : 0.f;
        const uint32_t taddr = tmem_base + (static_cast<uint32_t>(ew * 32) << 16) + ts * C::kTmemStageCols;
        const float* xsk = xs_sm + kb * TT;
#pragma unroll
        for (int c0 = 0; c0 < TT; c0 += 16) {
          uint32_t rg[16];
          uint32_t ru[16];
          tmem_ld_x16(taddr + c0, rg);
          if (MODE == 0) tmem_ld_x16(taddr + TT + c0, ru);
          tmem_ld_wait();
#pragma unroll
          for (int c = 0; c < 16; ++c) {
            const float xsv = xsk[c0 + c];
            acc_g[c0 + c] = fmaf(__uint_as_float(rg[c]), xsv * wg, acc_g[c0 + c]);
            if (MODE == 0) acc_u[c0 + c] = fmaf(__uint_as_float(ru[c]), xsv * wu, acc_u[c0 + c]);
          }
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&tempty[ts]);
      }
      if (!ok) break;
      // ---- tile epilogue: transpose through shared memory so that each thread owns half a token row ----
#pragma unroll
      for (int c = 0; c < TT; ++c) {
        float v = acc_g[c];
        if (MODE == 0) v = (v / (1.f + __expf(-v))) * acc_u[c];
        trans[c * kTransStride + tid] = v;
      }
      bar_epi();
      const int t = tid & 63, half = tid >> 6;
      const float* src = trans + t * kTransStride + half * 64;
      const int row = row0 + t;
      if (MODE == 0) {
        float amax = 0.f;
#pragma unroll 8
        for (int i = 0; i < 64; ++i) amax = fmaxf(amax, fabsf(src[i]));
        amax_sm[tid] = amax;
        bar_epi();
        amax = fmaxf(fmaxf(amax_sm[t], amax_sm[t + 64]), 1e-4f);
        const float inv = 448.f / amax;
        if (t < m) {
          uint8_t* dst = a.hq + (size_t)row * a.Nout + j * BMW + half * 64;
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            int4 o;
            o.x = pack_fp8x4(src[q * 16 + 0] * inv, src[q * 16 + 1] * inv, src[q * 16 + 2] * inv, src[q * 16 + 3] * inv);
            o.y = pack_fp8x4(src[q * 16 + 4] * inv, src[q * 16 + 5] * inv, src[q * 16 + 6] * inv, src[q * 16 + 7] * inv);
            o.z = pack_fp8x4(src[q * 16 + 8] * inv, src[q * 16 + 9] * inv, src[q * 16 + 10] * inv, src[q * 16 + 11] * inv);
            o.w = pack_fp8x4(src[q * 16 + 12] * inv, src[q * 16 + 13] * inv, src[q * 16 + 14] * inv, src[q * 16 + 15] * inv);
            reinterpret_cast<int4*>(dst)[q] = o;
          }
          if (half == 0) a.hs[(size_t)row * (a.Nout / 128) + j] = amax * (1.f / 448.f);
        }
      } else {
        if (t < m) {
          uint8_t* dst;
          if (MODE == 1) {
            dst = reinterpret_cast<uint8_t*>(a.y + (size_t)row * a.Nout + j * BMW + half * 64);
          } else {
            const int owner = a.row_meta[2 * row], slot = a.row_meta[2 * row + 1];
            if (owner < 0 || owner >= a.R || slot < 0 || slot >= a.T_cap * a.Kt) {
              umdk_set_status(a.status, UMDK_ERR_OVERFLOW, UMDK_PH_COMBINE_DATA, owner, slot);
              dst = nullptr;
            } else {
              dst = a.peers.base[owner] + a.comb_buf_off[h] + ((size_t)slot * a.Nout + j * BMW + half * 64) * 2;
            }
          }
          if (dst != nullptr) {
#pragma unroll
            for (int q = 0; q < 8; ++q) {
              int4 o;
              __nv_bfloat162* po = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
              for (int i = 0; i < 4; ++i) po[i] = __floats2bfloat162_rn(src[q * 8 + 2 * i], src[q * 8 + 2 * i + 1]);
              if (MODE == 2) st_na_v4(dst + q * 16, o);
              else reinterpret_cast<int4*>(dst)[q] = o;
            }
          }
        }
      }
      bar_epi();  // trans / scale staging is reused by the next tile
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 2) {
    tc_fence_after();
    tmem_dealloc(tmem_base, C::kTmemCols);
  }

  if (MODE == 2) {
    // ---- completion flags to every peer, then the owner-side weighted reduction ----
    if (a.phase_mask & 1) {
      if (cta_done_is_last(&a.ctrl[1], gridDim.x)) {
        // the slab has been consumed: its arrival words return to zero before the flags that let the peers go on
        if (a.exp_cnt != nullptr)
          for (int i = threadIdx.x; i < a.G; i += blockDim.x) a.exp_cnt[i] = 0;
        __threadfence_system();
        __syncthreads();
        if (threadIdx.x < a.R) {
          st_release_sys(reinterpret_cast<uint64_t*>(a.peers.base[threadIdx.x] + a.comb_flag_off[h]) + a.rank, tag);
        }
      }
    }
    if (!(a.phase_mask & 2)) return;
    uint8_t* self = a.peers.base[a.rank];
    if (threadIdx.x < a.R) {
      const uint64_t* f = reinterpret_cast<const uint64_t*>(self + a.comb_flag_off[h]) + threadIdx.x;
      if (!wait_flag_ge_sys(f, tag)) {
        umdk_set_status(a.status, UMDK_ERR_TIMEOUT, UMDK_PH_COMBINE_DATA, threadIdx.x, (int)epoch);
        s_ok = 0;
      }
    }
    __syncthreads();
    if (s_ok) {
      const int nvec = a.Nout / 8;
      const int nwarps = kThreads / 32;
      for (int t = blockIdx.x * nwarps + warp; t < a.T; t += gridDim.x * nwarps) {
        const int4* src = reinterpret_cast<const int4*>(self + a.comb_buf_off[h] + (size_t)t * a.Kt * a.Nout * 2);
        for (int v = lane; v < nvec; v += 32) {
          float acc[8];
#pragma unroll
          for (int i = 0; i < 8; ++i) acc[i] = 0.f;
          for (int k = 0; k < a.Kt; ++k) {
            if (a.topk_idx[(size_t)t * a.Kt + k] < 0) continue;
            const float wk = a.topk_w[(size_t)t * a.Kt + k];
            const int4 val = ld_relaxed_sys_v4(src + (size_t)k * nvec + v);
            const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&val);
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              const float2 f = __bfloat1622float2(p[i]);
              acc[2 * i] = fmaf(wk, f.x, acc[2 * i]);
              acc[2 * i + 1] = fmaf(wk, f.y, acc[2 * i + 1]);
            }
          }
          int4 o;
          __nv_bfloat162* po = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
          for (int i = 0; i < 4; ++i) po[i] = __floats2bfloat162_rn(acc[2 * i], acc[2 * i + 1]);
          reinterpret_cast<int4*>(a.out + (size_t)t * a.Nout)[v] = o;
        }
      }
    }
    if (cta_done_is_last(&a.ctrl[2], gridDim.x)) {
      if (threadIdx.x == 0) a.ctrl[0] = epoch + 1;
    }
  }
}

template <int MODE>
size_t smem_bytes(int K, int G) {
  using C = Cfg<MODE>;
  const int kb = K / BKB;
  return 1024 + (size_t)C::kStages * C::kStageBytes + C::kTransBytes + (size_t)kb * TT * 4 + 2 * kb * 4 + 128 * 4 +
         2 * (size_t)(G + 1) * 4 + 16 + (2 * C::kStages + 4) * 8 + 16;
}

template <int MODE>
int launch(const void* W, const void* X, const MoeGemmArgs& a, cudaStream_t stream, int max_ctas) {
  CUtensorMap tmW, tmX;
  if (make_tmap_2d(&tmW, TMAP_U8, W, a.K, (uint64_t)a.G * a.w_rows, a.K, BKB, BMW, TMAP_SW_128B))
    return -UMDK_ERR_BAD_ARG;
  if (make_tmap_2d(&tmX, TMAP_U8, X, a.K, a.n_rows_cap, a.K, BKB, TT, TMAP_SW_128B)) return -UMDK_ERR_BAD_ARG;
  const size_t smem = smem_bytes<MODE>(a.K, a.G);
  if (smem > 227 * 1024) return -UMDK_ERR_BAD_ARG;
  UMDK_CUDA_CHECK(cudaFuncSetAttribute(moe_gemm_kernel<MODE>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  int grid = sm_count();
  if (max_ctas > 0 && max_ctas < grid) grid = max_ctas;
  moe_gemm_kernel<MODE><<<grid, kThreads, smem, stream>>>(tmW, tmX, a);
  UMDK_CUDA_CHECK(cudaGetLastError());
  return 0;
}

}  // namespace
}  // namespace umdk

using namespace umdk;

struct UmdkMoeGemmParams {
  int mode;                // 0, 1 or 2
  int G, Nout, K, n_rows_cap, max_ctas;
  const void* w;           // fp8 [G, w_rows, K] (mode 0: w_rows = 2 * Nout, gate rows first)
  const float* ws;         // [G, w_rows/128, K/128]
  const void* x;           // fp8 [n_rows_cap, K]
  const float* xs;         // [n_rows_cap, K/128]
  const int* group_off;    // [G + 1]
  void* hq;
  float* hs;
  void* y;
  const void* wait_flags[2];
  int wait_n;
  const uint32_t* epoch_ptr;
  // mode 2
  int R, rank, T, Kt, T_cap;
  void* peers[kMaxRanks];
  uint64_t comb_buf_off[2];
  uint64_t comb_flag_off[2];
  const int* row_meta;
  const int64_t* topk_idx;
  const float* topk_w;
  void* out;
  uint32_t* ctrl;
  int* status;
  int phase_mask;
};

UMDK_API int umdk_moe_gemm(const UmdkMoeGemmParams* p, void* stream) {
  if (p->G < 1 || p->Nout < 128 || (p->Nout % 128) || p->K < 128 || (p->K % 128) || p->n_rows_cap < 1)
    return -UMDK_ERR_BAD_ARG;
  MoeGemmArgs a;
  a.G = p->G;
  a.Nout = p->Nout;
  a.K = p->K;
  a.w_rows = p->mode == 0 ? 2 * p->Nout : p->Nout;
  a.n_rows_cap = p->n_rows_cap;
  a.group_off = p->group_off;
  a.xs = p->xs;
  a.ws = p->ws;
  a.hq = static_cast<uint8_t*>(p->hq);
  a.hs = p->hs;
  a.y = static_cast<__nv_bfloat16*>(p->y);
  a.wait_flags[0] = static_cast<const uint64_t*>(p->wait_flags[0]);
  a.wait_flags[1] = static_cast<const uint64_t*>(p->wait_flags[1]);
  a.wait_n = p->wait_n;
  a.epoch_ptr = p->epoch_ptr;
  a.R = p->R;
  a.rank = p->rank;
  for (int i = 0; i < kMaxRanks; ++i) a.peers.base[i] = i < p->R ? static_cast<uint8_t*>(p->peers[i]) : nullptr;
  a.comb_buf_off[0] = p->comb_buf_off[0];
  a.comb_buf_off[1] = p->comb_buf_off[1];
  a.comb_flag_off[0] = p->comb_flag_off[0];
  a.comb_flag_off[1] = p->comb_flag_off[1];
  a.exp_cnt = nullptr;
  if (p->mode == 2 && p->R >= 1 && p->R <= kMaxRanks && a.peers.base[p->rank] != nullptr) {
    EpLLGeom lg;
    if (fill_ll_geom(&lg, p->R, p->rank, p->G * p->R, p->Kt, p->Nout, p->T_cap) == 0)
      a.exp_cnt = reinterpret_cast<uint32_t*>(a.peers.base[p->rank] + ep_ll_offsets(lg).exp_cnt[0]);
  }
  a.row_meta = p->row_meta;
  a.topk_idx = p->topk_idx;
  a.topk_w = p->topk_w;
  a.out = static_cast<__nv_bfloat16*>(p->out);
  a.T = p->T;
  a.Kt = p->Kt;
  a.T_cap = p->T_cap;
  a.ctrl = p->ctrl;
  a.status = p->status;
  a.phase_mask = p->phase_mask ? p->phase_mask : 3;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  switch (p->mode) {
    case 0: return launch<0>(p->w, p->x, a, s, p->max_ctas);
    case 1: return launch<1>(p->w, p->x, a, s, p->max_ctas);
    case 2:
      if (p->R < 1 || p->R > kMaxRanks || p->ctrl == nullptr || p->epoch_ptr == nullptr) return -UMDK_ERR_BAD_ARG;
      return launch<2>(p->w, p->x, a, s, p->max_ctas);
    default: return -UMDK_ERR_BAD_ARG;
  }
}
