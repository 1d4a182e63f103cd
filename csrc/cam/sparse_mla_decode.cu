// Sparse top-k MLA flash-attention decode over a paged KV cache, on tcgen05 tensor cores.
//
// Shapes (DeepSeek-V3 style multi-head latent attention with absorbed projections): per sequence one query token,
// 128 heads, each head a 576-vector (512 latent + 64 rope); every head attends to the SAME key rows, which are the
// 576-wide latent rows of the paged cache, and the value of a key is the first 512 entries of that row. Only the
// `topk` rows listed in `indices` take part (-1 or >= seq_len: masked).
//
// Mapping to the hardware: the 128 heads are exactly the M = 128 rows of one tcgen05 MMA, and one sequence (one
// split of its key list) is handled by a CLUSTER OF TWO CTAs that split the work by feature dimension:
//   CTA 0 owns latent dims [0, 256) plus the 64 rope dims, CTA 1 owns latent dims [256, 512).
// Per chunk of 48 selected keys each CTA
//   gathers only ITS dims of the 48 rows (640 or 512 bytes per row; no byte of the cache is read twice),
//   computes a PARTIAL S[128 x 48] = Q[:, own dims] * K[:, own dims]^T   (20 or 16 MMAs of K = 16),
//   sends the partial to its partner through distributed shared memory and adds the partner's partial,
//   runs the online softmax (one head per thread; both CTAs arrive at the same P),
//   and accumulates its own 256 output columns O[128 x 256] += P[128 x 48] * V[48 x own latent dims]  (3 MMAs),
//   reading V from the SAME gathered tile through an MN-major descriptor.
// Splitting by dimension halves the resident Q (80 KB instead of 144 KB), which makes room for a three-stage ring
// of key tiles, and halves the Q*K^T work of each SM. Roles inside a CTA (13 warps):
//   warps 0-3  softmax: tcgen05.ld of S, add the partner's partial, exp2, P to shared memory, lazy rescale of O
//   warps 9-12 exchange: tcgen05.ld of the same S and asynchronous stores of it into the partner's shared memory,
//              so that the round trip between the two CTAs is off the softmax warps' critical path
//   warp  4    one thread issues every MMA: Q*K^T of chunk c+1 is issued BEFORE P*V of chunk c, so the tensor
//              pipe works on the next scores while the softmax of the current chunk runs (S is double-buffered)
//   warp  5    gather producer: TMA tile::gather4 copies (four selected rows x 128 bytes per instruction, written
//              in the 128-byte-swizzled layout the MMA descriptors expect), completion counted in bytes on the
//              stage's barrier. Gathering with 16-byte cp.async was measured first: an SM sustains only about
//              10 bytes per clock of such loads (2800 cycles for a 30 KB tile), whatever the access pattern
// All row addresses of the split are resolved once, up front, into shared memory (index -> page -> row).
// The running maximum is only raised when it grows by more than 8 (in log2 units); P then stays below 2^8 and the
// accumulated O needs rescaling only a few times per row instead of in most chunks.
// Every wait is bounded; a CTA that gives up raises the abort flag of both CTAs so the partner leaves at once.
// There is no attention code in the reference project; the op is specified by the serving configuration only.
#include "common.h"
#include "ptx.cuh"

namespace umdk {
namespace {

constexpr int kHeads = 128;
constexpr int kDim = 576;
constexpr int kDimV = 512;
constexpr int kPage = 64;
constexpr int kChunk = 48;                       // keys per pipeline step
constexpr int kStages = 3;
constexpr int kMaxSlabs = 5;                     // 64-dim slabs per CTA: 4 latent (+ 1 rope in CTA 0)
constexpr int kQSlabBytes = kHeads * 128;        // 16 KB
constexpr int kKSlabBytes = kChunk * 128;        // 6 KB
constexpr int kQBytes = kMaxSlabs * kQSlabBytes; // 81920
constexpr int kStageBytes = kMaxSlabs * kKSlabBytes;  // 30720
constexpr int kPBytes = kHeads * 128;            // 16 KB (96 of every 128 bytes used)
constexpr int kXBytes = kChunk * kHeads * 4;     // 24 KB, [key / 4][head][4] fp32
constexpr int kMaxChunks = 43;                   // 2064 keys per split at most
constexpr int kMaxKeys = kMaxChunks * kChunk;
constexpr int kThreads = 416;
constexpr int kProducerWarps = 4;   // warps 5..8 issue the gather copies: the TMA unit takes them faster from several warps
constexpr int kTmemCols = 512;
constexpr int kColS = 0;                         // two S buffers of 64 columns (48 used)
constexpr int kColO = 128;
constexpr int kOffK = kQBytes;
constexpr int kOffP = kOffK + kStages * kStageBytes;
constexpr int kOffX = kOffP + kPBytes;
constexpr int kOffRows = kOffX + kXBytes;
constexpr int kOffMask = kOffRows + kMaxKeys * 4;   // one 64-bit validity mask per chunk
constexpr int kOffTail = kOffMask + ((kMaxChunks * 8 + 63) / 64) * 64;
constexpr int kSmemBytes = 1024 + kOffTail + 256;
static_assert(kSmemBytes <= 232448, "shared memory budget");
static_assert(kStageBytes % 1024 == 0 && kKSlabBytes % 1024 == 0, "swizzle atoms must stay 1024-byte aligned");

struct MlaArgs {
  const __nv_bfloat16* kv;   // [num_pages, 64, 576]
  const int* block_table;    // [B, max_pages]
  const int* indices;        // [B, topk]
  const int* seq_lens;       // [B] or null
  __nv_bfloat16* out;        // [B, 128, 512]
  float* lse;                // [B, 128]
  float* part_o;             // [B, splits, 128, 512] fp32 (splits > 1)
  float* part_lse;           // [B, splits, 128]
  int B, topk, max_pages, num_pages, num_splits;
  float scale_log2;
  int* status;
  // optional [16] cycle counters of the first CTA (diagnose mode): softmax thread 0: [0] wait S, [1] TMEM load,
  // [2] wait partner-free, [3] remote stores, [4] wait partner's partial, [5] add + max + exp2, [6] wait P*V, [7] P
  // store (+ rescale); MMA thread: [8] wait tile, [9] wait S buffer, [10] wait P, [11] issue; producer thread 0:
  // [12] wait landed, [13] wait free stage, [14] issue; [15] total cycles of the CTA
  long long* diag;
};

__device__ __forceinline__ bool mbar_try_wait_cluster(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n"
      "selp.u32 %0, 1, 0, p;\n"
      "}\n"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
// Bounded waits that also leave when either CTA of the pair has raised the abort flag.
template <bool kCluster>
__device__ __forceinline__ bool wait_bar(uint64_t* bar, uint32_t parity, volatile int* abort_flag) {
  if (kCluster ? mbar_try_wait_cluster(bar, parity) : mbar_try_wait(bar, parity)) return true;
  const long long t0 = clock64();
  uint32_t spins = 0;
  while (!(kCluster ? mbar_try_wait_cluster(bar, parity) : mbar_try_wait(bar, parity))) {
    if ((++spins & 31u) == 0) {
      if (*abort_flag) return false;
      if (clock64() - t0 > kSpinLimitCycles) return false;
    }
  }
  return true;
}
// Asynchronous 16-byte store into the partner CTA's shared memory; the bytes are counted on the partner's mbarrier
// (complete_tx), so the sender needs no release fence that would wait for every store to be acknowledged.
__device__ __forceinline__ void st_async_v4(uint32_t cluster_addr, uint32_t a, uint32_t b, uint32_t c, uint32_t d,
                                            uint32_t cluster_bar) {
  asm volatile("st.async.weak.shared::cluster.mbarrier::complete_tx::bytes.v4.b32 [%0], {%1, %2, %3, %4}, [%5];" ::"r"(
                   cluster_addr),
               "r"(a), "r"(b), "r"(c), "r"(d), "r"(cluster_bar)
               : "memory");
}
// Four rows of a 2-D tensor (row numbers r.x .. r.w, `col` = first element of the box in each row) into four
// consecutive 128-byte rows of shared memory; the tensor map has a box of {64 elements, 1 row} and the 128-byte swizzle.
__device__ __forceinline__ void tma_gather4(void* smem_dst, const CUtensorMap* m, uint64_t* bar, int col, int4 r) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.tile::gather4.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, "
      "%5, %6, %7}], [%2];" ::"r"(smem_u32(smem_dst)),
      "l"(reinterpret_cast<uint64_t>(m)), "r"(smem_u32(bar)), "r"(col), "r"(r.x), "r"(r.y), "r"(r.z), "r"(r.w)
      : "memory");
}
// Arrival on the partner's barrier WITHOUT release semantics. A release at cluster scope waits until every store this
// thread has in flight (the asynchronous remote stores above all) is acknowledged, which was measured at about 3000
// cycles per chunk. The barrier it is used for (`partner may overwrite my exchange buffer`) only has to follow this
// warp's LOADS of that buffer, and those have completed once their values were used: instructions issue in order.
__device__ __forceinline__ void mbar_arrive_cluster_relaxed(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.relaxed.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
// 2^x with the special-function unit's native approximation (2 ulp; -inf gives 0): P is rounded to bf16 anyway.
__device__ __forceinline__ float ex2_approx(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ void st_cluster_u32(uint32_t cluster_addr, uint32_t v) {
  asm volatile("st.shared::cluster.u32 [%0], %1;" ::"r"(cluster_addr), "r"(v) : "memory");
}

__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kThreads, 1)
sparse_mla_decode_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmKV,
                         const MlaArgs a) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* q_sm = smem;
  uint8_t* k_sm = smem + kOffK;
  uint8_t* p_sm = smem + kOffP;
  float* x_sm = reinterpret_cast<float*>(smem + kOffX);
  int* rows_sm = reinterpret_cast<int*>(smem + kOffRows);
  unsigned long long* mask_sm = reinterpret_cast<unsigned long long*>(smem + kOffMask);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + kOffTail);
  uint64_t* bar_q = bars;            // 1
  // Arrivals are one per WARP: the lanes order their own accesses before a __syncwarp() and lane 0 arrives, so a
  // barrier sees 4 arrivals per phase instead of 128 (128 arrivals on one barrier, remote ones above all, cost
  // more than the work they guard).
  uint64_t* bar_full = bars + 1;     // kStages, one arrival that expects the tile's bytes from the TMA gathers
  uint64_t* bar_empty = bars + 4;    // kStages, one commit
  uint64_t* bar_s = bars + 7;        // 2, one commit
  uint64_t* bar_sfree = bars + 9;    // 2, arrivals of the 4 softmax warps and the 4 exchange warps
  uint64_t* bar_p = bars + 11;       // 4 softmax-warp arrivals
  uint64_t* bar_o = bars + 12;       // one commit
  uint64_t* bar_xfull = bars + 13;   // one local arrival that expects the 24 KB the partner's st.async stores deliver
  uint64_t* bar_xfree = bars + 14;   // 4 arrivals from the partner's softmax warps: its X may be overwritten
  uint64_t* bar_fin = bars + 15;     // one commit (drain on the abort path)
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 16);
  volatile int* s_abort = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int b = blockIdx.y;
  const int half = static_cast<int>(cluster_ctarank());   // == blockIdx.x & 1
  const int split = blockIdx.x >> 1;
  const int n_slabs = half == 0 ? 5 : 4;
  const int per_split = ((a.topk + a.num_splits - 1) / a.num_splits + kChunk - 1) / kChunk * kChunk;
  const int k_begin = split * per_split;
  const int k_end = min(a.topk, k_begin + per_split);
  const int num_chunks = k_end > k_begin ? (k_end - k_begin + kChunk - 1) / kChunk : 0;
  const int seq_len = a.seq_lens ? a.seq_lens[b] : 0x7fffffff;

  if (tid == 0) {
    mbar_init(bar_q, 1);
    for (int i = 0; i < kStages; ++i) {
      mbar_init(&bar_full[i], 1);
      mbar_init(&bar_empty[i], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&bar_s[i], 1);
      mbar_init(&bar_sfree[i], 8);
    }
    mbar_init(bar_p, 4);
    mbar_init(bar_o, 1);
    mbar_init(bar_xfull, 1);
    mbar_init(bar_xfree, 4);
    mbar_init(bar_fin, 1);
    mbar_fence_init();
    tma_prefetch_desc(&tmQ);
    tma_prefetch_desc(&tmKV);
    *s_abort = 0;
  }
  if (warp == 4) {
    tmem_alloc(tmem_slot, kTmemCols);
    tmem_relinquish();
  }
  // resolve every selected row of this split once: index -> page -> row number in the pool (-1 = masked)
  for (int k = tid; k < num_chunks * kChunk; k += kThreads) {
    const int kpos = k_begin + k;
    int idx = kpos < k_end ? a.indices[(size_t)b * a.topk + kpos] : -1;
    if (idx < 0 || idx >= seq_len) idx = -1;
    int row = -1;
    if (idx >= 0) {
      const int pg = idx / kPage;
      const int page = pg < a.max_pages ? a.block_table[(size_t)b * a.max_pages + pg] : -1;
      if (page < 0 || page >= a.num_pages) {
        umdk_set_status(a.status, UMDK_ERR_OVERFLOW, UMDK_PH_NONE, b, idx);
      } else {
        row = page * kPage + (idx % kPage);
      }
    }
    rows_sm[k] = row;
  }
  __syncthreads();
  for (int c = tid; c < num_chunks; c += kThreads) {   // bit j of mask c: key j of chunk c takes part
    unsigned long long m = 0;
    for (int j = 0; j < kChunk; ++j)
      if (rows_sm[c * kChunk + j] >= 0) m |= 1ull << j;
    mask_sm[c] = m;
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();   // the partner's barriers exist before anything is signalled across
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t peer = static_cast<uint32_t>(half ^ 1);
  const uint32_t peer_abort = map_to_cta(const_cast<int*>(s_abort), peer);

  auto give_up = [&](int phase, int detail) {
    if (!*s_abort) umdk_set_status(a.status, UMDK_ERR_TIMEOUT, phase, b, detail);
    *s_abort = 1;
    st_cluster_u32(peer_abort, 1u);
  };

  if (num_chunks > 0) {
    if (warp < 4) {
      // ===================================== softmax ======================================================
      const int head = tid;   // == TMEM lane
      const uint32_t lane_addr = tmem_base + (static_cast<uint32_t>(warp * 32) << 16);
      if (tid == 0) mbar_expect_tx(bar_xfull, kXBytes);   // arms the first phase; re-armed after every chunk
      const uint32_t peer_xfree = map_to_cta(bar_xfree, peer);
      float m_run = -INFINITY, l_run = 0.f;
      bool ok = true;
      const bool dg = a.diag != nullptr && blockIdx.x == 0 && blockIdx.y == 0 && tid == 0;
      long long dt[8] = {0, 0, 0, 0, 0, 0, 0, 0};
      long long t_prev = dg ? clock64() : 0;
      auto lap = [&](int i) {
        if (dg) {
          const long long t = clock64();
          dt[i] += t - t_prev;
          t_prev = t;
        }
      };
      for (int c = 0; c < num_chunks && ok; ++c) {
        const int sb = c & 1;
        if (!__all_sync(0xffffffffu, wait_bar<false>(&bar_s[sb], (c >> 1) & 1, s_abort))) {
          give_up(UMDK_PH_TMEM_FULL, c);
          ok = false;
          break;
        }
        lap(0);
        tc_fence_after();
        uint32_t sr[kChunk];
        tmem_ld_x16(lane_addr + kColS + sb * 64, sr);
        tmem_ld_x16(lane_addr + kColS + sb * 64 + 16, sr + 16);
        tmem_ld_x16(lane_addr + kColS + sb * 64 + 32, sr + 32);
        tmem_ld_wait();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&bar_sfree[sb]);
        lap(1);
        // the partner's partial comes in through the exchange warps of the other CTA
        if (!__all_sync(0xffffffffu, wait_bar<true>(bar_xfull, c & 1, s_abort))) {
          give_up(UMDK_PH_GROUP_READY, 1000 + c);
          ok = false;
          break;
        }
        lap(4);
        // S = own partial + partner's partial (raw dot products; the scale is folded into the exponent below)
        const unsigned long long valid = mask_sm[c];
        float mx = -INFINITY;
#pragma unroll
        for (int j4 = 0; j4 < kChunk / 4; ++j4) {
          const float4 xv = reinterpret_cast<const float4*>(x_sm)[j4 * kHeads + head];
          const float xs4[4] = {xv.x, xv.y, xv.z, xv.w};
#pragma unroll
          for (int u = 0; u < 4; ++u) {
            const int j = 4 * j4 + u;
            float t = __uint_as_float(sr[j]) + xs4[u];
            if (!((valid >> j) & 1ull)) t = -INFINITY;
            sr[j] = __float_as_uint(t);
            mx = fmaxf(mx, t);
          }
        }
        // every lane's loads of x_sm have returned (mx depends on them); keep the arrival behind that dependence
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 0));
        if (tid == 0 && c + 1 < num_chunks) mbar_expect_tx(bar_xfull, kXBytes);   // next phase, before the partner may send
        __syncwarp();
        if (lane == 0) mbar_arrive_cluster_relaxed(peer_xfree);
        mx *= a.scale_log2;   // scale_log2 > 0: the maximum of the scaled scores
        // lazy maximum: raise it only when it grows by more than 8 (P stays below 2^8)
        float alpha = 1.f;
        if (mx > m_run + 8.f || m_run == -INFINITY) {
          const float m_new = fmaxf(m_run, mx);
          alpha = (m_run == -INFINITY) ? 0.f : ex2_approx(m_run - m_new);
          if (m_new == -INFINITY) alpha = 1.f;   // nothing seen yet, nothing to scale
          m_run = m_new;
        }
        const float neg_m = m_run == -INFINITY ? 0.f : -m_run;
        float sum = 0.f;
        uint32_t pk[kChunk / 2];
#pragma unroll
        for (int j = 0; j < kChunk / 2; ++j) {
          const float p0 = ex2_approx(fmaf(__uint_as_float(sr[2 * j]), a.scale_log2, neg_m));
          const float p1 = ex2_approx(fmaf(__uint_as_float(sr[2 * j + 1]), a.scale_log2, neg_m));
          sum += p0 + p1;
          const __nv_bfloat162 hh = __floats2bfloat162_rn(p0, p1);
          pk[j] = *reinterpret_cast<const uint32_t*>(&hh);
        }
        l_run = l_run * alpha + sum;
        lap(5);
        // P(c) overwrites P(c-1) and O may be rescaled: P(c-1) * V must have finished
        if (c >= 1 && !__all_sync(0xffffffffu, wait_bar<false>(bar_o, (c - 1) & 1, s_abort))) {
          give_up(UMDK_PH_TMEM_EMPTY, c);
          ok = false;
          break;
        }
        lap(6);
        tc_fence_after();
        if (c >= 1 && __any_sync(0xffffffffu, alpha != 1.f)) {
#pragma unroll 1
          for (int c0 = 0; c0 < 256; c0 += 32) {
            uint32_t o[32];
            tmem_ld_x32(lane_addr + kColO + c0, o);
            tmem_ld_wait();
#pragma unroll
            for (int j = 0; j < 32; ++j) o[j] = __float_as_uint(__uint_as_float(o[j]) * alpha);
            tmem_st_x32(lane_addr + kColO + c0, o);
          }
          tmem_st_wait();
        }
        uint8_t* prow = p_sm + head * 128;
#pragma unroll
        for (int j8 = 0; j8 < kChunk / 8; ++j8)
          *reinterpret_cast<uint4*>(prow + ((j8 ^ (head & 7)) << 4)) =
              make_uint4(pk[4 * j8], pk[4 * j8 + 1], pk[4 * j8 + 2], pk[4 * j8 + 3]);
        fence_proxy_async_smem();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(bar_p);
        lap(7);
      }
      if (dg) {
        for (int i = 0; i < 8; ++i)
          if (i != 2 && i != 3) a.diag[i] = dt[i];
      }
      // ---- epilogue: this CTA's 256 output columns ----
      // (every decision below is warp-uniform: the TMEM loads are warp-collective)
      if (ok && !__all_sync(0xffffffffu, wait_bar<false>(bar_o, (num_chunks - 1) & 1, s_abort))) {
        give_up(UMDK_PH_TMEM_EMPTY, 2000);
        ok = false;
      }
      tc_fence_after();
      if (ok) {
        const float inv = l_run > 0.f ? 1.f / l_run : 0.f;
        const float lse2 = l_run > 0.f ? m_run + log2f(l_run) : -INFINITY;
        if (a.num_splits == 1) {
          __nv_bfloat16* dst = a.out + ((size_t)b * kHeads + head) * kDimV + half * 256;
#pragma unroll 1
          for (int c0 = 0; c0 < 256; c0 += 32) {
            uint32_t o[32];
            tmem_ld_x32(lane_addr + kColO + c0, o);
            tmem_ld_wait();
#pragma unroll
            for (int q = 0; q < 4; ++q) {
              uint32_t w4[4];
#pragma unroll
              for (int i = 0; i < 4; ++i) {
                const __nv_bfloat162 hh = __floats2bfloat162_rn(__uint_as_float(o[q * 8 + 2 * i]) * inv,
                                                                __uint_as_float(o[q * 8 + 2 * i + 1]) * inv);
                w4[i] = *reinterpret_cast<const uint32_t*>(&hh);
              }
              *reinterpret_cast<uint4*>(dst + c0 + q * 8) = make_uint4(w4[0], w4[1], w4[2], w4[3]);
            }
          }
          if (half == 0 && a.lse) a.lse[(size_t)b * kHeads + head] = lse2 * 0.6931471805599453f;
        } else {
          float* dst = a.part_o + (((size_t)b * a.num_splits + split) * kHeads + head) * kDimV + half * 256;
#pragma unroll 1
          for (int c0 = 0; c0 < 256; c0 += 32) {
            uint32_t o[32];
            tmem_ld_x32(lane_addr + kColO + c0, o);
            tmem_ld_wait();
#pragma unroll
            for (int q = 0; q < 8; ++q) {
              *reinterpret_cast<float4*>(dst + c0 + q * 4) =
                  make_float4(__uint_as_float(o[q * 4]) * inv, __uint_as_float(o[q * 4 + 1]) * inv,
                              __uint_as_float(o[q * 4 + 2]) * inv, __uint_as_float(o[q * 4 + 3]) * inv);
            }
          }
          if (half == 0) a.part_lse[((size_t)b * a.num_splits + split) * kHeads + head] = lse2;
        }
      }
    } else if (warp == 4) {
      // ===================================== MMA issuer ===================================================
      if (lane == 0) {
        mbar_expect_tx(bar_q, static_cast<uint32_t>(n_slabs) * kQSlabBytes);
        for (int j = 0; j < n_slabs; ++j) {
          const int dim0 = j < 4 ? half * 256 + j * 64 : 512;
          tma_load_2d(q_sm + j * kQSlabBytes, &tmQ, bar_q, dim0, b * kHeads);
        }
        constexpr uint32_t idesc_qk = umma_idesc(kFmtBF16, kFmtBF16, kHeads, kChunk);
        constexpr uint32_t idesc_pv = umma_idesc(kFmtBF16, kFmtBF16, kHeads, 256, 0, 1);
        bool ok = wait_bar<false>(bar_q, 0, s_abort);
        if (!ok) give_up(UMDK_PH_TMA_FULL, 0);
        const bool dg = a.diag != nullptr && blockIdx.x == 0 && blockIdx.y == 0;
        long long dt[4] = {0, 0, 0, 0};
        const long long t_begin = dg ? clock64() : 0;
        long long t_prev = t_begin;
        auto lap = [&](int i) {
          if (dg) {
            const long long t = clock64();
            dt[i] += t - t_prev;
            t_prev = t;
          }
        };
        auto issue_qk = [&](int c) -> bool {
          const int st = c % kStages;
          if (!wait_bar<false>(&bar_full[st], (c / kStages) & 1, s_abort)) {
            give_up(UMDK_PH_TMA_FULL, 100 + c);
            return false;
          }
          lap(0);
          if (c >= 2 && !wait_bar<false>(&bar_sfree[c & 1], ((c >> 1) - 1) & 1, s_abort)) {
            give_up(UMDK_PH_TMEM_EMPTY, 100 + c);
            return false;
          }
          lap(1);
          tc_fence_after();
          const uint32_t d = tmem_base + kColS + (c & 1) * 64;
          for (int j = 0; j < n_slabs; ++j) {
            const uint64_t ad = umma_desc_k_sw128(smem_u32(q_sm + j * kQSlabBytes));
            const uint64_t bd = umma_desc_k_sw128(smem_u32(k_sm + st * kStageBytes + j * kKSlabBytes));
#pragma unroll
            for (int k = 0; k < 4; ++k) umma_f16(d, ad + 2 * k, bd + 2 * k, idesc_qk, (j | k) ? 1u : 0u);
          }
          umma_commit(&bar_s[c & 1]);
          lap(3);
          return true;
        };
        if (ok) ok = issue_qk(0);
        for (int c = 0; c < num_chunks && ok; ++c) {
          if (c + 1 < num_chunks) ok = issue_qk(c + 1);
          if (!ok) break;
          if (!wait_bar<false>(bar_p, c & 1, s_abort)) {
            give_up(UMDK_PH_GROUP_READY, 200 + c);
            ok = false;
            break;
          }
          lap(2);
          tc_fence_after();
          const int st = c % kStages;
          const uint32_t v_base = smem_u32(k_sm + st * kStageBytes);
#pragma unroll
          for (int k = 0; k < kChunk / 16; ++k) {   // 16 keys per step: A advances 32 bytes, B two 8-key groups
            const uint64_t ad = umma_desc_k_sw128(smem_u32(p_sm)) + 2 * k;
            const uint64_t bd = umma_desc_mn_sw128(v_base + k * 2048, kKSlabBytes, 1024);
            umma_f16(tmem_base + kColO, ad, bd, idesc_pv, (c | k) ? 1u : 0u);
          }
          umma_commit(&bar_empty[st]);
          umma_commit(bar_o);
          lap(3);
        }
        if (dg) {
          for (int i = 0; i < 4; ++i) a.diag[8 + i] = dt[i];
          a.diag[15] = clock64() - t_begin;
        }
        if (!ok) {   // leave only after every MMA already issued has retired (they read smem and write TMEM)
          umma_commit(bar_fin);
          mbar_wait(bar_fin, 0);
        }
      }
    } else if (warp >= 9) {
      // ===================================== exchange (warps 9..12) =======================================
      const int head = (warp & 3) * 32 + lane;   // == TMEM lane
      const uint32_t lane_addr = tmem_base + (static_cast<uint32_t>((warp & 3) * 32) << 16);
      const uint32_t peer_x = map_to_cta(x_sm, peer) + static_cast<uint32_t>(head) * 16u;
      const uint32_t peer_xfull = map_to_cta(bar_xfull, peer);
      const bool dg = a.diag != nullptr && blockIdx.x == 0 && blockIdx.y == 0 && head == 0;
      long long dt[2] = {0, 0};
      long long t_prev = dg ? clock64() : 0;
      for (int c = 0; c < num_chunks; ++c) {
        const int sb = c & 1;
        if (!__all_sync(0xffffffffu, wait_bar<false>(&bar_s[sb], (c >> 1) & 1, s_abort))) {
          give_up(UMDK_PH_TMEM_FULL, 3000 + c);
          break;
        }
        tc_fence_after();
        uint32_t sr[kChunk];
        tmem_ld_x16(lane_addr + kColS + sb * 64, sr);
        tmem_ld_x16(lane_addr + kColS + sb * 64 + 16, sr + 16);
        tmem_ld_x16(lane_addr + kColS + sb * 64 + 32, sr + 32);
        tmem_ld_wait();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&bar_sfree[sb]);
        if (dg) t_prev = clock64();
        // the partner's softmax warps must have read the previous partial out of their exchange buffer
        if (c >= 1 && !__all_sync(0xffffffffu, wait_bar<false>(bar_xfree, (c - 1) & 1, s_abort))) {
          give_up(UMDK_PH_GROUP_READY, c);
          break;
        }
        if (dg) {
          const long long t = clock64();
          dt[0] += t - t_prev;
          t_prev = t;
        }
#pragma unroll
        for (int j4 = 0; j4 < kChunk / 4; ++j4)
          st_async_v4(peer_x + j4 * (kHeads * 16), sr[4 * j4], sr[4 * j4 + 1], sr[4 * j4 + 2], sr[4 * j4 + 3],
                      peer_xfull);
        if (dg) dt[1] += clock64() - t_prev;
      }
      if (dg) {
        a.diag[2] = dt[0];
        a.diag[3] = dt[1];
      }
    } else if (warp >= 5 && warp < 5 + kProducerWarps) {
      // ===================================== gather producers (warps 5..) =====================================
      bool ok = true;
      const bool dg = a.diag != nullptr && blockIdx.x == 0 && blockIdx.y == 0 && lane == 0 && warp == 5;
      long long dt[3] = {0, 0, 0};
      long long t_prev = dg ? clock64() : 0;
      auto lap = [&](int i) {
        if (dg) {
          const long long t = clock64();
          dt[i] += t - t_prev;
          t_prev = t;
        }
      };
      const int n_inst = (kChunk / 4) * n_slabs;   // gather4 copies per tile
      for (int c = 0; c < num_chunks && ok; ++c) {
        const int st = c % kStages;
        if (c >= kStages) {
          ok = __all_sync(0xffffffffu, wait_bar<false>(&bar_empty[st], ((c / kStages) - 1) & 1, s_abort));
          if (!ok) {
            if (lane == 0) give_up(UMDK_PH_TMA_EMPTY, c);
            break;
          }
        }
        lap(1);
        if (warp == 5 && lane == 0) mbar_expect_tx(&bar_full[st], static_cast<uint32_t>(n_slabs) * kKSlabBytes);
        __syncwarp();
        uint8_t* stage = k_sm + st * kStageBytes;
        const int4* rows4 = reinterpret_cast<const int4*>(rows_sm + c * kChunk);
        for (int u = (warp - 5) * 32 + lane; u < n_inst; u += 32 * kProducerWarps) {
          const int grp = u / n_slabs, slab = u - grp * n_slabs;
          int4 r = rows4[grp];
          r.x = max(r.x, 0);   // masked keys read row 0: their scores are set to -inf before the softmax
          r.y = max(r.y, 0);
          r.z = max(r.z, 0);
          r.w = max(r.w, 0);
          const int col = slab < 4 ? half * 256 + slab * 64 : 512;
          tma_gather4(stage + slab * kKSlabBytes + grp * 512, &tmKV, &bar_full[st], col, r);
        }
        lap(2);
      }
      if (dg) {
        for (int i = 0; i < 3; ++i) a.diag[12 + i] = dt[i];
      }
    }
  } else if (warp < 4) {
    // empty split: zeros and -inf so that the merge ignores it
    const int head = tid;
    if (a.num_splits == 1) {
      __nv_bfloat16* dst = a.out + ((size_t)b * kHeads + head) * kDimV + half * 256;
      for (int c0 = 0; c0 < 256; c0 += 8) *reinterpret_cast<uint4*>(dst + c0) = make_uint4(0, 0, 0, 0);
      if (half == 0 && a.lse) a.lse[(size_t)b * kHeads + head] = -INFINITY;
    } else {
      float* dst = a.part_o + (((size_t)b * a.num_splits + split) * kHeads + head) * kDimV + half * 256;
      for (int c0 = 0; c0 < 256; c0 += 4) *reinterpret_cast<float4*>(dst + c0) = make_float4(0.f, 0.f, 0.f, 0.f);
      if (half == 0) a.part_lse[((size_t)b * a.num_splits + split) * kHeads + head] = -INFINITY;
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 4) {
    tc_fence_after();
    tmem_dealloc(tmem_base, kTmemCols);
  }
  cluster_sync_all();   // neither CTA leaves while the other may still write into its shared memory
}

// Joins the key-list splits: out = sum_i exp2(lse_i - lse) * o_i.
__global__ void __launch_bounds__(128) mla_merge_kernel(const float* __restrict__ part_o,
                                                        const float* __restrict__ part_lse,
                                                        __nv_bfloat16* __restrict__ out, float* __restrict__ lse,
                                                        int num_splits) {
  const int bh = blockIdx.x;  // b * 128 + head
  const int b = bh / kHeads, head = bh % kHeads;
  float mx = -INFINITY;
  for (int s = 0; s < num_splits; ++s) mx = fmaxf(mx, part_lse[((size_t)b * num_splits + s) * kHeads + head]);
  float den = 0.f;
  for (int s = 0; s < num_splits; ++s) {
    const float v = part_lse[((size_t)b * num_splits + s) * kHeads + head];
    den += v == -INFINITY ? 0.f : exp2f(v - mx);
  }
  for (int d = threadIdx.x; d < kDimV; d += blockDim.x) {
    float acc = 0.f;
    for (int s = 0; s < num_splits; ++s) {
      const float v = part_lse[((size_t)b * num_splits + s) * kHeads + head];
      const float w = (v == -INFINITY || den == 0.f) ? 0.f : exp2f(v - mx) / den;
      acc += w * part_o[(((size_t)b * num_splits + s) * kHeads + head) * kDimV + d];
    }
    out[(size_t)bh * kDimV + d] = __float2bfloat16(acc);
  }
  if (threadIdx.x == 0 && lse) lse[bh] = den > 0.f ? (mx + log2f(den)) * 0.6931471805599453f : -INFINITY;
}

}  // namespace
}  // namespace umdk

using namespace umdk;

// Smallest num_splits the kernel accepts for a key list of `topk` entries.
UMDK_API int umdk_sparse_mla_min_splits(int topk) { return (topk + kMaxKeys - 1) / kMaxKeys; }

// q: [B, 128, 576] bf16; kv: [num_pages, 64, 576] bf16; block_table: [B, max_pages]; indices: [B, topk];
// out: [B, 128, 512] bf16; lse: [B, 128] fp32 (may be null). part_o / part_lse: scratch for num_splits > 1
// ([B, splits, 128, 512] and [B, splits, 128] fp32).
UMDK_API int umdk_sparse_mla_decode(const void* q, const void* kv, const int* block_table, const int* indices,
                                    const int* seq_lens, void* out, float* lse, float* part_o, float* part_lse,
                                    int B, int topk, int max_pages, int num_pages, int num_splits, float sm_scale,
                                    int* status, void* stream, long long* diag) {
  if (B < 1 || topk < 1 || max_pages < 1 || num_pages < 1 || num_splits < 1) return -UMDK_ERR_BAD_ARG;
  if (num_splits > 1 && (part_o == nullptr || part_lse == nullptr)) return -UMDK_ERR_BAD_ARG;
  // one CTA pair resolves at most kMaxKeys rows of the key list up front (see umdk_sparse_mla_min_splits)
  if (((topk + num_splits - 1) / num_splits + kChunk - 1) / kChunk > kMaxChunks) return -UMDK_ERR_BAD_ARG;
  if ((size_t)num_pages * kPage > 0x7fffffffull) return -UMDK_ERR_BAD_ARG;
  CUtensorMap tmQ, tmKV;
  if (make_tmap_2d(&tmQ, TMAP_BF16, q, kDim, (uint64_t)B * kHeads, kDim * 2, 64, kHeads, TMAP_SW_128B))
    return -UMDK_ERR_BAD_ARG;
  // the cache as a matrix of token rows; box = one 128-byte piece of one row (tile::gather4 takes four of them)
  if (make_tmap_2d(&tmKV, TMAP_BF16, kv, kDim, (uint64_t)num_pages * kPage, kDim * 2, 64, 1, TMAP_SW_128B))
    return -UMDK_ERR_BAD_ARG;
  static bool attr = false;
  if (!attr) {
    UMDK_CUDA_CHECK(cudaFuncSetAttribute(sparse_mla_decode_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         kSmemBytes));
    attr = true;
  }
  MlaArgs a;
  a.kv = static_cast<const __nv_bfloat16*>(kv);
  a.block_table = block_table;
  a.indices = indices;
  a.seq_lens = seq_lens;
  a.out = static_cast<__nv_bfloat16*>(out);
  a.lse = lse;
  a.part_o = part_o;
  a.part_lse = part_lse;
  a.B = B;
  a.topk = topk;
  a.max_pages = max_pages;
  a.num_pages = num_pages;
  a.num_splits = num_splits;
  a.scale_log2 = sm_scale * 1.4426950408889634f;
  a.status = status;
  a.diag = diag;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  dim3 grid(2 * num_splits, B);
  sparse_mla_decode_kernel<<<grid, kThreads, kSmemBytes, s>>>(tmQ, tmKV, a);
  UMDK_CUDA_CHECK(cudaGetLastError());
  if (num_splits > 1) {
    mla_merge_kernel<<<B * kHeads, 128, 0, s>>>(part_o, part_lse, static_cast<__nv_bfloat16*>(out), lse, num_splits);
    UMDK_CUDA_CHECK(cudaGetLastError());
  }
  return 0;
}
