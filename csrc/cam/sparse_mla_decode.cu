// Sparse top-k MLA flash-attention decode over a paged KV cache, on tcgen05 tensor cores.
//
// Shapes (DeepSeek-V3 style multi-head latent attention with absorbed projections): per sequence one query token,
// 128 heads, each head a 576-vector (512 latent + 64 rope); every head attends to the SAME key rows, which are the
// 576-wide latent rows of the paged cache, and the value of a key is the first 512 entries of that row. Only the
// `topk` rows listed in `indices` take part (-1 or >= seq_len: masked).
//
// Mapping to the hardware: the 128 heads are exactly the M = 128 rows of one tcgen05 MMA.
//   S[128 x 64]  = Q[128 x 576] * Kc[64 x 576]^T      36 MMAs (K = 16), Q resident in shared memory (TMA, 9 slabs)
//   P            = online softmax of S, one head per thread of the 4 softmax warps (tcgen05.ld), bf16 into smem
//   O[128 x 256] += P[128 x 64] * Vc[64 x 256]         4 MMAs (K = 16 keys), V read from the SAME gathered smem tile
//                                                      through an MN-major descriptor (no second copy of K)
// Each sequence is handled by two CTAs that own one 256-wide half of the output (O for all 512 columns plus S does
// not fit the 512 TMEM columns) and by `num_splits` CTAs along the key list; a merge kernel joins the splits.
// The 64 selected rows of a chunk are gathered with 16-byte cp.async into the 128-byte-swizzled layout that both
// descriptors expect. There is no attention code in the reference project; the op is specified by the serving
// configuration only.
#include "common.h"
#include "ptx.cuh"

namespace umdk {
namespace {

constexpr int kHeads = 128;
constexpr int kDim = 576;
constexpr int kDimV = 512;
constexpr int kPage = 64;
constexpr int kChunk = 64;
constexpr int kSlabs = kDim / 64;              // 9 slabs of 64 dims
constexpr int kQSlabBytes = kHeads * 128;      // 16 KB
constexpr int kKSlabBytes = kChunk * 128;      // 8 KB
constexpr int kQBytes = kSlabs * kQSlabBytes;  // 147456
constexpr int kKBytes = kSlabs * kKSlabBytes;  // 73728
constexpr int kThreads = 256;
constexpr int kTmemCols = 512;
constexpr int kColS = 0;
constexpr int kColO = 64;
constexpr int kSmemBytes = 1024 + kQBytes + kKBytes + 1024;

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
};

__device__ __forceinline__ void bar_softmax() { asm volatile("bar.sync 1, 128;" ::: "memory"); }

__global__ void __launch_bounds__(kThreads, 1)
sparse_mla_decode_kernel(const __grid_constant__ CUtensorMap tmQ, const MlaArgs a) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* q_sm = smem;
  uint8_t* k_sm = smem + kQBytes;
  uint8_t* tail = k_sm + kKBytes;
  uint64_t* bar_q = reinterpret_cast<uint64_t*>(tail);
  uint64_t* bar_s = bar_q + 1;
  uint64_t* bar_o = bar_q + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bar_q + 3);
  int* s_abort = reinterpret_cast<int*>(tmem_slot + 1);
  int* idx_sm = reinterpret_cast<int*>(tail + 64);                                   // [64]
  const uint8_t** row_sm = reinterpret_cast<const uint8_t**>(tail + 64 + 256);        // [64]

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int b = blockIdx.y;
  const int half = blockIdx.x & 1;
  const int split = blockIdx.x >> 1;
  const int per_split = ((a.topk + a.num_splits - 1) / a.num_splits + kChunk - 1) / kChunk * kChunk;
  const int k_begin = split * per_split;
  const int k_end = min(a.topk, k_begin + per_split);
  const int num_chunks = k_end > k_begin ? (k_end - k_begin + kChunk - 1) / kChunk : 0;
  const int seq_len = a.seq_lens ? a.seq_lens[b] : 0x7fffffff;

  if (tid == 0) {
    mbar_init(bar_q, 1);
    mbar_init(bar_s, 1);
    mbar_init(bar_o, 1);
    mbar_fence_init();
    tma_prefetch_desc(&tmQ);
    *s_abort = 0;
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (tid == 0 && num_chunks > 0) {
    mbar_expect_tx(bar_q, kQBytes);
    for (int j = 0; j < kSlabs; ++j) tma_load_2d(q_sm + j * kQSlabBytes, &tmQ, bar_q, j * 64, b * kHeads);
  }

  // softmax state of this thread's head (softmax warps only)
  const int head = (warp & 3) * 32 + lane;
  float m_run = -INFINITY, l_run = 0.f;
  const uint32_t lane_addr = tmem_base + (static_cast<uint32_t>((warp & 3) * 32) << 16);
  uint8_t* p_sm = k_sm + (half ? 0 : 4) * kKSlabBytes;  // P lives in two slabs this CTA does not need for P*V

  for (int c = 0; c < num_chunks; ++c) {
    const uint32_t ph = c & 1;
    // ---- 1. gather 64 key rows into the swizzled slabs ----
    if (tid < kChunk) {
      const int kpos = k_begin + c * kChunk + tid;
      int idx = kpos < k_end ? a.indices[(size_t)b * a.topk + kpos] : -1;
      if (idx < 0 || idx >= seq_len) idx = -1;
      size_t row = 0;
      if (idx >= 0) {
        const int pg = idx / kPage;
        int page = pg < a.max_pages ? a.block_table[(size_t)b * a.max_pages + pg] : -1;
        if (page < 0 || page >= a.num_pages) {
          umdk_set_status(a.status, UMDK_ERR_OVERFLOW, UMDK_PH_NONE, b, idx);
          idx = -1;
        } else {
          row = (size_t)page * kPage + (idx % kPage);
        }
      }
      idx_sm[tid] = idx;
      row_sm[tid] = reinterpret_cast<const uint8_t*>(a.kv) + row * (kDim * 2);
    }
    __syncthreads();
#pragma unroll 6
    for (int it = 0; it < (kChunk * 72) / kThreads; ++it) {
      const int i = it * kThreads + tid;
      const int key = i / 72, ch = i - key * 72;
      const int slab = ch >> 3, c8 = ch & 7;
      cp_async_16(k_sm + slab * kKSlabBytes + key * 128 + ((c8 ^ (key & 7)) << 4), row_sm[key] + ch * 16);
    }
    cp_async_commit();
    cp_async_wait<0>();
    fence_proxy_async_smem();
    __syncthreads();

    // ---- 2. S = Q K^T ----
    if (tid == 0) {
      bool ok = true;
      if (c == 0) ok = mbar_wait(bar_q, 0);
      if (!ok) {
        umdk_set_status(a.status, UMDK_ERR_TIMEOUT, UMDK_PH_TMA_FULL, b, 0);
        *s_abort = 1;
      }
      tc_fence_after();
      constexpr uint32_t idesc = umma_idesc(kFmtBF16, kFmtBF16, kHeads, kChunk);
#pragma unroll 1
      for (int j = 0; j < kSlabs; ++j) {
        const uint64_t ad = umma_desc_k_sw128(smem_u32(q_sm + j * kQSlabBytes));
        const uint64_t bd = umma_desc_k_sw128(smem_u32(k_sm + j * kKSlabBytes));
#pragma unroll
        for (int k = 0; k < 4; ++k) umma_f16(tmem_base + kColS, ad + 2 * k, bd + 2 * k, idesc, (j | k) ? 1u : 0u);
      }
      umma_commit(bar_s);
    }

    // ---- 3. online softmax, P to smem, O += P V ----
    if (warp >= 4) {
      if (!mbar_wait(bar_s, ph)) {
        umdk_set_status(a.status, UMDK_ERR_TIMEOUT, UMDK_PH_TMEM_FULL, b, c);
        *s_abort = 1;
      }
      tc_fence_after();
      uint32_t sr[64];
      tmem_ld_x32(lane_addr + kColS, sr);
      tmem_ld_x32(lane_addr + kColS + 32, sr + 32);
      tmem_ld_wait();
      float mx = -INFINITY;
#pragma unroll
      for (int j = 0; j < 64; ++j) {
        float s = __uint_as_float(sr[j]) * a.scale_log2;
        if (idx_sm[j] < 0) s = -INFINITY;
        sr[j] = __float_as_uint(s);
        mx = fmaxf(mx, s);
      }
      const float m_new = fmaxf(m_run, mx);
      const float m_use = m_new == -INFINITY ? 0.f : m_new;
      const float alpha = exp2f(m_run - m_use);  // m_run = -inf -> 0
      float sum = 0.f;
      uint8_t* prow = p_sm + head * 128;
#pragma unroll
      for (int j8 = 0; j8 < 8; ++j8) {
        uint32_t pk[4];
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          const float p0 = exp2f(__uint_as_float(sr[j8 * 8 + 2 * q]) - m_use);
          const float p1 = exp2f(__uint_as_float(sr[j8 * 8 + 2 * q + 1]) - m_use);
          sum += p0 + p1;
          const __nv_bfloat162 hh = __floats2bfloat162_rn(p0, p1);
          pk[q] = *reinterpret_cast<const uint32_t*>(&hh);
        }
        *reinterpret_cast<uint4*>(prow + ((j8 ^ (head & 7)) << 4)) = make_uint4(pk[0], pk[1], pk[2], pk[3]);
      }
      l_run = l_run * alpha + sum;
      m_run = m_new;
      // rescale the running output when the maximum moved (warp-uniform decision)
      if (c > 0 && __any_sync(0xffffffffu, alpha != 1.f)) {
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
      fence_proxy_async_smem();
      tc_fence_before();
      bar_softmax();
      if (tid == 128) {
        tc_fence_after();
        constexpr uint32_t idesc_pv = umma_idesc(kFmtBF16, kFmtBF16, kHeads, 256, 0, 1);
        const uint32_t v_base = smem_u32(k_sm + (half * 4) * kKSlabBytes);
#pragma unroll
        for (int k = 0; k < 4; ++k) {  // 16 keys per step: A advances 32 bytes, B advances two 8-key groups
          const uint64_t ad = umma_desc_k_sw128(smem_u32(p_sm)) + 2 * k;
          const uint64_t bd = umma_desc_mn_sw128(v_base + k * 2048, kKSlabBytes, 1024);
          umma_f16(tmem_base + kColO, ad, bd, idesc_pv, (c | k) ? 1u : 0u);
        }
        umma_commit(bar_o);
      }
    }
    // ---- 4. the tile (and P) may be overwritten only after P V has finished ----
    if (!mbar_wait(bar_o, ph)) {
      umdk_set_status(a.status, UMDK_ERR_TIMEOUT, UMDK_PH_TMEM_EMPTY, b, c);
      *s_abort = 1;
    }
    tc_fence_after();
    __syncthreads();
    if (*s_abort) break;
  }

  // ---- epilogue ----
  if (warp >= 4 && !*s_abort) {
    const float inv = l_run > 0.f ? 1.f / l_run : 0.f;
    const float lse2 = l_run > 0.f ? m_run + log2f(l_run) : -INFINITY;
    if (a.num_splits == 1) {
      __nv_bfloat16* dst = a.out + ((size_t)b * kHeads + head) * kDimV + half * 256;
#pragma unroll 1
      for (int c0 = 0; c0 < 256; c0 += 32) {
        uint32_t o[32];
        if (num_chunks > 0) {
          tmem_ld_x32(lane_addr + kColO + c0, o);
          tmem_ld_wait();
        } else {
#pragma unroll
          for (int j = 0; j < 32; ++j) o[j] = 0;
        }
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          uint32_t pk[4];
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const __nv_bfloat162 hh = __floats2bfloat162_rn(__uint_as_float(o[q * 8 + 2 * i]) * inv,
                                                            __uint_as_float(o[q * 8 + 2 * i + 1]) * inv);
            pk[i] = *reinterpret_cast<const uint32_t*>(&hh);
          }
          *reinterpret_cast<uint4*>(dst + c0 + q * 8) = make_uint4(pk[0], pk[1], pk[2], pk[3]);
        }
      }
      if (half == 0 && a.lse) a.lse[(size_t)b * kHeads + head] = lse2 * 0.6931471805599453f;
    } else {
      float* dst = a.part_o + (((size_t)b * a.num_splits + split) * kHeads + head) * kDimV + half * 256;
#pragma unroll 1
      for (int c0 = 0; c0 < 256; c0 += 32) {
        uint32_t o[32];
        if (num_chunks > 0) {
          tmem_ld_x32(lane_addr + kColO + c0, o);
          tmem_ld_wait();
        } else {
#pragma unroll
          for (int j = 0; j < 32; ++j) o[j] = 0;
        }
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
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, kTmemCols);
  }
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

// q: [B, 128, 576] bf16; kv: [num_pages, 64, 576] bf16; block_table: [B, max_pages]; indices: [B, topk];
// out: [B, 128, 512] bf16; lse: [B, 128] fp32 (may be null). part_o / part_lse: scratch for num_splits > 1
// ([B, splits, 128, 512] and [B, splits, 128] fp32).
UMDK_API int umdk_sparse_mla_decode(const void* q, const void* kv, const int* block_table, const int* indices,
                                    const int* seq_lens, void* out, float* lse, float* part_o, float* part_lse,
                                    int B, int topk, int max_pages, int num_pages, int num_splits, float sm_scale,
                                    int* status, void* stream) {
  if (B < 1 || topk < 1 || max_pages < 1 || num_pages < 1 || num_splits < 1) return -UMDK_ERR_BAD_ARG;
  if (num_splits > 1 && (part_o == nullptr || part_lse == nullptr)) return -UMDK_ERR_BAD_ARG;
  CUtensorMap tmQ;
  if (make_tmap_2d(&tmQ, TMAP_BF16, q, kDim, (uint64_t)B * kHeads, kDim * 2, 64, kHeads, TMAP_SW_128B))
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
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  dim3 grid(2 * num_splits, B);
  sparse_mla_decode_kernel<<<grid, kThreads, kSmemBytes, s>>>(tmQ, a);
  UMDK_CUDA_CHECK(cudaGetLastError());
  if (num_splits > 1) {
    mla_merge_kernel<<<B * kHeads, 128, 0, s>>>(part_o, part_lse, static_cast<__nv_bfloat16*>(out), lse, num_splits);
    UMDK_CUDA_CHECK(cudaGetLastError());
  }
  return 0;
}
