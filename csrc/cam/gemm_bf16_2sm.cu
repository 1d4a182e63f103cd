// Dense bf16 GEMM with CTA pairs: C[M,N] = A[M,K] * B[N,K]^T, one 256 x 256 output tile per pair of SMs.
//
// The two CTAs of a cluster run one `tcgen05.mma.cta_group::2` together: each CTA stages 128 rows of A and 128 rows
// of B per k-block (32 KB instead of the 48 KB a single-CTA 128 x 256 tile needs), the tensor cores of both SMs read
// the B halves from both shared memories, and each CTA keeps its 128 x 256 half of the accumulator in its own TMEM.
// Per FLOP this halves the shared-memory fill traffic of B, which is what limits the single-CTA kernel
// (gemm_bf16.cu) below the library's throughput.
//
// Roles (per CTA, 256 threads):
//   warp 0     TMA producer: own A half + own B half into its ring; completion bytes are counted on the LEADER CTA's
//              full barrier (`.cta_group::2` loads; no multicast anywhere)
//   warp 1     leader CTA only: one thread issues the pair's MMAs and commits stage release / accumulator ready to the
//              barriers of both CTAs (two plain commits, one per CTA)
//   warp 2     TMEM allocation (both CTAs, `cta_group::2`)
//   warps 4-7  epilogue of the CTA's own 128 rows: tcgen05.ld -> bf16 -> swizzled staging -> TMA store; the
//              accumulator buffer is handed back by arriving on the leader's barrier (remote arrive for CTA 1)
// Every wait is bounded; a timeout is recorded in `status` and all roles drain. No counterpart in the reference.
#include "common.h"
#include "ptx.cuh"

#include <cuda_runtime.h>

namespace umdk {
namespace {

constexpr int BMH = 128;   // rows of A per CTA (tile M = 256 per pair)
constexpr int BNH = 128;   // rows of B per CTA (tile N = 256 per pair)
constexpr int BN = 256;
constexpr int BK = 64;
constexpr int kStages = 6;
constexpr int kThreads = 256;
constexpr int kEpiWarps = 4;
constexpr int kEpiChunkCols = 64;
constexpr int kEpiBufBytes = 32 * kEpiChunkCols * 2;
constexpr int kABytes = BMH * BK * 2;
constexpr int kBBytes = BNH * BK * 2;
constexpr int kStageBytes = kABytes + kBBytes;            // 32 KB per CTA
constexpr int kEpiBytes = kEpiWarps * 2 * kEpiBufBytes;   // 32 KB
constexpr int kSmemBytes = kStages * kStageBytes + kEpiBytes + 256 + 1024;
constexpr int kTmemCols = 512;                            // two 256-column accumulators
constexpr int kGroupM = 8;                                // super-rows of 8 x 256 rows

__device__ __forceinline__ void tile_to_mn(int t, int mb, int nb, int* m_blk, int* n_blk) {
  const int per_group = kGroupM * nb;
  const int g = t / per_group;
  const int first_m = g * kGroupM;
  const int gm = min(kGroupM, mb - first_m);
  const int r = t - g * per_group;
  *m_blk = first_m + r % gm;
  *n_blk = r / gm;
}

__global__ void __launch_bounds__(kThreads, 1)
gemm_bf16_2sm_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                     const __grid_constant__ CUtensorMap tmC, int M, int N, int K, int* status) {
  extern __shared__ uint8_t smem_raw[];
  // identical offsets in both CTAs: the MMA addresses the peer's operands by the leader's offsets
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* epi = smem + kStages * kStageBytes;
  uint64_t* bars = reinterpret_cast<uint64_t*>(epi + kEpiBytes);
  uint64_t* full = bars;
  uint64_t* empty = bars + kStages;
  uint64_t* tfull = bars + 2 * kStages;
  uint64_t* tempty = bars + 2 * kStages + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * kStages + 4);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t cta = cluster_ctarank();      // 0 = leader
  const int pair = blockIdx.x >> 1;
  const int num_pairs = gridDim.x >> 1;
  const int mb = (M + 2 * BMH - 1) / (2 * BMH);
  const int nb = (N + BN - 1) / BN;
  const int kb_total = (K + BK - 1) / BK;
  const int num_tiles = mb * nb;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(&full[s], 1);    // leader's copy is the one in use: one arrive (expect_tx) + the bytes of both CTAs
      mbar_init(&empty[s], 1);   // one commit per CTA copy
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&tfull[i], 1);
      mbar_init(&tempty[i], 2 * kEpiWarps);   // leader's copy: the epilogue warps of both CTAs
    }
    mbar_fence_init();
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmB);
    tma_prefetch_desc(&tmC);
  }
  if (warp == 2) {
    tmem_alloc_pair(tmem_slot, kTmemCols);
    tmem_relinquish_pair();
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();   // the peer's barriers exist before anything is signalled on them
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    if (elect_one()) {
      int s = 0;
      uint32_t ph = 0;
      bool ok = true;
      for (int t = pair; t < num_tiles && ok; t += num_pairs) {
        int m_blk, n_blk;
        tile_to_mn(t, mb, nb, &m_blk, &n_blk);
        const int m0 = m_blk * 2 * BMH + (int)cta * BMH, n0 = n_blk * BN + (int)cta * BNH;
        for (int kb = 0; kb < kb_total; ++kb) {
          if (!mbar_wait(&empty[s], ph ^ 1)) {
            umdk_set_status(status, UMDK_ERR_TIMEOUT, UMDK_PH_TMA_EMPTY, t, kb);
            ok = false;
            break;
          }
          if (cta == 0) mbar_expect_tx(&full[s], 2 * kStageBytes);
          const uint32_t leader_full = map_to_cta(&full[s], 0);
          uint8_t* sa = smem + s * kStageBytes;
          tma_load_2d_pair(sa, &tmA, leader_full, kb * BK, m0);
          tma_load_2d_pair(sa + kABytes, &tmB, leader_full, kb * BK, n0);
          if (++s == kStages) {
            s = 0;
            ph ^= 1;
          }
        }
      }
    }
  } else if (warp == 1 && cta == 0) {
    if (elect_one()) {
      constexpr uint32_t idesc = umma_idesc(kFmtBF16, kFmtBF16, 2 * BMH, BN);
      int s = 0;
      uint32_t ph = 0;
      int it = 0;
      bool ok = true;
      for (int t = pair; t < num_tiles && ok; t += num_pairs, ++it) {
        const int ab = it & 1;
        const uint32_t aph = (it >> 1) & 1;
        if (!mbar_wait(&tempty[ab], aph ^ 1)) {
          umdk_set_status(status, UMDK_ERR_TIMEOUT, UMDK_PH_TMEM_EMPTY, t, 0);
          break;
        }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + ab * BN;
        for (int kb = 0; kb < kb_total; ++kb) {
          if (!mbar_wait(&full[s], ph)) {
            umdk_set_status(status, UMDK_ERR_TIMEOUT, UMDK_PH_TMA_FULL, t, kb);
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t sa = smem_u32(smem + s * kStageBytes);
          const uint64_t adesc = umma_desc_k_sw128(sa);
          const uint64_t bdesc = umma_desc_k_sw128(sa + kABytes);
#pragma unroll
          for (int k = 0; k < BK / 16; ++k) {
            umma_f16_pair(d_tmem, adesc + 2 * k, bdesc + 2 * k, idesc, (kb | k) != 0 ? 1u : 0u);
          }
          // the stage is free in both CTAs once these MMAs have read it
          umma_commit_pair(smem_u32(&empty[s]));
          umma_commit_pair(map_to_cta(&empty[s], 1));
          if (++s == kStages) {
            s = 0;
            ph ^= 1;
          }
        }
        if (ok) {
          umma_commit_pair(smem_u32(&tfull[ab]));
          umma_commit_pair(map_to_cta(&tfull[ab], 1));
        }
      }
    }
  } else if (warp >= 4) {
    const int ew = warp - 4;
    uint8_t* my_epi = epi + ew * 2 * kEpiBufBytes;
    int it = 0;
    int buf = 0;
    for (int t = pair; t < num_tiles; t += num_pairs, ++it) {
      int m_blk, n_blk;
      tile_to_mn(t, mb, nb, &m_blk, &n_blk);
      const int m0 = m_blk * 2 * BMH + (int)cta * BMH, n0 = n_blk * BN;
      const int ab = it & 1;
      const uint32_t aph = (it >> 1) & 1;
      if (!mbar_wait(&tfull[ab], aph)) {
        umdk_set_status(status, UMDK_ERR_TIMEOUT, UMDK_PH_TMEM_FULL, t, 0);
        break;
      }
      tc_fence_after();
      const uint32_t t_addr = tmem_base + (static_cast<uint32_t>(ew * 32) << 16) + ab * BN;
#pragma unroll 1
      for (int c = 0; c < BN / kEpiChunkCols; ++c) {
        uint32_t r[64];
        tmem_ld_x32(t_addr + c * kEpiChunkCols, r);
        tmem_ld_x32(t_addr + c * kEpiChunkCols + 32, r + 32);
        if (lane == 0) tma_store_wait_read<1>();
        __syncwarp();
        tmem_ld_wait();
        uint8_t* dst = my_epi + buf * kEpiBufBytes + lane * 128;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          uint32_t p[4];
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            __nv_bfloat162 h = __floats2bfloat162_rn(__uint_as_float(r[j * 8 + 2 * q]),
                                                     __uint_as_float(r[j * 8 + 2 * q + 1]));
            p[q] = *reinterpret_cast<uint32_t*>(&h);
          }
          *reinterpret_cast<uint4*>(dst + ((j ^ (lane & 7)) << 4)) = make_uint4(p[0], p[1], p[2], p[3]);
        }
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) {
          tma_store_2d(&tmC, my_epi + buf * kEpiBufBytes, n0 + c * kEpiChunkCols, m0 + ew * 32);
          tma_store_commit();
        }
        buf ^= 1;
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(map_to_cta(&tempty[ab], 0));
    }
    if (lane == 0) tma_store_wait<0>();
  }

  // nobody leaves (or frees TMEM) while the peer may still signal this CTA's barriers or read its operands
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();
  if (warp == 2) {
    tc_fence_after();
    tmem_dealloc_pair(tmem_base, kTmemCols);
  }
}

}  // namespace
}  // namespace umdk

// Same contract as umdk_gemm_bf16 (C[M,N] = A[M,K] * B[N,K]^T, bf16 row-major, leading dimensions in elements) for
// shapes with M and N multiples of 256 and K a multiple of 64; other shapes are refused with -UMDK_ERR_BAD_ARG and
// belong to the single-CTA kernel.
UMDK_API int umdk_gemm_bf16_2sm(const void* A, const void* B, void* C, int M, int N, int K, int lda, int ldb, int ldc,
                                int* status, void* stream, int max_ctas) {
  using namespace umdk;
  if (M <= 0 || N <= 0 || K <= 0 || (M % 256) || (N % 256) || (K % BK) || (lda % 8) || (ldb % 8) || (ldc % 8))
    return -UMDK_ERR_BAD_ARG;
  CUtensorMap tmA, tmB, tmC;
  if (make_tmap_2d(&tmA, TMAP_BF16, A, K, M, (uint64_t)lda * 2, BK, BMH, TMAP_SW_128B)) return -UMDK_ERR_BAD_ARG;
  if (make_tmap_2d(&tmB, TMAP_BF16, B, K, N, (uint64_t)ldb * 2, BK, BNH, TMAP_SW_128B)) return -UMDK_ERR_BAD_ARG;
  if (make_tmap_2d(&tmC, TMAP_BF16, C, N, M, (uint64_t)ldc * 2, kEpiChunkCols, 32, TMAP_SW_128B))
    return -UMDK_ERR_BAD_ARG;
  UMDK_CUDA_CHECK(cudaFuncSetAttribute(gemm_bf16_2sm_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes));
  const int tiles = (M / 256) * (N / 256);
  int grid = sm_count();
  if (max_ctas > 0 && max_ctas < grid) grid = max_ctas;
  grid &= ~1;
  if (2 * tiles < grid) grid = 2 * tiles;
  if (grid < 2) return -UMDK_ERR_BAD_ARG;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid, 1, 1);
  cfg.blockDim = dim3(kThreads, 1, 1);
  cfg.dynamicSmemBytes = kSmemBytes;
  cfg.stream = static_cast<cudaStream_t>(stream);
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  UMDK_CUDA_CHECK(cudaLaunchKernelEx(&cfg, gemm_bf16_2sm_kernel, tmA, tmB, tmC, M, N, K, status));
  return 0;
}
