// Dense bf16 GEMM on the 5th-generation tensor cores: C[M,N] = A[M,K] * B[N,K]^T with fp32 accumulation in TMEM.
//
// Persistent, warp-specialised kernel (one CTA per SM):
//   warp 0     TMA producer: streams 128x64 A tiles and BNx64 B tiles (128-byte swizzle) through a 4-stage ring
//   warp 1     MMA issuer: one elected thread issues tcgen05.mma (M=128, N=BN, K=16) into one of two TMEM
//              accumulator buffers and commits stage/accumulator completion to mbarriers
//   warp 2     TMEM allocator
//   warps 4-7  epilogue: tcgen05.ld -> bf16 -> swizzled smem staging -> TMA store (overlaps the next tile's MMAs)
//
// Used directly as the building block of the tensor-parallel fused ops; there is no counterpart in the reference
// project, whose tensor-parallel hooks are disabled (tpSize = 1, src/cam/comm_operator/pybind/moe_dispatch_prefill.cpp:55).
#include "common.h"
#include "ptx.cuh"

namespace umdk {

namespace {

constexpr int BM = 128;
constexpr int BK = 64;  // 64 bf16 = one 128-byte swizzle atom
constexpr int kStages = 4;
constexpr int kThreads = 256;
constexpr int kEpiWarps = 4;
constexpr int kEpiChunkCols = 64;                       // bf16 columns per TMA-store box (128 bytes)
constexpr int kEpiBufBytes = 32 * kEpiChunkCols * 2;    // one warp's 32 rows x 64 cols

template <int BN>
struct Cfg {
  static constexpr int kABytes = BM * BK * 2;
  static constexpr int kBBytes = BN * BK * 2;
  static constexpr int kStageBytes = kABytes + kBBytes;
  static constexpr int kEpiBytes = kEpiWarps * 2 * kEpiBufBytes;
  static constexpr int kBarBytes = 256;
  static constexpr int kSmemBytes = kStages * kStageBytes + kEpiBytes + kBarBytes + 1024;
  static constexpr int kTmemCols = 2 * BN;  // two accumulator buffers (power of two: 256 or 512)
};

// Tile order: super-rows of kGroupM m-tiles are swept column by column, so that the ~148 tiles in flight at any time
// touch about 16 A panels and 9 B panels (tens of MB, L2-resident) instead of every A panel of the matrix.
constexpr int kGroupM = 16;
__device__ __forceinline__ void tile_to_mn(int t, int mb, int nb, int* m_blk, int* n_blk) {
  const int per_group = kGroupM * nb;
  const int g = t / per_group;
  const int first_m = g * kGroupM;
  const int gm = min(kGroupM, mb - first_m);
  const int r = t - g * per_group;
  *m_blk = first_m + r % gm;
  *n_blk = r / gm;
}

template <int BN>
__global__ void __launch_bounds__(kThreads, 1)
gemm_bf16_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                 const __grid_constant__ CUtensorMap tmC, int M, int N, int K, int* status) {
  using C = Cfg<BN>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* epi = smem + kStages * C::kStageBytes;
  uint64_t* bars = reinterpret_cast<uint64_t*>(epi + C::kEpiBytes);
  uint64_t* full = bars;
  uint64_t* empty = bars + kStages;
  uint64_t* tfull = bars + 2 * kStages;
  uint64_t* tempty = bars + 2 * kStages + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * kStages + 4);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int mb = (M + BM - 1) / BM;
  const int nb = (N + BN - 1) / BN;
  const int kb_total = (K + BK - 1) / BK;
  const int num_tiles = mb * nb;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&tfull[i], 1);
      mbar_init(&tempty[i], kEpiWarps);
    }
    mbar_fence_init();
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmB);
    tma_prefetch_desc(&tmC);
  }
  if (warp == 2) {
    tmem_alloc(tmem_slot, C::kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    if (elect_one()) {
      int s = 0;
      uint32_t ph = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
        int m_blk, n_blk;
        tile_to_mn(t, mb, nb, &m_blk, &n_blk);
        const int m0 = m_blk * BM, n0 = n_blk * BN;
        for (int kb = 0; kb < kb_total; ++kb) {
          if (!mbar_wait(&empty[s], ph ^ 1)) {
            umdk_set_status(status, UMDK_ERR_TIMEOUT, UMDK_PH_TMA_EMPTY, t, kb);
            ok = false;
            break;
          }
          mbar_expect_tx(&full[s], C::kStageBytes);
          uint8_t* sa = smem + s * C::kStageBytes;
          tma_load_2d(sa, &tmA, &full[s], kb * BK, m0);
          tma_load_2d(sa + C::kABytes, &tmB, &full[s], kb * BK, n0);
          if (++s == kStages) {
            s = 0;
            ph ^= 1;
          }
        }
      }
    }
  } else if (warp == 1) {
    if (elect_one()) {
      constexpr uint32_t idesc = umma_idesc(kFmtBF16, kFmtBF16, BM, BN);
      int s = 0;
      uint32_t ph = 0;
      int it = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x, ++it) {
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
          const uint32_t sa = smem_u32(smem + s * C::kStageBytes);
          const uint64_t adesc = umma_desc_k_sw128(sa);
          const uint64_t bdesc = umma_desc_k_sw128(sa + C::kABytes);
#pragma unroll
          for (int k = 0; k < BK / 16; ++k) {
            // 16 bf16 = 32 bytes per K step inside the swizzle atom: +2 in the (addr >> 4) field
            umma_f16(d_tmem, adesc + 2 * k, bdesc + 2 * k, idesc, (kb | k) != 0 ? 1u : 0u);
          }
          umma_commit(&empty[s]);
          if (++s == kStages) {
            s = 0;
            ph ^= 1;
          }
        }
        if (ok) umma_commit(&tfull[ab]);
      }
    }
  } else if (warp >= 4) {
    const int ew = warp - 4;  // == warp % 4: TMEM lanes [32*ew, 32*ew+32)
    uint8_t* my_epi = epi + ew * 2 * kEpiBufBytes;
    int it = 0;
    int buf = 0;
    for (int t = blockIdx.x; t < num_tiles; t += gridDim.x, ++it) {
      int m_blk, n_blk;
      tile_to_mn(t, mb, nb, &m_blk, &n_blk);
      const int m0 = m_blk * BM, n0 = n_blk * BN;
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
        if (lane == 0) tma_store_wait_read<1>();  // the buffer written two chunks ago has been read out
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
      if (lane == 0) mbar_arrive(&tempty[ab]);
    }
    if (lane == 0) tma_store_wait<0>();
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 2) {
    tc_fence_after();
    tmem_dealloc(tmem_base, C::kTmemCols);
  }
}

template <int BN>
int launch(const void* A, const void* B, void* Cp, int M, int N, int K, int lda, int ldb, int ldc, int* status,
           cudaStream_t stream, int max_ctas) {
  using C = Cfg<BN>;
  CUtensorMap tmA, tmB, tmC;
  if (make_tmap_2d(&tmA, TMAP_BF16, A, K, M, (uint64_t)lda * 2, BK, BM, TMAP_SW_128B)) return -UMDK_ERR_BAD_ARG;
  if (make_tmap_2d(&tmB, TMAP_BF16, B, K, N, (uint64_t)ldb * 2, BK, BN, TMAP_SW_128B)) return -UMDK_ERR_BAD_ARG;
  if (make_tmap_2d(&tmC, TMAP_BF16, Cp, N, M, (uint64_t)ldc * 2, kEpiChunkCols, 32, TMAP_SW_128B))
    return -UMDK_ERR_BAD_ARG;
  static bool attr_set = false;
  if (!attr_set) {
    UMDK_CUDA_CHECK(cudaFuncSetAttribute(gemm_bf16_kernel<BN>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         C::kSmemBytes));
    attr_set = true;
  }
  const int tiles = ((M + BM - 1) / BM) * ((N + BN - 1) / BN);
  int grid = sm_count();
  if (max_ctas > 0 && max_ctas < grid) grid = max_ctas;
  if (tiles < grid) grid = tiles;
  gemm_bf16_kernel<BN><<<grid, kThreads, C::kSmemBytes, stream>>>(tmA, tmB, tmC, M, N, K, status);
  UMDK_CUDA_CHECK(cudaGetLastError());
  return 0;
}

}  // namespace
}  // namespace umdk

// C[M,N] = A[M,K] * B[N,K]^T, all bf16 row-major with leading dimensions in elements (multiples of 8).
// `status` points to 4 ints of device memory (zeroed by the caller) that receive an error record when a bounded
// wait runs out. `max_ctas` <= 0 uses one CTA per SM.
UMDK_API int umdk_gemm_bf16(const void* A, const void* B, void* C, int M, int N, int K, int lda, int ldb, int ldc,
                            int* status, void* stream, int max_ctas) {
  if (M <= 0 || N <= 0 || K <= 0 || (lda % 8) || (ldb % 8) || (ldc % 8) || (N % 8)) return -UMDK_ERR_BAD_ARG;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (N % 256 == 0 || N > 1024) return umdk::launch<256>(A, B, C, M, N, K, lda, ldb, ldc, status, s, max_ctas);
  return umdk::launch<128>(A, B, C, M, N, K, lda, ldb, ldc, status, s, max_ctas);
}
