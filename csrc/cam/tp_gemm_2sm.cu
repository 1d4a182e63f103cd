// Tensor-parallel fused GEMM + collective kernels with CTA pairs (one `tcgen05.mma.cta_group::2` per 256 x 256
// output tile). Same protocol, heap layout and arguments as tp_gemm.cu - copy CTAs that gather peer shards for
// MODE 0, push epilogue + owner reduce for MODE 1 - with the main loop of gemm_bf16_2sm.cu: each CTA of a pair stages
// 128 rows of A and 128 rows of B per k-block and keeps its 128 x 256 half of the accumulator in its own TMEM.
// Needs Ts and N to be multiples of 256; other shapes run on the single-CTA kernel.
#include "tp_common.cuh"

#include <cuda_runtime.h>

namespace umdk {
namespace {

constexpr int BMH = 128;
constexpr int BNH = 128;
constexpr int BN = 256;
constexpr int BK = 64;
constexpr int kStages = 6;
constexpr int kThreads = kTpThreads;
constexpr int kABytes = BMH * BK * 2;
constexpr int kBBytes = BNH * BK * 2;
constexpr int kStageBytes = kABytes + kBBytes;
constexpr int kEpiBufBytes = 32 * 64 * 2;
constexpr int kEpiBytes = 4 * 2 * kEpiBufBytes;
constexpr int kSmemBytes = kStages * kStageBytes + kEpiBytes + 256 + 1024;
constexpr int kTmemCols = 512;

__global__ void __launch_bounds__(kThreads, 1)
tp_gemm_2sm_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                   const __grid_constant__ CUtensorMap tmC, const TpArgs a) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* epi = smem + kStages * kStageBytes;
  uint64_t* bars = reinterpret_cast<uint64_t*>(epi + kEpiBytes);
  uint64_t* full = bars;
  uint64_t* empty = bars + kStages;
  uint64_t* tfull = bars + 2 * kStages;
  uint64_t* tempty = tfull + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty + 2);
  __shared__ uint32_t s_epoch;
  __shared__ int s_ok;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    s_epoch = a.ctrl[0];
    s_ok = 1;
  }
  __syncthreads();
  const uint32_t epoch = s_epoch;
  const int slot = epoch & 1;
  const uint64_t tag = (uint64_t)epoch + 1;
  const int mb_per_chunk = a.Ts / (2 * BMH);
  const int nb = a.N / BN;
  const int kb_total = a.K / BK;
  const int num_tiles = a.R * mb_per_chunk * nb;
  const int n_copy = a.mode == 0 ? a.n_copy : 0;      // even: whole pairs take the copy role
  const bool is_copy_cta = (int)blockIdx.x < n_copy;

  if (a.mode == 0 && is_copy_cta) {
    // dedicated copy CTAs (whole pairs): the GEMM ring and barrier area serve as the bulk-copy ring
    tp_copy_role_bulk(a, n_copy, slot, tag, epoch, &s_ok, smem, bars);
  } else {
    const uint32_t cta = cluster_ctarank();
    const int pair = ((int)blockIdx.x - n_copy) >> 1;
    const int num_pairs = ((int)gridDim.x - n_copy) >> 1;
    if (threadIdx.x == 0) {
      for (int s = 0; s < kStages; ++s) {
        mbar_init(&full[s], 1);
        mbar_init(&empty[s], 1);
      }
      for (int i = 0; i < 2; ++i) {
        mbar_init(&tfull[i], 1);
        mbar_init(&tempty[i], 8);   // leader's copy: four epilogue warps of each CTA
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
    cluster_sync_all();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    const int my_tiles_end = (a.mode == 1 && !(a.phase_mask & 1)) ? 0 : num_tiles;
    // tile t -> chunk i = t / tiles_per_chunk (source / owner rank (rank + shift + i) % R; MODE 0 starts with the own
    // shard, MODE 1 ends with the own rows), 256-row block and 256-column block inside the chunk
    const int tiles_per_chunk = mb_per_chunk * nb;
    // inside a chunk, groups of kGroupM row blocks are swept column by column: the ~74 tiles in flight then share
    // 8 A panels and ~9 B panels, which stay in L2
    constexpr int kGroupM = 8;
    auto tile_coords = [&](int t, int* m0, int* n0, int* peer) {
      const int i = t / tiles_per_chunk, r = t - i * tiles_per_chunk;
      const int p = (a.rank + (a.mode == 0 ? 0 : 1) + i) % a.R;
      const int per_group = kGroupM * nb;
      const int g = r / per_group, rg = r - g * per_group;
      const int gm = min(kGroupM, mb_per_chunk - g * kGroupM);
      const int mblk = g * kGroupM + rg % gm, nblk = rg / gm;
      *peer = p;
      *m0 = (p * mb_per_chunk + mblk) * 2 * BMH + (int)cta * BMH;   // this CTA's 128 rows
      *n0 = nblk * BN;
    };

    if (warp == 0) {
      if (elect_one()) {
        int s = 0;
        uint32_t ph = 0;
        bool ok = true;
        int have_chunk = -1;
        for (int t = pair; t < my_tiles_end && ok; t += num_pairs) {
          int m0, n0, peer;
          tile_coords(t, &m0, &n0, &peer);
          if (a.mode == 0 && peer != have_chunk) {
            if (!wait_flag_ge_gpu(&a.chunk_done[peer], (uint32_t)tag * (uint32_t)n_copy)) {
              umdk_set_status(a.status, UMDK_ERR_TIMEOUT, UMDK_PH_AG_CHUNK, peer, t);
              break;
            }
            have_chunk = peer;
            fence_proxy_async_all();
          }
          for (int kb = 0; kb < kb_total; ++kb) {
            if (!mbar_wait(&empty[s], ph ^ 1)) {
              umdk_set_status(a.status, UMDK_ERR_TIMEOUT, UMDK_PH_TMA_EMPTY, t, kb);
              ok = false;
              break;
            }
            if (cta == 0) mbar_expect_tx(&full[s], 2 * kStageBytes);
            const uint32_t leader_full = map_to_cta(&full[s], 0);
            uint8_t* sa = smem + s * kStageBytes;
            tma_load_2d_pair(sa, &tmA, leader_full, kb * BK, m0);
            tma_load_2d_pair(sa + kABytes, &tmB, leader_full, kb * BK, n0 + (int)cta * BNH);
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
        for (int t = pair; t < my_tiles_end && ok; t += num_pairs, ++it) {
          const int ab = it & 1;
          const uint32_t aph = (it >> 1) & 1;
          if (!mbar_wait(&tempty[ab], aph ^ 1)) {
            umdk_set_status(a.status, UMDK_ERR_TIMEOUT, UMDK_PH_TMEM_EMPTY, t, 0);
            break;
          }
          tc_fence_after();
          const uint32_t d_tmem = tmem_base + ab * BN;
          for (int kb = 0; kb < kb_total; ++kb) {
            if (!mbar_wait(&full[s], ph)) {
              umdk_set_status(a.status, UMDK_ERR_TIMEOUT, UMDK_PH_TMA_FULL, t, kb);
              ok = false;
              break;
            }
            tc_fence_after();
            const uint32_t sa = smem_u32(smem + s * kStageBytes);
            const uint64_t adesc = umma_desc_k_sw128(sa);
            const uint64_t bdesc = umma_desc_k_sw128(sa + kABytes);
#pragma unroll
            for (int k = 0; k < BK / 16; ++k)
              umma_f16_pair(d_tmem, adesc + 2 * k, bdesc + 2 * k, idesc, (kb | k) ? 1u : 0u);
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
      int it = 0, buf = 0;
      for (int t = pair; t < my_tiles_end; t += num_pairs, ++it) {
        int m0, n0, peer;
        tile_coords(t, &m0, &n0, &peer);
        const int ab = it & 1;
        const uint32_t aph = (it >> 1) & 1;
        if (!mbar_wait(&tfull[ab], aph)) {
          umdk_set_status(a.status, UMDK_ERR_TIMEOUT, UMDK_PH_TMEM_FULL, t, 0);
          break;
        }
        tc_fence_after();
        const uint32_t t_addr = tmem_base + (static_cast<uint32_t>(ew * 32) << 16) + ab * BN;
        if (a.mode == 0) {
#pragma unroll 1
          for (int c = 0; c < BN / 64; ++c) {
            uint32_t r[64];
            tmem_ld_x32(t_addr + c * 64, r);
            tmem_ld_x32(t_addr + c * 64 + 32, r + 32);
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
              tma_store_2d(&tmC, my_epi + buf * kEpiBufBytes, n0 + c * 64, m0 + ew * 32);
              tma_store_commit();
            }
            buf ^= 1;
          }
        } else {
          // rows m0 + ew*32 .. +31 of the full result belong to rank `peer`. Each 32 x 64 chunk goes through the
          // warp's swizzled staging buffer so that the stores to the owner are whole 128-byte lines (4 rows per
          // instruction) instead of 32 scattered 16-byte pieces.
          const int lrow0 = m0 - peer * a.Ts + ew * 32;
          uint8_t* tile_base = a.peers.base[peer] + a.recv_off[slot] + (((size_t)a.rank * a.Ts + lrow0) * a.N + n0) * 2;
          uint8_t* stage = my_epi;
#pragma unroll 1
          for (int c = 0; c < BN / 64; ++c) {
            uint32_t r[64];
            tmem_ld_x32(t_addr + c * 64, r);
            tmem_ld_x32(t_addr + c * 64 + 32, r + 32);
            tmem_ld_wait();
            uint8_t* dst = stage + lane * 128;
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
            __syncwarp();
#pragma unroll
            for (int i = 0; i < 8; ++i) {
              const int row = i * 4 + (lane >> 3), seg = lane & 7;
              const int4 v = *reinterpret_cast<const int4*>(stage + row * 128 + ((seg ^ (row & 7)) << 4));
              st_na_v4(tile_base + (size_t)row * a.N * 2 + c * 128 + seg * 16, v);
            }
            __syncwarp();
          }
          __threadfence_system();
          __syncwarp();
          if (lane == 0) {
            red_add_release_sys(reinterpret_cast<uint32_t*>(a.peers.base[peer] + a.arrive_off) + a.rank, 1u);
          }
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive_cluster(map_to_cta(&tempty[ab], 0));
      }
      if (a.mode == 0 && lane == 0) tma_store_wait<0>();
    }
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();   // the peer may still signal this CTA's barriers or read its operands until here
    if (warp == 2) {
      tc_fence_after();
      tmem_dealloc_pair(tmem_base, kTmemCols);
    }

    if (a.mode == 1 && (a.phase_mask & 2)) {
      // per (source, owner): tiles x 2 CTAs x 4 epilogue warps
      tp_owner_reduce(a, (uint32_t)(mb_per_chunk * nb * 8), slot, tag, epoch, &s_ok);
    }
  }
  if (cta_done_is_last(&a.ctrl[1], gridDim.x)) {
    if (threadIdx.x == 0 && (a.phase_mask & 2)) a.ctrl[0] = epoch + 1;
  }
}

}  // namespace

// Launch of the CTA-pair kernel; called by umdk_tp_gemm when the shape allows. Returns 0 or a negative error.
int tp_gemm_2sm_launch(const TpArgs& a, const void* A, const void* w, void* out, int grid, cudaStream_t stream) {
  const int M = a.R * a.Ts;
  CUtensorMap tmA, tmB, tmC;
  if (make_tmap_2d(&tmA, TMAP_BF16, A, a.K, M, (uint64_t)a.K * 2, BK, BMH, TMAP_SW_128B)) return -UMDK_ERR_BAD_ARG;
  if (make_tmap_2d(&tmB, TMAP_BF16, w, a.K, a.N, (uint64_t)a.K * 2, BK, BNH, TMAP_SW_128B)) return -UMDK_ERR_BAD_ARG;
  if (make_tmap_2d(&tmC, TMAP_BF16, out, a.N, a.mode == 0 ? M : a.Ts, (uint64_t)a.N * 2, 64, 32, TMAP_SW_128B))
    return -UMDK_ERR_BAD_ARG;
  UMDK_CUDA_CHECK(cudaFuncSetAttribute(tp_gemm_2sm_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes));
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid, 1, 1);
  cfg.blockDim = dim3(kThreads, 1, 1);
  cfg.dynamicSmemBytes = kSmemBytes;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  UMDK_CUDA_CHECK(cudaLaunchKernelEx(&cfg, tp_gemm_2sm_kernel, tmA, tmB, tmC, a));
  return 0;
}

}  // namespace umdk
