// Tensor-parallel fused GEMM + collective kernels on tcgen05 tensor cores, over NVLink peer memory.
//
//   MODE 0  all-gather -> GEMM   Y[R*Ts, N] = gather_r(X_r[Ts, K]) * W[N, K]^T
//           A few "copy" CTAs of the SAME kernel pull the peers' activation shards over NVLink into a local
//           gathered buffer (16-byte loads from peer memory, local stores) chunk by chunk and raise a per-chunk
//           counter; the GEMM CTAs walk the output tiles in chunk order (own shard first, then rank+1, ...) and
//           their TMA producer waits - bounded - for the chunk's counter before loading A tiles, so the transfer
//           of chunk i+1 hides behind the MMAs of chunk i. TMA only ever reads local memory.
//   MODE 1  GEMM -> reduce-scatter   out[Ts, N] = sum_r P_r[rank*Ts .. , N],  P_r = Y_r[R*Ts, Kr] * W_r[N, Kr]^T
//           The epilogue stores each bf16 output tile straight into the row owner's receive slot [src rank] over
//           NVLink (tiles for rank+1 first, own rows last) and bumps the owner's arrival counter with a
//           system-scope release; after its tiles every CTA waits for all sources and reduces its share of the
//           owned rows in fp32.
// Both build on the same persistent warp-specialised pipeline as gemm_bf16.cu (TMA producer warp, single-thread MMA
// issuer, double-buffered TMEM accumulators, 4 epilogue warps). Shards sit in the symmetric heap, double-buffered on
// an epoch counter kept in device memory, so back-to-back calls need no host-side barrier.
// The reference has no tensor-parallel operator (its TP hooks are compiled out, tpSize = 1 in
// src/cam/comm_operator/pybind/moe_dispatch_prefill.cpp:55-56); these kernels implement the tensor-parallel part of
// the serving configuration.
#include "tp_common.cuh"

namespace umdk {
namespace {

constexpr int BM = 128;
constexpr int BN = 256;
constexpr int BK = 64;
constexpr int kStages = 4;
constexpr int kThreads = kTpThreads;
constexpr int kABytes = BM * BK * 2;
constexpr int kBBytes = BN * BK * 2;
constexpr int kStageBytes = kABytes + kBBytes;
constexpr int kEpiBufBytes = 32 * 64 * 2;
constexpr int kEpiBytes = 4 * 2 * kEpiBufBytes;
constexpr int kSmemBytes = kStages * kStageBytes + kEpiBytes + 256 + 1024;
constexpr int kTmemCols = 2 * BN;

__global__ void __launch_bounds__(kThreads, 1)
tp_gemm_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
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
  const int M = a.R * a.Ts;
  const int mb_per_chunk = a.Ts / BM;
  const int nb = a.N / BN;
  const int kb_total = a.K / BK;
  const int num_tiles = (M / BM) * nb;
  const int n_copy = a.mode == 0 ? a.n_copy : 0;
  const bool is_copy_cta = (int)blockIdx.x < n_copy;
  const int gemm_cta = blockIdx.x - n_copy;
  const int gemm_ctas = gridDim.x - n_copy;
  if (a.phase_mask == 4) {  // publish only: one CTA copies the shard into its slot and raises the flags
    const size_t shard_vec = (size_t)a.Ts * a.K * 2 / 16;
    const int4* from = reinterpret_cast<const int4*>(a.x_local);
    int4* to = reinterpret_cast<int4*>(a.peers.base[a.rank] + a.x_slot_off[slot]);
    for (size_t v = threadIdx.x; v < shard_vec; v += kThreads) to[v] = from[v];
    __threadfence_system();
    __syncthreads();
    if (threadIdx.x < a.R) {
      st_release_sys(reinterpret_cast<uint64_t*>(a.peers.base[threadIdx.x] + a.ready_off[slot]) + a.rank, tag);
    }
    return;
  }

  if (a.mode == 0 && is_copy_cta) {
    tp_copy_role(a, n_copy, slot, tag, epoch, &s_ok);
  } else {
    // ---------------------------------------------------------------- GEMM role
    if (threadIdx.x == 0) {
      for (int s = 0; s < kStages; ++s) {
        mbar_init(&full[s], 1);
        mbar_init(&empty[s], 1);
      }
      for (int i = 0; i < 2; ++i) {
        mbar_init(&tfull[i], 1);
        mbar_init(&tempty[i], 4);
      }
      mbar_fence_init();
      tma_prefetch_desc(&tmA);
      tma_prefetch_desc(&tmB);
      tma_prefetch_desc(&tmC);
    }
    if (warp == 2) {
      tmem_alloc(tmem_slot, kTmemCols);
      tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    const int my_tiles_end = (a.mode == 1 && !(a.phase_mask & 1)) ? 0 : num_tiles;
    // tile t -> chunk index i = t / tiles_per_chunk; chunk's source / owner rank = (rank + shift + i) % R, where
    // MODE 0 starts with the own shard (shift 0) and MODE 1 ends with the own rows (shift 1)
    const int tiles_per_chunk = mb_per_chunk * nb;
    auto tile_coords = [&](int t, int* m0, int* n0, int* peer) {
      const int i = t / tiles_per_chunk, r = t - i * tiles_per_chunk;
      const int p = (a.rank + (a.mode == 0 ? 0 : 1) + i) % a.R;
      *peer = p;
      *m0 = (p * mb_per_chunk + r % mb_per_chunk) * BM;
      *n0 = (r / mb_per_chunk) * BN;
    };

    if (warp == 0) {
      if (elect_one()) {
        int s = 0;
        uint32_t ph = 0;
        bool ok = true;
        int have_chunk = -1;
        for (int t = gemm_cta; t < my_tiles_end && ok; t += gemm_ctas) {
          int m0, n0, peer;
          tile_coords(t, &m0, &n0, &peer);
          if (a.mode == 0 && peer != have_chunk) {
            if (!wait_flag_ge_gpu(&a.chunk_done[peer], (uint32_t)tag * (uint32_t)n_copy)) {
              umdk_set_status(a.status, UMDK_ERR_TIMEOUT, UMDK_PH_AG_CHUNK, peer, t);
              break;
            }
            have_chunk = peer;
            fence_proxy_async_all();  // generic-proxy writes of the copy CTAs -> async-proxy (TMA) reads
          }
          for (int kb = 0; kb < kb_total; ++kb) {
            if (!mbar_wait(&empty[s], ph ^ 1)) {
              umdk_set_status(a.status, UMDK_ERR_TIMEOUT, UMDK_PH_TMA_EMPTY, t, kb);
              ok = false;
              break;
            }
            mbar_expect_tx(&full[s], kStageBytes);
            uint8_t* sa = smem + s * kStageBytes;
            tma_load_2d(sa, &tmA, &full[s], kb * BK, m0);
            tma_load_2d(sa + kABytes, &tmB, &full[s], kb * BK, n0);
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
        for (int t = gemm_cta; t < my_tiles_end && ok; t += gemm_ctas, ++it) {
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
            for (int k = 0; k < BK / 16; ++k) umma_f16(d_tmem, adesc + 2 * k, bdesc + 2 * k, idesc, (kb | k) ? 1u : 0u);
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
      const int ew = warp - 4;
      uint8_t* my_epi = epi + ew * 2 * kEpiBufBytes;
      int it = 0, buf = 0;
      for (int t = gemm_cta; t < my_tiles_end; t += gemm_ctas, ++it) {
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
          // rows m0 + ew*32 + lane of the full result belong to rank `peer`; local row inside its shard:
          const int lrow = m0 - peer * a.Ts + ew * 32 + lane;
          uint8_t* rowp = a.peers.base[peer] + a.recv_off[slot] + (((size_t)a.rank * a.Ts + lrow) * a.N + n0) * 2;
#pragma unroll 1
          for (int c = 0; c < BN / 32; ++c) {
            uint32_t r[32];
            tmem_ld_x32(t_addr + c * 32, r);
            tmem_ld_wait();
#pragma unroll
            for (int q = 0; q < 4; ++q) {
              int4 o;
              __nv_bfloat162* po = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
              for (int i = 0; i < 4; ++i)
                po[i] = __floats2bfloat162_rn(__uint_as_float(r[q * 8 + 2 * i]), __uint_as_float(r[q * 8 + 2 * i + 1]));
              st_na_v4(rowp + c * 64 + q * 16, o);
            }
          }
          __threadfence_system();
          __syncwarp();
          if (lane == 0) {
            red_add_release_sys(reinterpret_cast<uint32_t*>(a.peers.base[peer] + a.arrive_off) + a.rank, 1u);
          }
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&tempty[ab]);
      }
      if (a.mode == 0 && lane == 0) tma_store_wait<0>();
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 2) {
      tc_fence_after();
      tmem_dealloc(tmem_base, kTmemCols);
    }

    if (a.mode == 1 && (a.phase_mask & 2)) {
      tp_owner_reduce(a, (uint32_t)(mb_per_chunk * nb * 4), slot, tag, epoch, &s_ok);
    }
  }
  if (cta_done_is_last(&a.ctrl[1], gridDim.x)) {
    if (threadIdx.x == 0 && (a.phase_mask & 2)) a.ctrl[0] = epoch + 1;
  }
}

}  // namespace
}  // namespace umdk

namespace umdk {
int tp_gemm_2sm_launch(const TpArgs& a, const void* A, const void* w, void* out, int grid, cudaStream_t stream);
}
using namespace umdk;

struct UmdkTpGemmParams {
  int mode, R, rank, Ts, N, K, n_copy, max_ctas;
  void* peers[kMaxRanks];
  uint64_t x_slot_off[2];
  uint64_t ready_off[2];
  uint64_t recv_off[2];
  uint64_t arrive_off;
  const void* a_local;   // MODE 1: this rank's A operand [R*Ts, K]; MODE 0: this rank's shard [Ts, K] (local memory)
  void* xg;              // MODE 0: gathered activations [R*Ts, K] (local memory)
  const void* w;         // [N, K]
  void* out;             // MODE 0: [R*Ts, N]; MODE 1: [Ts, N]
  uint32_t* chunk_done;  // MODE 0: [R] local counters
  uint32_t* ctrl;        // [0] epoch, [1] done counter
  int* status;
  int phase_mask;        // 0 = 3 (everything); see TpArgs
  int impl;              // 0 = CTA pairs where the shape allows (Ts and N multiples of 256), 1 = one CTA per tile
};

// Symmetric-heap bytes a rank needs: MODE 0 regions (two shards + flags) followed by MODE 1 regions.
UMDK_API long long umdk_tp_heap_bytes(int R, int Ts, int K_ag, int N_rs) {
  if (R < 1 || R > kMaxRanks || Ts < 128 || (Ts % 128)) return -1;
  uint64_t off = 0;
  off += 2 * align_up_u64((uint64_t)Ts * K_ag * 2, 1024);
  off += 2 * align_up_u64((uint64_t)R * 8, 256);
  off += 2 * align_up_u64((uint64_t)R * Ts * N_rs * 2, 1024);
  off += align_up_u64((uint64_t)R * 4, 256);
  return (long long)off;
}

UMDK_API int umdk_tp_gemm(const UmdkTpGemmParams* p, void* stream) {
  if (p->R < 1 || p->R > kMaxRanks || p->Ts < BM || (p->Ts % BM) || (p->N % BN) || (p->K % BK) || p->N < BN ||
      p->K < BK || (p->mode != 0 && p->mode != 1))
    return -UMDK_ERR_BAD_ARG;
  TpArgs a;
  a.mode = p->mode;
  a.R = p->R;
  a.rank = p->rank;
  a.Ts = p->Ts;
  a.N = p->N;
  a.K = p->K;
  a.n_copy = p->mode == 0 ? (p->n_copy > 0 ? p->n_copy : 16) : 0;
  for (int i = 0; i < kMaxRanks; ++i) a.peers.base[i] = i < p->R ? static_cast<uint8_t*>(p->peers[i]) : nullptr;
  a.x_slot_off[0] = p->x_slot_off[0];
  a.x_slot_off[1] = p->x_slot_off[1];
  a.ready_off[0] = p->ready_off[0];
  a.ready_off[1] = p->ready_off[1];
  a.x_local = static_cast<const __nv_bfloat16*>(p->a_local);
  a.xg = static_cast<__nv_bfloat16*>(p->xg);
  a.chunk_done = p->chunk_done;
  a.recv_off[0] = p->recv_off[0];
  a.recv_off[1] = p->recv_off[1];
  a.arrive_off = p->arrive_off;
  a.out = static_cast<__nv_bfloat16*>(p->out);
  a.ctrl = p->ctrl;
  a.status = p->status;
  a.phase_mask = p->phase_mask ? p->phase_mask : 3;
  const int M = p->R * p->Ts;
  const void* A = p->mode == 0 ? p->xg : p->a_local;
  if (p->impl == 0 && a.phase_mask != 4 && (p->Ts % 256) == 0 && (p->N % 256) == 0) {
    int grid = sm_count();
    if (p->max_ctas > 0 && p->max_ctas < grid) grid = p->max_ctas;
    grid &= ~1;
    // whole pairs take the copy role; the bulk-copy engine needs few of them (default 4 pairs)
    a.n_copy = p->n_copy > 0 ? ((p->n_copy + 1) & ~1) : 8;
    if (grid <= a.n_copy + 1) return -UMDK_ERR_BAD_ARG;
    return tp_gemm_2sm_launch(a, A, p->w, p->out, grid, static_cast<cudaStream_t>(stream));
  }
  CUtensorMap tmA, tmB, tmC;
  if (make_tmap_2d(&tmA, TMAP_BF16, A, p->K, M, (uint64_t)p->K * 2, BK, BM, TMAP_SW_128B)) return -UMDK_ERR_BAD_ARG;
  if (make_tmap_2d(&tmB, TMAP_BF16, p->w, p->K, p->N, (uint64_t)p->K * 2, BK, BN, TMAP_SW_128B))
    return -UMDK_ERR_BAD_ARG;
  // MODE 1 never stores through TMA; the map still has to be valid, so it points at the small local output
  if (make_tmap_2d(&tmC, TMAP_BF16, p->out, p->N, p->mode == 0 ? M : p->Ts, (uint64_t)p->N * 2, 64, 32, TMAP_SW_128B))
    return -UMDK_ERR_BAD_ARG;
  static bool attr = false;
  if (!attr) {
    UMDK_CUDA_CHECK(cudaFuncSetAttribute(tp_gemm_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes));
    attr = true;
  }
  int grid = sm_count();  // CTAs wait on each other and on peers: the whole grid has to be resident
  if (p->max_ctas > 0 && p->max_ctas < grid) grid = p->max_ctas;
  if (grid <= a.n_copy) return -UMDK_ERR_BAD_ARG;
  if (a.phase_mask == 4) grid = 1;
  tp_gemm_kernel<<<grid, kThreads, kSmemBytes, static_cast<cudaStream_t>(stream)>>>(tmA, tmB, tmC, a);
  UMDK_CUDA_CHECK(cudaGetLastError());
  return 0;
}
