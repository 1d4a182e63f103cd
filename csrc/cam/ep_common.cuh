// Geometry and symmetric-heap layout shared by the expert-parallel (EP) dispatch/combine kernels.
#pragma once
#include "common.h"

namespace umdk {

constexpr int kMaxRanks = 32;    // one box: peers are addressed through a 32-bit rank mask
constexpr int kMaxTopk = 16;     // same limit as the reference's prefill path (CAM API Guide: top-k <= 16)

struct EpGeom {
  int R;          // ranks in the EP group
  int rank;       // this rank
  int E;          // global routed experts
  int E_local;    // experts per rank
  int K;          // top-k
  int H;          // hidden size (elements)
  int cap;        // max tokens any rank sends in one call (per-source capacity of the arrival buffers)
  int quant;      // 1: fp8 e4m3 payload with fp32 scale per 1x128 block; 0: bf16 payload
  int row_bytes;  // payload bytes per token on the wire
  int nscale;     // H / 128 (0 when quant == 0)
  int meta_words; // int32 words of per-token metadata on the wire
  int J;          // combine slots per token on the owner (max(R, K))
};

__host__ __device__ inline uint64_t align_up_u64(uint64_t x, uint64_t a) { return (x + a - 1) / a * a; }

// Byte offsets inside every rank's symmetric heap. Index [h] selects the ping-pong half (epoch parity).
struct EpNormalOffsets {
  uint64_t notify[2];       // [R src][E_local + 4] int32
  uint64_t notify_flag[2];  // [R] uint64
  uint64_t data_flag[2];    // [R] uint64
  uint64_t comb_flag[2];    // [R] uint64
  uint64_t arr_x[2];        // [R][cap][row_bytes]
  uint64_t arr_scale[2];    // [R][cap][nscale] fp32
  uint64_t arr_meta[2];     // [R][cap][meta_words] int32
  uint64_t comb_buf[2];     // [cap][J][H] bf16
  uint64_t snotify[2];      // standalone notify op: [R src][E_local + 4] int32
  uint64_t snotify_flag[2]; // [R] uint64
  uint64_t stage_x;         // [cap][H] fp8: this rank's quantised tokens, read by its own per-destination passes
  uint64_t stage_scale;     // [cap][H / 128] fp32
  uint64_t total;
};

__host__ __device__ inline int ep_meta_words(int K) { return ((2 * K + 2) + 3) / 4 * 4; }
__host__ __device__ inline int ep_notify_words(int E_local) { return E_local + 4; }

__host__ __device__ inline EpNormalOffsets ep_normal_offsets(const EpGeom& g) {
  EpNormalOffsets o;
  uint64_t off = 0;
  for (int h = 0; h < 2; ++h) {
    o.notify[h] = off;
    off = align_up_u64(off + (uint64_t)g.R * ep_notify_words(g.E_local) * 4, 256);
    o.notify_flag[h] = off;
    off = align_up_u64(off + (uint64_t)g.R * 8, 256);
    o.data_flag[h] = off;
    off = align_up_u64(off + (uint64_t)g.R * 8, 256);
    o.comb_flag[h] = off;
    off = align_up_u64(off + (uint64_t)g.R * 8, 256);
  }
  for (int h = 0; h < 2; ++h) {
    o.arr_x[h] = off;
    off = align_up_u64(off + (uint64_t)g.R * g.cap * g.row_bytes, 256);
    o.arr_scale[h] = off;
    off = align_up_u64(off + (uint64_t)g.R * g.cap * (g.nscale > 0 ? g.nscale : 1) * 4, 256);
    o.arr_meta[h] = off;
    off = align_up_u64(off + (uint64_t)g.R * g.cap * g.meta_words * 4, 256);
    o.comb_buf[h] = off;
    off = align_up_u64(off + (uint64_t)g.cap * g.J * g.H * 2, 256);
  }
  for (int h = 0; h < 2; ++h) {
    o.snotify[h] = off;
    off = align_up_u64(off + (uint64_t)g.R * ep_notify_words(g.E_local) * 4, 256);
    o.snotify_flag[h] = off;
    off = align_up_u64(off + (uint64_t)g.R * 8, 256);
  }
  o.stage_x = off;
  off = align_up_u64(off + (uint64_t)g.cap * g.H, 256);
  o.stage_scale = off;
  off = align_up_u64(off + (uint64_t)g.cap * (g.H / 128) * 4, 256);
  o.total = off;
  return o;
}

// Low-latency (decode) layout. Rows are pushed straight to their final position in an expert-major slab, so the
// slab is directly the activation operand of the grouped GEMM.
struct EpLLGeom {
  int R, rank, E, E_local, K, H, T_cap;
  int n_cap;   // rows of the receive slab: R * T_cap * min(K, E_local)
};

struct EpLLOffsets {
  uint64_t cnt[2];        // [R src][E] int32: every rank's per-expert token counts (all-gathered)
  uint64_t cnt_flag[2];   // [R] uint64
  uint64_t data_flag[2];  // [R] uint64
  uint64_t comb_flag[2];  // [R] uint64
  uint64_t exp_cnt[2];    // [E_local] uint32: row parts that have landed per local expert in the running call (every
                          // sender adds one per 2 KiB part it stored; the receiver zeroes the words when it ends the call,
                          // before it raises the combine flags that let the senders start the next one)
  uint64_t slab_x[2];     // [n_cap][H] fp8
  uint64_t slab_s[2];     // [n_cap][H/128] fp32
  uint64_t slab_meta[2];  // [n_cap][2] int32: owner rank, owner slot (token * K + k)
  uint64_t comb_buf[2];   // [T_cap][K][H] bf16
  uint64_t total;
};

__host__ __device__ inline int ep_ll_n_cap(int R, int T_cap, int K, int E_local) {
  return R * T_cap * (K < E_local ? K : E_local);
}

__host__ __device__ inline EpLLOffsets ep_ll_offsets(const EpLLGeom& g) {
  // Single-buffered: a rank can only start call n+1 after it has received every peer's combine flags of call n,
  // i.e. after every peer has finished reading its slab and combine buffer of call n. Both halves alias.
  EpLLOffsets o;
  uint64_t off = 0;
  for (int h = 0; h < 1; ++h) {
    o.cnt[h] = off;
    off = align_up_u64(off + (uint64_t)g.R * g.E * 4, 256);
    o.cnt_flag[h] = off;
    off = align_up_u64(off + (uint64_t)g.R * 8, 256);
    o.data_flag[h] = off;
    off = align_up_u64(off + (uint64_t)g.R * 8, 256);
    o.comb_flag[h] = off;
    off = align_up_u64(off + (uint64_t)g.R * 8, 256);
    o.exp_cnt[h] = off;
    off = align_up_u64(off + (uint64_t)g.E_local * 4, 256);
  }
  for (int h = 0; h < 1; ++h) {
    o.slab_x[h] = off;
    off = align_up_u64(off + (uint64_t)g.n_cap * g.H, 1024);
    o.slab_s[h] = off;
    off = align_up_u64(off + (uint64_t)g.n_cap * (g.H / 128) * 4, 256);
    o.slab_meta[h] = off;
    off = align_up_u64(off + (uint64_t)g.n_cap * 8, 256);
    o.comb_buf[h] = off;
    off = align_up_u64(off + (uint64_t)g.T_cap * g.K * g.H * 2, 1024);
  }
  o.cnt[1] = o.cnt[0];
  o.cnt_flag[1] = o.cnt_flag[0];
  o.data_flag[1] = o.data_flag[0];
  o.comb_flag[1] = o.comb_flag[0];
  o.exp_cnt[1] = o.exp_cnt[0];
  o.slab_x[1] = o.slab_x[0];
  o.slab_s[1] = o.slab_s[0];
  o.slab_meta[1] = o.slab_meta[0];
  o.comb_buf[1] = o.comb_buf[0];
  o.total = off;
  return o;
}

// Checks and fills the low-latency geometry; 0 on success.
inline int fill_ll_geom(EpLLGeom* g, int R, int rank, int E, int K, int H, int T_cap) {
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

// 2 KiB parts per slab row: the unit in which the low-latency dispatch stores rows and counts their arrival.
__host__ __device__ inline int ep_ll_row_parts(int H) { return (H / 128 + 15) / 16; }

struct PeerTable {
  uint8_t* base[kMaxRanks];
};

}  // namespace umdk
