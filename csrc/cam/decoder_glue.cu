// Small fused kernels between the GEMMs of the MLA + MoE decode step: each replaces a chain of element-wise
// framework launches (residual adds, RMSNorm, rotary embedding, concatenation, KV-page write, router softmax + top-k +
// renormalisation + expert renumbering) with one launch that touches its rows once. bf16 in and out, fp32 math.
// The reference project has no model code; these serve the serving benchmark's decoder (models/dsv3_decoder.py).
#include "common.h"

#include <cuda_bf16.h>

namespace umdk {
namespace {

constexpr int kNormThreads = 256;
constexpr int kMaxVecPerThread = 4;   // 8 bf16 per vector: rows of up to 8192 elements

__device__ __forceinline__ float block_sum(float v, float* red) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  __syncthreads();
  if (lane == 0) red[warp] = v;
  __syncthreads();
  float t = 0.f;
  for (int i = 0; i < (int)(blockDim.x >> 5); ++i) t += red[i];
  return t;
}

__device__ __forceinline__ void unpack8(const uint4& u, float* f) {
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 t = __bfloat1622float2(h[i]);
    f[2 * i] = t.x;
    f[2 * i + 1] = t.y;
  }
}
__device__ __forceinline__ uint4 pack8(const float* f) {
  uint4 u;
  __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&u);
#pragma unroll
  for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
  return u;
}

// x_out[t] = x_in[t] (+ a[t]) (+ b[t]);  h[t] = x_out[t] * rsqrt(mean(x_out[t]^2) + eps) * w.   One CTA per row.
// x_out may be null (nothing added, nothing written back) and may alias x_in.
__global__ void __launch_bounds__(kNormThreads)
add_rmsnorm_kernel(const __nv_bfloat16* __restrict__ x_in, const __nv_bfloat16* __restrict__ a,
                   const __nv_bfloat16* __restrict__ b, const __nv_bfloat16* __restrict__ w,
                   __nv_bfloat16* x_out, __nv_bfloat16* __restrict__ h, int H, int ld_in, float eps) {
  __shared__ float red[kNormThreads / 32];
  const int t = blockIdx.x;
  const int nvec = H >> 3;
  float v[kMaxVecPerThread][8];
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < kMaxVecPerThread; ++i) {
    const int j = threadIdx.x + i * kNormThreads;
    if (j < nvec) {
      unpack8(reinterpret_cast<const uint4*>(x_in + (size_t)t * ld_in)[j], v[i]);
      float e[8];
      if (a != nullptr) {
        unpack8(reinterpret_cast<const uint4*>(a + (size_t)t * H)[j], e);
#pragma unroll
        for (int q = 0; q < 8; ++q) v[i][q] += e[q];
      }
      if (b != nullptr) {
        unpack8(reinterpret_cast<const uint4*>(b + (size_t)t * H)[j], e);
#pragma unroll
        for (int q = 0; q < 8; ++q) v[i][q] += e[q];
      }
      if (x_out != nullptr) {
        const uint4 u = pack8(v[i]);
        reinterpret_cast<uint4*>(x_out + (size_t)t * H)[j] = u;
        unpack8(u, v[i]);   // the norm sees the rounded residual, as a separate kernel would
      }
#pragma unroll
      for (int q = 0; q < 8; ++q) ss += v[i][q] * v[i][q];
    }
  }
  const float inv = rsqrtf(block_sum(ss, red) / (float)H + eps);
#pragma unroll
  for (int i = 0; i < kMaxVecPerThread; ++i) {
    const int j = threadIdx.x + i * kNormThreads;
    if (j < nvec) {
      float g[8];
      unpack8(reinterpret_cast<const uint4*>(w)[j], g);
#pragma unroll
      for (int q = 0; q < 8; ++q) v[i][q] = v[i][q] * inv * g[q];
      reinterpret_cast<uint4*>(h + (size_t)t * H)[j] = pack8(v[i]);
    }
  }
}

// After the fused q_a / kv_a projection: row t of `qkv` is [q_lora | 512 latent | 64 rope].
//   blockIdx.y == 0: qa[t] = rmsnorm(qkv[t, :q_lora]) * q_norm
//   blockIdx.y == 1: kv_pool row new_row[t] = [ rmsnorm(latent) * kv_norm | rope(rope part) ]  (the token's KV entry)
// Rotary pairs are interleaved (2i, 2i+1) and share one position (cos / sin [32]).
__global__ void __launch_bounds__(kNormThreads)
qkv_post_kernel(const __nv_bfloat16* __restrict__ qkv, int q_lora, const __nv_bfloat16* __restrict__ q_norm,
                const __nv_bfloat16* __restrict__ kv_norm, const float* __restrict__ cos_t,
                const float* __restrict__ sin_t, __nv_bfloat16* __restrict__ qa, __nv_bfloat16* __restrict__ kv_pool,
                const long long* __restrict__ new_row, long long pool_rows, float eps, int* status) {
  __shared__ float red[kNormThreads / 32];
  const int t = blockIdx.x;
  const int ld = q_lora + 576;
  const __nv_bfloat16* row = qkv + (size_t)t * ld;
  if (blockIdx.y == 0) {
    const int nvec = q_lora >> 3;
    float v[kMaxVecPerThread][8];
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < kMaxVecPerThread; ++i) {
      const int j = threadIdx.x + i * kNormThreads;
      if (j < nvec) {
        unpack8(reinterpret_cast<const uint4*>(row)[j], v[i]);
#pragma unroll
        for (int q = 0; q < 8; ++q) ss += v[i][q] * v[i][q];
      }
    }
    const float inv = rsqrtf(block_sum(ss, red) / (float)q_lora + eps);
#pragma unroll
    for (int i = 0; i < kMaxVecPerThread; ++i) {
      const int j = threadIdx.x + i * kNormThreads;
      if (j < nvec) {
        float g[8];
        unpack8(reinterpret_cast<const uint4*>(q_norm)[j], g);
#pragma unroll
        for (int q = 0; q < 8; ++q) v[i][q] = v[i][q] * inv * g[q];
        reinterpret_cast<uint4*>(qa + (size_t)t * q_lora)[j] = pack8(v[i]);
      }
    }
    return;
  }
  const long long dst_row = new_row[t];
  const bool ok = dst_row >= 0 && dst_row < pool_rows;
  if (!ok && threadIdx.x == 0) umdk_set_status(status, UMDK_ERR_OVERFLOW, UMDK_PH_NONE, t, (int)dst_row);
  const __nv_bfloat16* lat = row + q_lora;   // q_lora is a multiple of 8, so this stays 16-byte aligned
  float v[8];
  float ss = 0.f;
  const int j = threadIdx.x;   // 64 latent vectors + 8 rope vectors
  if (j < 64) {
    unpack8(reinterpret_cast<const uint4*>(lat)[j], v);
#pragma unroll
    for (int q = 0; q < 8; ++q) ss += v[q] * v[q];
  }
  const float inv = rsqrtf(block_sum(ss, red) / 512.f + eps);
  if (!ok) return;
  __nv_bfloat16* dst = kv_pool + (size_t)dst_row * 576;
  if (j < 64) {
    float g[8];
    unpack8(reinterpret_cast<const uint4*>(kv_norm)[j], g);
#pragma unroll
    for (int q = 0; q < 8; ++q) v[q] = v[q] * inv * g[q];
    reinterpret_cast<uint4*>(dst)[j] = pack8(v);
  } else if (j < 72) {
    unpack8(reinterpret_cast<const uint4*>(lat)[j], v);
    float r[8];
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      const int pair = (j - 64) * 4 + q;
      const float c = cos_t[pair], s = sin_t[pair];
      r[2 * q] = v[2 * q] * c - v[2 * q + 1] * s;
      r[2 * q + 1] = v[2 * q] * s + v[2 * q + 1] * c;
    }
    reinterpret_cast<uint4*>(dst)[j] = pack8(r);
  }
}

// q_full[t, h, 512:576] = rope(q[t, h, nope:nope+64]); the latent part [.., :512] is written by the absorbing GEMM.
// One thread per (t, h, 8-element vector).
__global__ void q_rope_kernel(const __nv_bfloat16* __restrict__ q, int q_head_dim, int nope,
                              const float* __restrict__ cos_t, const float* __restrict__ sin_t,
                              __nv_bfloat16* __restrict__ q_full, int rows) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= rows * 8) return;
  const int r = i >> 3, j = i & 7;
  float v[8], o[8];
  unpack8(reinterpret_cast<const uint4*>(q + (size_t)r * q_head_dim + nope)[j], v);
#pragma unroll
  for (int p = 0; p < 4; ++p) {
    const float c = cos_t[j * 4 + p], s = sin_t[j * 4 + p];
    o[2 * p] = v[2 * p] * c - v[2 * p + 1] * s;
    o[2 * p + 1] = v[2 * p] * s + v[2 * p + 1] * c;
  }
  reinterpret_cast<uint4*>(q_full + (size_t)r * 576 + 512)[j] = pack8(o);
}

// Router: softmax over E logits, top-K, weights renormalised over the K winners. One warp per token.
// With fold_el > 0 the expert ids are renumbered for a layout in which every rank owns fold_el routed experts followed
// by one shared expert (id' = id + id / fold_el), and a (K+1)-th slot selects this rank's shared expert with weight 1.
constexpr int kRouterMaxPerLane = 32;   // E <= 1024
template <int PER>   // experts per lane, E <= 32 * PER
__global__ void __launch_bounds__(128)
router_topk_kernel(const __nv_bfloat16* __restrict__ logits, int T, int E, int K, int fold_el, int rank,
                   long long* __restrict__ idx_out, float* __restrict__ w_out) {
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  if (warp >= T) return;
  float v[PER];
  float mx = -INFINITY;
#pragma unroll
  for (int i = 0; i < PER; ++i) {
    const int e = i * 32 + lane;
    v[i] = e < E ? __bfloat162float(logits[(size_t)warp * E + e]) : -INFINITY;
    mx = fmaxf(mx, v[i]);
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
  const int Ko = K + (fold_el > 0 ? 1 : 0);
  float wsum = 0.f;
  float my_w = 0.f;      // lane k keeps the k-th winner
  int my_e = -1;
  for (int k = 0; k < K; ++k) {
    float best = -INFINITY;
    int be = 0x7fffffff;
#pragma unroll
    for (int i = 0; i < PER; ++i) {
      const int e = i * 32 + lane;
      if (v[i] > best) {   // ascending e inside a lane: ties keep the lower index
        best = v[i];
        be = e;
      }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, best, o);
      const int oe = __shfl_xor_sync(0xffffffffu, be, o);
      if (ob > best || (ob == best && oe < be)) {
        best = ob;
        be = oe;
      }
    }
    const float p = __expf(best - mx);
    wsum += p;
    if (lane == k) {
      my_w = p;
      my_e = be;
    }
    if ((be & 31) == lane) {
#pragma unroll
      for (int i = 0; i < PER; ++i)
        if (i == (be >> 5)) v[i] = -INFINITY;
    }
  }
  if (lane < K) {
    const int e = fold_el > 0 ? my_e + my_e / fold_el : my_e;
    idx_out[(size_t)warp * Ko + lane] = e;
    w_out[(size_t)warp * Ko + lane] = my_w / wsum;
  } else if (lane == K && fold_el > 0) {
    idx_out[(size_t)warp * Ko + K] = (long long)rank * (fold_el + 1) + fold_el;
    w_out[(size_t)warp * Ko + K] = 1.f;
  }
}

}  // namespace
}  // namespace umdk

using namespace umdk;

UMDK_API int umdk_add_rmsnorm(const void* x_in, const void* a, const void* b, const void* w, void* x_out, void* h,
                              int T, int H, int ld_in, float eps, void* stream) {
  if (T < 1 || H < 8 || (H & 7) || H > kNormThreads * kMaxVecPerThread * 8 || ld_in < H || (ld_in & 7))
    return -UMDK_ERR_BAD_ARG;
  add_rmsnorm_kernel<<<T, kNormThreads, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(x_in), static_cast<const __nv_bfloat16*>(a),
      static_cast<const __nv_bfloat16*>(b), static_cast<const __nv_bfloat16*>(w), static_cast<__nv_bfloat16*>(x_out),
      static_cast<__nv_bfloat16*>(h), H, ld_in, eps);
  UMDK_CUDA_CHECK(cudaGetLastError());
  return 0;
}

UMDK_API int umdk_qkv_post(const void* qkv, int T, int q_lora, const void* q_norm, const void* kv_norm,
                           const float* cos_t, const float* sin_t, void* qa, void* kv_pool,
                           const long long* new_row, long long pool_rows, float eps, int* status, void* stream) {
  if (T < 1 || q_lora < 8 || (q_lora & 7) || q_lora > kNormThreads * kMaxVecPerThread * 8) return -UMDK_ERR_BAD_ARG;
  qkv_post_kernel<<<dim3(T, 2), kNormThreads, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(qkv), q_lora, static_cast<const __nv_bfloat16*>(q_norm),
      static_cast<const __nv_bfloat16*>(kv_norm), cos_t, sin_t, static_cast<__nv_bfloat16*>(qa),
      static_cast<__nv_bfloat16*>(kv_pool), new_row, pool_rows, eps, status);
  UMDK_CUDA_CHECK(cudaGetLastError());
  return 0;
}

UMDK_API int umdk_q_rope(const void* q, int rows, int q_head_dim, int nope, const float* cos_t, const float* sin_t,
                         void* q_full, void* stream) {
  if (rows < 1 || q_head_dim != nope + 64 || (nope & 7)) return -UMDK_ERR_BAD_ARG;
  const int n = rows * 8;
  q_rope_kernel<<<(n + 255) / 256, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(q), q_head_dim, nope, cos_t, sin_t, static_cast<__nv_bfloat16*>(q_full), rows);
  UMDK_CUDA_CHECK(cudaGetLastError());
  return 0;
}

UMDK_API int umdk_router_topk(const void* logits, int T, int E, int K, int fold_el, int rank, long long* idx_out,
                              float* w_out, void* stream) {
  if (T < 1 || E < 1 || E > 32 * kRouterMaxPerLane || K < 1 || K > 31 || K > E) return -UMDK_ERR_BAD_ARG;
  const dim3 grid((T * 32 + 127) / 128);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const __nv_bfloat16* lg = static_cast<const __nv_bfloat16*>(logits);
  if (E <= 32 * 4) router_topk_kernel<4><<<grid, 128, 0, s>>>(lg, T, E, K, fold_el, rank, idx_out, w_out);
  else if (E <= 32 * 8) router_topk_kernel<8><<<grid, 128, 0, s>>>(lg, T, E, K, fold_el, rank, idx_out, w_out);
  else if (E <= 32 * 16) router_topk_kernel<16><<<grid, 128, 0, s>>>(lg, T, E, K, fold_el, rank, idx_out, w_out);
  else router_topk_kernel<32><<<grid, 128, 0, s>>>(lg, T, E, K, fold_el, rank, idx_out, w_out);
  UMDK_CUDA_CHECK(cudaGetLastError());
  return 0;
}
