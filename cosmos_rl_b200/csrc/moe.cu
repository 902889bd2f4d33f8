// Mixture-of-experts routing and token movement kernels for sm_100a: fused softmax + top-k router,
// expert histogram / padded offsets, permute (gather rows by expert) and weighted un-permute (combine), with
// their backward forms. They replace the eager router (cosmos_rl/policy/kernel/moe/moe.py:563-635), the Triton
// permute / un-permute kernels (cosmos_rl/policy/kernel/megatron_moe/permutation.py:35-676) and the index
// converters of the reference. Every expert's block in the permuted buffer starts on a multiple of 128 rows so
// the grouped GEMMs (grouped_gemm.cu) never see a tile that straddles two experts; nothing here needs a host
// synchronisation: counts, offsets and the tile -> expert table stay on the device.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "api.h"

namespace {

constexpr int MOE_ALIGN = 128;

// ---- router: one warp per token, E <= 256, k <= 8 ---------------------------------------------------
__global__ void route_topk_kernel(const float* __restrict__ logits, int T, int E, int k, int renorm,
                                  float* __restrict__ probs, int* __restrict__ idx, int* __restrict__ counts) {
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  if (warp >= T) return;
  const float* row = logits + (long long)warp * E;
  float v[8];
  float mx = -INFINITY;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    int e = lane + 32 * i;
    v[i] = e < E ? row[e] : -INFINITY;
    mx = fmaxf(mx, v[i]);
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
  float s = 0.f;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    v[i] = (lane + 32 * i) < E ? __expf(v[i] - mx) : 0.f;
    s += v[i];
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
  const float inv = 1.f / s;
  float topv[8];
  int topi[8];
  float tsum = 0.f;
  for (int j = 0; j < k; ++j) {
    float bv = -1.f;
    int bi = 0x7fffffff;
#pragma unroll
    for (int i = 0; i < 8; ++i)
      if (v[i] > bv) { bv = v[i]; bi = lane + 32 * i; }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      float ov = __shfl_xor_sync(0xffffffffu, bv, o);
      int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
    }
    topv[j] = bv * inv;
    topi[j] = bi;
    tsum += topv[j];
    if ((bi & 31) == lane) v[bi >> 5] = -1.f;  // remove the winner
  }
  if (lane == 0) {
    const float r = renorm ? 1.f / tsum : 1.f;
    for (int j = 0; j < k; ++j) {
      probs[(long long)warp * k + j] = topv[j] * r;
      idx[(long long)warp * k + j] = topi[j];
      if (counts) atomicAdd(&counts[topi[j]], 1);
    }
  }
}

// ---- offsets: one block; padded exclusive scan + tile -> expert table --------------------------------
__global__ void offsets_kernel(const int* __restrict__ counts, int E, int* __restrict__ offsets,
                               int* __restrict__ tile_expert, int* __restrict__ n_tiles, int* __restrict__ cursor,
                               int max_tiles) {
  if (threadIdx.x != 0) return;
  int off = 0;
  for (int e = 0; e < E; ++e) {
    offsets[e] = off;
    cursor[e] = 0;
    const int padded = (counts[e] + MOE_ALIGN - 1) / MOE_ALIGN * MOE_ALIGN;
    for (int t = off / MOE_ALIGN; t < (off + padded) / MOE_ALIGN && t < max_tiles; ++t) tile_expert[t] = e;
    off += padded;
  }
  offsets[E] = off;
  n_tiles[0] = min(off / MOE_ALIGN, max_tiles);
}

// ---- permute: claim a slot per (token, choice), copy the row -------------------------------------------
__global__ void permute_kernel(const __nv_bfloat16* __restrict__ x, const int* __restrict__ idx,
                               const int* __restrict__ offsets, int* __restrict__ cursor, int* __restrict__ row_map,
                               __nv_bfloat16* __restrict__ xp, int T, int k, int H) {
  const int pair = blockIdx.x;  // one block per (token, choice)
  if (pair >= T * k) return;
  __shared__ int pos_sh;
  if (threadIdx.x == 0) {
    const int e = idx[pair];
    pos_sh = offsets[e] + atomicAdd(&cursor[e], 1);
    row_map[pair] = pos_sh;
  }
  __syncthreads();
  const uint4* src = reinterpret_cast<const uint4*>(x + (long long)(pair / k) * H);
  uint4* dst = reinterpret_cast<uint4*>(xp + (long long)pos_sh * H);
  for (int i = threadIdx.x; i < H / 8; i += blockDim.x) dst[i] = src[i];
}

// gather rows through an existing row_map (backward of combine: dy[pos] = prob * dout[t])
__global__ void scatter_scaled_kernel(const __nv_bfloat16* __restrict__ src, const float* __restrict__ probs,
                                      const int* __restrict__ row_map, __nv_bfloat16* __restrict__ dst, int T, int k,
                                      int H) {
  const int pair = blockIdx.x;
  if (pair >= T * k) return;
  const float p = probs ? probs[pair] : 1.f;
  const __nv_bfloat162* s = reinterpret_cast<const __nv_bfloat162*>(src + (long long)(pair / k) * H);
  __nv_bfloat162* d = reinterpret_cast<__nv_bfloat162*>(dst + (long long)row_map[pair] * H);
  for (int i = threadIdx.x; i < H / 2; i += blockDim.x) {
    float2 f = __bfloat1622float2(s[i]);
    d[i] = __floats2bfloat162_rn(f.x * p, f.y * p);
  }
}

// ---- combine: out[t] = sum_j prob[t,j] * y[row_map[t,j]]  (probs null: plain sum) ------------------------
__global__ void combine_kernel(const __nv_bfloat16* __restrict__ y, const float* __restrict__ probs,
                               const int* __restrict__ row_map, __nv_bfloat16* __restrict__ out, int T, int k, int H) {
  const int t = blockIdx.x;
  if (t >= T) return;
  for (int i = threadIdx.x; i < H / 2; i += blockDim.x) {
    float ax = 0.f, ay = 0.f;
    for (int j = 0; j < k; ++j) {
      const float p = probs ? probs[t * k + j] : 1.f;
      float2 f = __bfloat1622float2(reinterpret_cast<const __nv_bfloat162*>(y + (long long)row_map[t * k + j] * H)[i]);
      ax += p * f.x;
      ay += p * f.y;
    }
    reinterpret_cast<__nv_bfloat162*>(out + (long long)t * H)[i] = __floats2bfloat162_rn(ax, ay);
  }
}

// dprob[t,j] = <dout[t], y[row_map[t,j]]>
__global__ void combine_dprob_kernel(const __nv_bfloat16* __restrict__ dout, const __nv_bfloat16* __restrict__ y,
                                     const int* __restrict__ row_map, float* __restrict__ dprob, int T, int k, int H) {
  const int pair = blockIdx.x;
  if (pair >= T * k) return;
  __shared__ float sh[32];
  const __nv_bfloat162* a = reinterpret_cast<const __nv_bfloat162*>(dout + (long long)(pair / k) * H);
  const __nv_bfloat162* b = reinterpret_cast<const __nv_bfloat162*>(y + (long long)row_map[pair] * H);
  float s = 0.f;
  for (int i = threadIdx.x; i < H / 2; i += blockDim.x) {
    float2 f = __bfloat1622float2(a[i]), g = __bfloat1622float2(b[i]);
    s += f.x * g.x + f.y * g.y;
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
  if ((threadIdx.x & 31) == 0) sh[threadIdx.x >> 5] = s;
  __syncthreads();
  if (threadIdx.x == 0) {
    float t = 0.f;
    for (int w = 0; w < (blockDim.x + 31) / 32; ++w) t += sh[w];
    dprob[pair] = t;
  }
}

inline int ok() { return cudaGetLastError() == cudaSuccess ? 0 : B200_ERR_LAUNCH; }

}  // namespace

extern "C" {

int b200_moe_route_topk(const float* logits, int T, int E, int k, int renorm, float* probs, int* idx, int* counts,
                        cudaStream_t stream) {
  if (T <= 0) return 0;
  if (E > 256 || k > 8 || k > E) return B200_ERR_ARG;
  route_topk_kernel<<<(T * 32 + 255) / 256, 256, 0, stream>>>(logits, T, E, k, renorm, probs, idx, counts);
  return ok();
}

int b200_moe_offsets(const int* counts, int E, int* offsets, int* tile_expert, int* n_tiles, int* cursor,
                     int max_tiles, cudaStream_t stream) {
  offsets_kernel<<<1, 32, 0, stream>>>(counts, E, offsets, tile_expert, n_tiles, cursor, max_tiles);
  return ok();
}

int b200_moe_permute(const void* x, const int* idx, const int* offsets, int* cursor, int* row_map, void* xp, int T,
                     int k, int H, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (H & 7) return B200_ERR_ARG;
  permute_kernel<<<T * k, 128, 0, stream>>>((const __nv_bfloat16*)x, idx, offsets, cursor, row_map,
                                            (__nv_bfloat16*)xp, T, k, H);
  return ok();
}

int b200_moe_scatter_scaled(const void* src, const float* probs, const int* row_map, void* dst, int T, int k, int H,
                            cudaStream_t stream) {
  if (T <= 0) return 0;
  scatter_scaled_kernel<<<T * k, 128, 0, stream>>>((const __nv_bfloat16*)src, probs, row_map, (__nv_bfloat16*)dst, T,
                                                   k, H);
  return ok();
}

int b200_moe_combine(const void* y, const float* probs, const int* row_map, void* out, int T, int k, int H,
                     cudaStream_t stream) {
  if (T <= 0) return 0;
  combine_kernel<<<T, 256, 0, stream>>>((const __nv_bfloat16*)y, probs, row_map, (__nv_bfloat16*)out, T, k, H);
  return ok();
}

int b200_moe_combine_dprob(const void* dout, const void* y, const int* row_map, float* dprob, int T, int k, int H,
                           cudaStream_t stream) {
  if (T <= 0) return 0;
  combine_dprob_kernel<<<T * k, 128, 0, stream>>>((const __nv_bfloat16*)dout, (const __nv_bfloat16*)y, row_map, dprob,
                                                  T, k, H);
  return ok();
}

}  // extern "C"
