// Weight-streaming GEMM for decode-sized batches (M <= 256 rows) and the fused reductions that follow it.
//
//   y[M, N] = x[M, K] * W[N, K]^T      x, W bf16 (K contiguous)
//
// With so few rows the cost of a projection is reading W once from HBM, so the work is cut into
// (column tile, contraction split) units until every SM streams its own slice of W: a tile is 128 rows x 128
// columns on the tcgen05 pipeline of gemm_core.cuh, a split covers a contiguous range of 64-wide contraction
// blocks. With one split the epilogue writes bf16 (+ bias, or SwiGLU of a fused gate/up weight) directly;
// with several it writes fp32 partial tiles to a workspace [splits, M, N] that stays in L2, and one of the
// reduction kernels below finishes the layer step it belongs to:
//   * splitk_reduce                      y = sum (+ bias)
//   * splitk_reduce_residual_rmsnorm     res' = sum + res;  y = rmsnorm(res') * w          (o_proj, down_proj)
//   * splitk_reduce_qkv_rope_append      q = rope(sum + bias), K/V rows written into the paged cache (qkv_proj)
// so the decode layer has no separate bias / RoPE / cache-append / residual / norm launches. This replaces what
// the reference gets from vLLM's fused decode kernels (cosmos_rl/rollout/vllm_rollout/vllm_rollout.py:249-339).
#include "gemm_core.cuh"
#include "api.h"

namespace b200 {

constexpr int SK_BN = 128;
constexpr int SK_STAGES = 6;

struct SkinnyParams {
  void* out;         // bf16 [M, ldo]: written when ws is null
  float* ws;         // fp32 [splits, M, N] partial results (nullable): a b200_splitk_reduce* kernel follows
  const void* bias;  // [N], nullable (direct output only; the reduce kernels add it otherwise)
  int bias_bf16;
  long long ldo;
  int M, N;          // N = columns of the output (for SwiGLU: the intermediate size)
  int splits;
  int up_row0;       // SwiGLU: first "up" row of W
};

template <bool SWIGLU>
struct SkinnySchedule {
  int num_m, num_n, splits, num_kb, total, up_row0;
  __device__ __forceinline__ void init(int M, int N, int K, int, const SkinnyParams& p) {
    num_m = (M + GEMM_BM - 1) / GEMM_BM;
    constexpr int OUT_BN = SWIGLU ? SK_BN / 2 : SK_BN;
    num_n = (p.N + OUT_BN - 1) / OUT_BN;
    splits = p.splits;
    num_kb = (K + GEMM_BK - 1) / GEMM_BK;
    total = num_m * num_n * splits;
    up_row0 = p.up_row0;
  }
  // units that share a slice of W (the row blocks of one (column tile, split)) are neighbours in the launch
  // order, so the slice is read from HBM once and from L2 by the others
  __device__ __forceinline__ bool get(int it, TileInfo& t) const {
    const int u = blockIdx.x + it * gridDim.x;
    if (u >= total) return false;
    t.m_blk = u % num_m;
    const int r = u / num_m;
    const int s = r % splits;
    t.n_blk = r / splits;
    const int kb0 = (int)(((long long)s * num_kb) / splits);
    const int kb1 = (int)(((long long)(s + 1) * num_kb) / splits);
    t.a_mn0 = t.m_blk * GEMM_BM;
    if (SWIGLU) {
      t.b_mn0 = t.n_blk * (SK_BN / 2);
      t.b_mn1 = up_row0 + t.n_blk * (SK_BN / 2);
    } else {
      t.b_mn0 = t.n_blk * SK_BN;
      t.b_mn1 = 0;
    }
    t.k0 = kb0 * GEMM_BK;
    t.num_kb = kb1 - kb0;
    t.batch = s;
    return true;
  }
};

template <bool SWIGLU>
struct SkinnyEpilogue {
  using Params = SkinnyParams;
  static constexpr bool CUSTOM_TILE = true;
  __device__ __forceinline__ void finish(const Params&) {}
  __device__ __forceinline__ void tile(const Params& p, const TileInfo& t, int row, uint32_t taddr) {
    const long long r = (long long)t.m_blk * GEMM_BM + row;
    constexpr int OUT_BN = SWIGLU ? SK_BN / 2 : SK_BN;
#pragma unroll 1
    for (int c = 0; c < OUT_BN; c += 32) {
      uint32_t a[32];
      float v[32];
      tmem_ld_32x32b_x32(taddr + c, a);
      if constexpr (SWIGLU) {
        uint32_t u[32];
        tmem_ld_32x32b_x32(taddr + SK_BN / 2 + c, u);
        tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < 32; ++j) {
          const float g = __uint_as_float(a[j]);
          v[j] = g / (1.f + __expf(-g)) * __uint_as_float(u[j]);
        }
      } else {
        tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < 32; ++j) v[j] = (t.num_kb > 0) ? __uint_as_float(a[j]) : 0.f;
      }
      const int col = t.n_blk * OUT_BN + c;
      if (r >= p.M || col >= p.N) continue;
      if (p.ws != nullptr) {
        float* dst = p.ws + ((long long)t.batch * p.M + r) * p.N + col;
        if (col + 32 <= p.N && (reinterpret_cast<uintptr_t>(dst) & 15) == 0) {
#pragma unroll
          for (int j = 0; j < 32; j += 4) *reinterpret_cast<float4*>(dst + j) = make_float4(v[j], v[j + 1], v[j + 2], v[j + 3]);
        } else {
          for (int j = 0; j < 32 && col + j < p.N; ++j) dst[j] = v[j];
        }
      } else {
        if (p.bias != nullptr) {
#pragma unroll
          for (int j = 0; j < 32; ++j)
            if (col + j < p.N)
              v[j] += p.bias_bf16 ? __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(p.bias)[col + j])
                                  : reinterpret_cast<const float*>(p.bias)[col + j];
        }
        __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(p.out) + r * p.ldo + col;
        if (col + 32 <= p.N && (reinterpret_cast<uintptr_t>(dst) & 15) == 0) {
#pragma unroll
          for (int j = 0; j < 32; j += 8) {
            uint4 o;
            o.x = pack_bf16x2(v[j], v[j + 1]);
            o.y = pack_bf16x2(v[j + 2], v[j + 3]);
            o.z = pack_bf16x2(v[j + 4], v[j + 5]);
            o.w = pack_bf16x2(v[j + 6], v[j + 7]);
            *reinterpret_cast<uint4*>(dst + j) = o;
          }
        } else {
          for (int j = 0; j < 32 && col + j < p.N; ++j) dst[j] = __float2bfloat16(v[j]);
        }
      }
    }
  }
};

template <bool SWIGLU>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
gemm_skinny_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, int M, int N, int K,
                   SkinnyParams ep, uint32_t* status) {
  gemm_mainloop<SK_BN, SK_STAGES, SkinnyEpilogue<SWIGLU>, SkinnySchedule<SWIGLU>,
                GemmTraits<false, false, false, false, 0, false, SWIGLU>>(&tmA, &tmB, M, N, K, ep, status);
}

// ---------------------------------------------------------------------------------------------------
// reductions over the split-K workspace
// ---------------------------------------------------------------------------------------------------
__device__ __forceinline__ float bias_at(const void* bias, int bias_bf16, int i) {
  return bias_bf16 ? __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(bias)[i])
                   : reinterpret_cast<const float*>(bias)[i];
}

// y[r, :] = sum_s ws[s, r, :] (+ bias); N % 4 == 0
__global__ void splitk_reduce_kernel(const float* __restrict__ ws, int splits, int M, int N, const void* bias,
                                     int bias_bf16, __nv_bfloat16* __restrict__ out, long long ldo) {
  const long long n4 = (long long)M * (N / 4);
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += (long long)gridDim.x * blockDim.x) {
    const int r = (int)(i / (N / 4)), c = (int)(i % (N / 4)) * 4;
    float4 acc = *reinterpret_cast<const float4*>(ws + (long long)r * N + c);
    for (int s = 1; s < splits; ++s) {
      const float4 v = *reinterpret_cast<const float4*>(ws + ((long long)s * M + r) * N + c);
      acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
    }
    if (bias) {
      acc.x += bias_at(bias, bias_bf16, c); acc.y += bias_at(bias, bias_bf16, c + 1);
      acc.z += bias_at(bias, bias_bf16, c + 2); acc.w += bias_at(bias, bias_bf16, c + 3);
    }
    uint2 o;
    o.x = pack_bf16x2(acc.x, acc.y);
    o.y = pack_bf16x2(acc.z, acc.w);
    *reinterpret_cast<uint2*>(out + (long long)r * ldo + c) = o;
  }
}

// One CTA per row: res_out = sum_s ws[s, r, :] (+ res_in);  y = res_out * rsqrt(mean(res_out^2) + eps) * w.
// The row (H <= RN_MAX_H fp32 values) is kept in registers between the two passes.
constexpr int RN_THREADS = 256;
constexpr int RN_VPT = 8;  // float4 per thread -> H <= 256 * 8 * 4 = 8192
__global__ void __launch_bounds__(RN_THREADS)
splitk_reduce_residual_rmsnorm_kernel(const float* __restrict__ ws, int splits, int M, int H,
                                      const __nv_bfloat16* __restrict__ res_in, const __nv_bfloat16* __restrict__ w,
                                      float eps, __nv_bfloat16* __restrict__ res_out, __nv_bfloat16* __restrict__ y) {
  const int r = blockIdx.x;
  const int n4 = H / 4;
  float4 v[RN_VPT];
  float ss = 0.f;
#pragma unroll
  for (int j = 0; j < RN_VPT; ++j) {
    const int c4 = threadIdx.x + j * RN_THREADS;
    v[j] = make_float4(0.f, 0.f, 0.f, 0.f);
    if (c4 < n4) {
      float4 acc = *reinterpret_cast<const float4*>(ws + (long long)r * H + c4 * 4);
      for (int s = 1; s < splits; ++s) {
        const float4 t = *reinterpret_cast<const float4*>(ws + ((long long)s * M + r) * H + c4 * 4);
        acc.x += t.x; acc.y += t.y; acc.z += t.z; acc.w += t.w;
      }
      if (res_in) {
        const uint2 rr = *reinterpret_cast<const uint2*>(res_in + (long long)r * H + c4 * 4);
        const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&rr.x));
        const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&rr.y));
        acc.x += a.x; acc.y += a.y; acc.z += b.x; acc.w += b.y;
      }
      // the residual stream is stored in bf16; normalise what is stored
      uint2 o;
      o.x = pack_bf16x2(acc.x, acc.y);
      o.y = pack_bf16x2(acc.z, acc.w);
      *reinterpret_cast<uint2*>(res_out + (long long)r * H + c4 * 4) = o;
      const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&o.x));
      const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&o.y));
      v[j] = make_float4(a.x, a.y, b.x, b.y);
      ss += a.x * a.x + a.y * a.y + b.x * b.x + b.y * b.y;
    }
  }
  __shared__ float red[RN_THREADS / 32];
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
  __syncthreads();
  float tot = 0.f;
#pragma unroll
  for (int i = 0; i < RN_THREADS / 32; ++i) tot += red[i];
  const float rstd = rsqrtf(tot / (float)H + eps);
#pragma unroll
  for (int j = 0; j < RN_VPT; ++j) {
    const int c4 = threadIdx.x + j * RN_THREADS;
    if (c4 < n4) {
      const uint2 ww = *reinterpret_cast<const uint2*>(w + c4 * 4);
      const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&ww.x));
      const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&ww.y));
      uint2 o;
      o.x = pack_bf16x2(v[j].x * rstd * a.x, v[j].y * rstd * a.y);
      o.y = pack_bf16x2(v[j].z * rstd * b.x, v[j].w * rstd * b.y);
      *reinterpret_cast<uint2*>(y + (long long)r * H + c4 * 4) = o;
    }
  }
}

// One CTA per token row of the fused qkv projection ([hq + 2 hkv] heads of d = 128): sums the split-K partials,
// adds the bias, rotates q and k (rotate-half RoPE at positions[r]), writes q [B, hq * d] and puts the K row and the
// V row of every kv head into the paged cache [pages, 2, hkv, page, d] at slot_mapping[r] (V slab transposed to
// [d, page] when v_transposed). A negative slot skips the cache write (padded batch rows).
__global__ void __launch_bounds__(256)
splitk_reduce_qkv_rope_append_kernel(const float* __restrict__ ws, int splits, int M, int hq, int hkv, int d,
                                     const void* bias, int bias_bf16, const long long* __restrict__ positions,
                                     const int* __restrict__ slot_mapping, float log2_theta,
                                     __nv_bfloat16* __restrict__ q_out, __nv_bfloat16* __restrict__ cache,
                                     int page_size, int v_transposed) {
  const int r = blockIdx.x;
  const int half = d >> 1;
  const int N = (hq + 2 * hkv) * d;
  const int heads = hq + 2 * hkv;
  const float pos = (float)positions[r];
  const int slot = slot_mapping[r];
  const int page = slot >= 0 ? slot / page_size : 0, off = slot >= 0 ? slot % page_size : 0;
  const long long slab = (long long)page_size * d;
  // one thread per (head, rotation pair)
  for (int idx = threadIdx.x; idx < heads * half; idx += blockDim.x) {
    const int h = idx / half, i = idx % half;
    const int c0 = h * d + i, c1 = c0 + half;
    float a = 0.f, b = 0.f;
    for (int s = 0; s < splits; ++s) {
      const float* row = ws + ((long long)s * M + r) * N;
      a += row[c0];
      b += row[c1];
    }
    if (bias) {
      a += bias_at(bias, bias_bf16, c0);
      b += bias_at(bias, bias_bf16, c1);
    }
    if (h < hq + hkv) {
      // the unfused path rounds the projection to bf16 before rotating; do the same
      a = __bfloat162float(__float2bfloat16(a));
      b = __bfloat162float(__float2bfloat16(b));
      const float inv_freq = exp2f(-(2.0f * (float)i / (float)d) * log2_theta);
      float sn, cs;
      sincosf(pos * inv_freq, &sn, &cs);
      const float ra = a * cs - b * sn, rb = b * cs + a * sn;
      a = ra;
      b = rb;
    }
    const __nv_bfloat16 oa = __float2bfloat16(a), ob = __float2bfloat16(b);
    if (h < hq) {
      q_out[(long long)r * hq * d + c0] = oa;
      q_out[(long long)r * hq * d + c1] = ob;
    } else if (slot >= 0) {
      if (h < hq + hkv) {
        __nv_bfloat16* kd = cache + ((long long)(page * 2 + 0) * hkv + (h - hq)) * slab + (long long)off * d;
        kd[i] = oa;
        kd[i + half] = ob;
      } else {
        __nv_bfloat16* vd = cache + ((long long)(page * 2 + 1) * hkv + (h - hq - hkv)) * slab;
        if (v_transposed) {
          vd[(long long)i * page_size + off] = oa;
          vd[(long long)(i + half) * page_size + off] = ob;
        } else {
          vd[(long long)off * d + i] = oa;
          vd[(long long)off * d + i + half] = ob;
        }
      }
    }
  }
}

}  // namespace b200

extern "C" {

// How many contraction splits fill the machine for this shape (1 = the GEMM writes its result directly).
int b200_gemm_skinny_splits(int M, int N, int K, int swiglu, int num_sms) {
  using namespace b200;
  const int out_bn = swiglu ? SK_BN / 2 : SK_BN;
  const int tiles = ((M + GEMM_BM - 1) / GEMM_BM) * ((N + out_bn - 1) / out_bn);
  if (swiglu) return 1;
  const int num_kb = (K + GEMM_BK - 1) / GEMM_BK;
  int s = num_sms / (tiles > 0 ? tiles : 1);
  if (s > num_kb / 4) s = num_kb / 4;  // at least four contraction blocks per unit
  if (s > 16) s = 16;
  if (s < 1) s = 1;
  return s;
}

// x [M, K] (M <= 256), W [N_w, K]; swiglu: W is a fused gate/up weight, N = intermediate size, up rows start at up_row0.
// ws == NULL: out (bf16 [M, ldo]) is written (+ bias), splits must be 1. Otherwise ws (fp32 [splits, M, N]) receives
// the partial results and one of the b200_splitk_reduce* kernels must follow.
int b200_gemm_skinny(const void* x, const void* W, void* out, float* ws, int M, int N, int K, long long ldx,
                     long long ldw, long long ldo, const void* bias, int bias_bf16, int swiglu, int up_row0,
                     int splits, uint32_t* status, int num_sms, cudaStream_t stream) {
  using namespace b200;
  if (M <= 0 || N <= 0 || K <= 0 || splits < 1 || (ldx & 7) || (ldw & 7)) return B200_ERR_ARG;
  if (splits > 1 && (!ws || swiglu)) return B200_ERR_ARG;
  if (!ws && !out) return B200_ERR_ARG;
  const int n_rows_w = swiglu ? up_row0 + N : N;
  CUtensorMap tmA, tmB;
  if (make_tmap_2d(&tmA, x, M, K, ldx, GEMM_BM, GEMM_BK, 2)) return B200_ERR_TENSORMAP;
  if (make_tmap_2d(&tmB, W, n_rows_w, K, ldw, swiglu ? SK_BN / 2 : SK_BN, GEMM_BK, 2)) return B200_ERR_TENSORMAP;
  using SM = GemmSmem<SK_BN, SK_STAGES>;
  static bool attr_set = false;
  if (!attr_set) {
    if (cudaFuncSetAttribute(gemm_skinny_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, SM::TOTAL) !=
            cudaSuccess ||
        cudaFuncSetAttribute(gemm_skinny_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, SM::TOTAL) !=
            cudaSuccess)
      return B200_ERR_LAUNCH;
    attr_set = true;
  }
  SkinnyParams ep{out, ws, ws ? nullptr : bias, bias_bf16, ldo, M, N, splits, up_row0};
  const int out_bn = swiglu ? SK_BN / 2 : SK_BN;
  const int units = ((M + GEMM_BM - 1) / GEMM_BM) * ((N + out_bn - 1) / out_bn) * splits;
  const int grid = units < num_sms ? units : num_sms;
  if (swiglu) gemm_skinny_kernel<true><<<grid, GEMM_THREADS, SM::TOTAL, stream>>>(tmA, tmB, M, N, K, ep, status);
  else gemm_skinny_kernel<false><<<grid, GEMM_THREADS, SM::TOTAL, stream>>>(tmA, tmB, M, N, K, ep, status);
  return cudaGetLastError() == cudaSuccess ? 0 : B200_ERR_LAUNCH;
}

int b200_splitk_reduce(const float* ws, int splits, int M, int N, const void* bias, int bias_bf16, void* out,
                       long long ldo, cudaStream_t stream) {
  if (M <= 0 || N <= 0 || (N & 3) || (ldo & 3) || splits < 1) return B200_ERR_ARG;
  const long long n4 = (long long)M * (N / 4);
  const int grid = (int)((n4 + 255) / 256 < 2048 ? (n4 + 255) / 256 : 2048);
  b200::splitk_reduce_kernel<<<grid, 256, 0, stream>>>(ws, splits, M, N, bias, bias_bf16, (__nv_bfloat16*)out, ldo);
  return cudaGetLastError() == cudaSuccess ? 0 : B200_ERR_LAUNCH;
}

int b200_splitk_reduce_residual_rmsnorm(const float* ws, int splits, int M, int H, const void* res_in, const void* w,
                                        float eps, void* res_out, void* y, cudaStream_t stream) {
  using namespace b200;
  if (M <= 0 || H <= 0 || (H & 3) || H > RN_THREADS * RN_VPT * 4 || splits < 1) return B200_ERR_ARG;
  splitk_reduce_residual_rmsnorm_kernel<<<M, RN_THREADS, 0, stream>>>(
      ws, splits, M, H, (const __nv_bfloat16*)res_in, (const __nv_bfloat16*)w, eps, (__nv_bfloat16*)res_out,
      (__nv_bfloat16*)y);
  return cudaGetLastError() == cudaSuccess ? 0 : B200_ERR_LAUNCH;
}

int b200_splitk_reduce_qkv_rope_append(const float* ws, int splits, int M, int hq, int hkv, int d, const void* bias,
                                       int bias_bf16, const long long* positions, const int* slot_mapping,
                                       float theta, void* q_out, void* cache, int page_size, int v_transposed,
                                       cudaStream_t stream) {
  if (M <= 0 || hq <= 0 || hkv <= 0 || d <= 0 || (d & 1) || splits < 1) return B200_ERR_ARG;
  b200::splitk_reduce_qkv_rope_append_kernel<<<M, 256, 0, stream>>>(ws, splits, M, hq, hkv, d, bias, bias_bf16, positions,
                                                                  slot_mapping, log2f(theta), (__nv_bfloat16*)q_out,
                                                                  (__nv_bfloat16*)cache, page_size, v_transposed);
  return cudaGetLastError() == cudaSuccess ? 0 : B200_ERR_LAUNCH;
}

}  // extern "C"
