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

// Tile widths: 128 columns (6 stages) when the contraction has to be split to occupy the machine, 256 columns (4
// stages) when the column tiles alone do: a wider tile re-reads the activation rows half as often, and with 128
// rows per tile that traffic out of L2 is as large as the weight stream itself.
template <int BN>
struct SkinnyCfg {
  static constexpr int STAGES = BN == 256 ? 4 : 6;
};

struct SkinnyParams {
  const CUtensorMap* tm_out;  // bf16 [M, N] (direct output) or fp32 [splits, M, N] (partials), boxes of 32 rows x 128 bytes
  const void* bias;           // [N], nullable (direct output only; the reduce kernels add it otherwise)
  int bias_bf16;
  int to_ws;                  // 1: fp32 partials through the 3-D map; 0: bf16 result through the 2-D map
  int M, N;                   // N = columns of the output (for SwiGLU: the intermediate size)
  int splits;
  int up_row0;                // SwiGLU: first "up" row of W
};

template <int BN, bool SWIGLU>
struct SkinnySchedule {
  int num_m, num_n, splits, num_kb, total, up_row0;
  __device__ __forceinline__ void init(int M, int N, int K, int, const SkinnyParams& p) {
    num_m = (M + GEMM_BM - 1) / GEMM_BM;
    constexpr int OUT_BN = SWIGLU ? BN / 2 : BN;
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
      t.b_mn0 = t.n_blk * (BN / 2);
      t.b_mn1 = up_row0 + t.n_blk * (BN / 2);
    } else {
      t.b_mn0 = t.n_blk * BN;
      t.b_mn1 = 0;
    }
    t.k0 = kb0 * GEMM_BK;
    t.num_kb = kb1 - kb0;
    t.batch = s;
    return true;
  }
};

// Epilogue: each warp turns its 32 accumulator rows into slabs of 32 rows x 128 bytes (32 fp32 or 64 bf16 columns) in
// swizzled shared memory and hands them to TMA stores, which clip rows >= M and columns >= N.
template <int BN, bool SWIGLU>
struct SkinnyEpilogue {
  using Params = SkinnyParams;
  static constexpr bool CUSTOM_TILE = true;
  uint32_t slab_idx = 0;
  __device__ __forceinline__ void finish(const Params&) {
    if ((threadIdx.x & 31) == 0) tma_store_wait<0>();
  }
  __device__ __forceinline__ void tile(const Params& p, const TileInfo& t, int row, uint32_t taddr, uint8_t* epi_smem) {
    constexpr int OUT_BN = SWIGLU ? BN / 2 : BN;
    const int lane = threadIdx.x & 31;
    const int quad = (threadIdx.x >> 5) & 3;
    uint8_t* slab0 = epi_smem + quad * 8192;
    const uint32_t sw = (uint32_t)(lane & 7);
    const int row0 = t.m_blk * GEMM_BM + quad * 32;
    const int slab_cols = p.to_ws ? 32 : 64;
#pragma unroll 1
    for (int c = 0; c < OUT_BN; c += slab_cols) {
      uint8_t* slab = slab0 + (slab_idx & 1) * 4096;
      if (lane == 0) tma_store_wait_read<1>();  // the store issued two slabs ago has finished reading this buffer
      __syncwarp();
      uint8_t* my_row = slab + lane * 128;
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        if (p.to_ws && h == 1) break;
        const int cc = c + h * 32;
        uint32_t a[32];
        float v[32];
        tmem_ld_32x32b_x32(taddr + cc, a);
        if constexpr (SWIGLU) {
          uint32_t u[32];
          tmem_ld_32x32b_x32(taddr + BN / 2 + cc, u);
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
        if (p.to_ws) {
#pragma unroll
          for (int j = 0; j < 8; ++j)
            *reinterpret_cast<float4*>(my_row + ((((uint32_t)j) ^ sw) << 4)) =
                make_float4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
        } else {
          if (p.bias != nullptr) {
            const int gc = t.n_blk * OUT_BN + cc;
#pragma unroll
            for (int j = 0; j < 32; ++j)
              if (gc + j < p.N)
                v[j] += p.bias_bf16 ? __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(p.bias)[gc + j])
                                    : reinterpret_cast<const float*>(p.bias)[gc + j];
          }
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            uint4 o;
            o.x = pack_bf16x2(v[8 * j], v[8 * j + 1]);
            o.y = pack_bf16x2(v[8 * j + 2], v[8 * j + 3]);
            o.z = pack_bf16x2(v[8 * j + 4], v[8 * j + 5]);
            o.w = pack_bf16x2(v[8 * j + 6], v[8 * j + 7]);
            *reinterpret_cast<uint4*>(my_row + ((((uint32_t)(4 * h + j)) ^ sw) << 4)) = o;
          }
        }
      }
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) {
        const int gc = t.n_blk * OUT_BN + c;
        if (gc < p.N && row0 < p.M) {
          if (p.to_ws) tma_store_3d(p.tm_out, slab, gc, row0, t.batch);
          else tma_store_2d(p.tm_out, slab, gc, row0);
        }
        tma_store_commit();
      }
      ++slab_idx;
    }
  }
};

template <int BN, bool SWIGLU>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
gemm_skinny_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                   const __grid_constant__ CUtensorMap tmO, int M, int N, int K, SkinnyParams ep, uint32_t* status) {
  ep.tm_out = &tmO;
  if (threadIdx.x == 0) tma_prefetch_desc(&tmO);
  gemm_mainloop<BN, SkinnyCfg<BN>::STAGES, SkinnyEpilogue<BN, SWIGLU>, SkinnySchedule<BN, SWIGLU>,
                GemmTraits<false, false, false, false, 0, false, SWIGLU>>(&tmA, &tmB, M, N, K, ep, status);
}

// fp32 [splits, M, N] partials: boxes of 32 rows x 32 columns, 128-byte swizzle
static int make_tmap_ws(CUtensorMap* out, const float* ws, int splits, int M, int N) {
  PFN_encodeTiled enc = get_encode_tiled();
  if (!enc) return -1;
  if ((reinterpret_cast<uintptr_t>(ws) & 15) || (N & 3)) return -2;
  cuuint64_t gdim[3] = {(cuuint64_t)N, (cuuint64_t)M, (cuuint64_t)splits};
  cuuint64_t gstr[2] = {(cuuint64_t)N * 4, (cuuint64_t)M * N * 4};
  cuuint32_t box[3] = {32, 32, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = encode_with_context([&] {
    return enc(out, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 3, const_cast<float*>(ws), gdim, gstr, box, estr,
               CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
               CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  });
  if (r != CUDA_SUCCESS) last_tmap_error() = (3 << 24) | 0x20000 | (int)r;
  return r == CUDA_SUCCESS ? 0 : -3;
}

// bf16 [M, N] result: boxes of 32 rows x 64 columns, 128-byte swizzle
static int make_tmap_out16(CUtensorMap* out, const void* ptr, int M, int N, long long ld) {
  PFN_encodeTiled enc = get_encode_tiled();
  if (!enc) return -1;
  if ((reinterpret_cast<uintptr_t>(ptr) & 15) || (ld & 7)) return -2;
  cuuint64_t gdim[2] = {(cuuint64_t)N, (cuuint64_t)M};
  cuuint64_t gstr[1] = {(cuuint64_t)ld * 2};
  cuuint32_t box[2] = {64, 32};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = encode_with_context([&] {
    return enc(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), gdim, gstr, box, estr,
               CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
               CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  });
  if (r != CUDA_SUCCESS) last_tmap_error() = (3 << 24) | 0x30000 | (int)r;
  return r == CUDA_SUCCESS ? 0 : -3;
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
  pdl_launch_dependents();
  pdl_wait();
  const long long n4 = (long long)M * (N / 4);
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += (long long)gridDim.x * blockDim.x) {
    const int r = (int)(i / (N / 4)), c = (int)(i % (N / 4)) * 4;
    float4 acc = *reinterpret_cast<const float4*>(ws + (long long)r * N + c);
#pragma unroll 4
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
  pdl_launch_dependents();
  pdl_wait();
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
#pragma unroll 4
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
  pdl_launch_dependents();
  pdl_wait();
  const int r = blockIdx.x;
  const int half = d >> 1;
  const int q4 = half >> 2;  // groups of four rotation pairs per head
  const int N = (hq + 2 * hkv) * d;
  const int heads = hq + 2 * hkv;
  const float pos = (float)positions[r];
  const int slot = slot_mapping[r];
  const int page = slot >= 0 ? slot / page_size : 0, off = slot >= 0 ? slot % page_size : 0;
  const long long slab = (long long)page_size * d;
  // one thread per (head, four rotation pairs): 16-byte loads of the partial sums. When the block size is a multiple
  // of d / 8 a thread keeps the same pair indices for every head it visits and evaluates their sines once.
  const bool fixed_i = (blockDim.x % q4) == 0;
  float sn[4], cs[4];
  if (fixed_i) {
    const int i0 = (threadIdx.x % q4) * 4;
#pragma unroll
    for (int j = 0; j < 4; ++j) sincosf(pos * exp2f(-(2.0f * (float)(i0 + j) / (float)d) * log2_theta), &sn[j], &cs[j]);
  }
  const float* row0 = ws + (long long)r * N;
  const long long split_stride = (long long)M * N;
#pragma unroll 2
  for (int idx = threadIdx.x; idx < heads * q4; idx += blockDim.x) {
    const int h = idx / q4, i0 = (idx % q4) * 4;
    const int c0 = h * d + i0, c1 = c0 + half;
    float4 a4 = make_float4(0.f, 0.f, 0.f, 0.f), b4 = a4;
#pragma unroll 4
    for (int s = 0; s < splits; ++s) {
      const float4 x = *reinterpret_cast<const float4*>(row0 + s * split_stride + c0);
      const float4 y = *reinterpret_cast<const float4*>(row0 + s * split_stride + c1);
      a4.x += x.x; a4.y += x.y; a4.z += x.z; a4.w += x.w;
      b4.x += y.x; b4.y += y.y; b4.z += y.z; b4.w += y.w;
    }
    float a[4] = {a4.x, a4.y, a4.z, a4.w}, b[4] = {b4.x, b4.y, b4.z, b4.w};
    if (bias) {
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        a[j] += bias_at(bias, bias_bf16, c0 + j);
        b[j] += bias_at(bias, bias_bf16, c1 + j);
      }
    }
    if (h < hq + hkv) {
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        // the unfused path rounds the projection to bf16 before rotating; do the same
        const float x = __bfloat162float(__float2bfloat16(a[j])), y = __bfloat162float(__float2bfloat16(b[j]));
        if (!fixed_i) sincosf(pos * exp2f(-(2.0f * (float)(i0 + j) / (float)d) * log2_theta), &sn[j], &cs[j]);
        a[j] = x * cs[j] - y * sn[j];
        b[j] = y * cs[j] + x * sn[j];
      }
    }
    uint2 oa, ob;
    oa.x = pack_bf16x2(a[0], a[1]); oa.y = pack_bf16x2(a[2], a[3]);
    ob.x = pack_bf16x2(b[0], b[1]); ob.y = pack_bf16x2(b[2], b[3]);
    if (h < hq) {
      *reinterpret_cast<uint2*>(q_out + (long long)r * hq * d + c0) = oa;
      *reinterpret_cast<uint2*>(q_out + (long long)r * hq * d + c1) = ob;
    } else if (slot >= 0) {
      if (h < hq + hkv) {
        __nv_bfloat16* kd = cache + ((long long)(page * 2 + 0) * hkv + (h - hq)) * slab + (long long)off * d;
        *reinterpret_cast<uint2*>(kd + i0) = oa;
        *reinterpret_cast<uint2*>(kd + i0 + half) = ob;
      } else {
        __nv_bfloat16* vd = cache + ((long long)(page * 2 + 1) * hkv + (h - hq - hkv)) * slab;
        if (v_transposed) {
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            vd[(long long)(i0 + j) * page_size + off] = __float2bfloat16(a[j]);
            vd[(long long)(i0 + j + half) * page_size + off] = __float2bfloat16(b[j]);
          }
        } else {
          *reinterpret_cast<uint2*>(vd + (long long)off * d + i0) = oa;
          *reinterpret_cast<uint2*>(vd + (long long)off * d + i0 + half) = ob;
        }
      }
    }
  }
}

}  // namespace b200

// Column tile width for a shape: 256 when that still leaves every SM at least two tiles (the second tile's main
// loop hides the first one's epilogue), else 128 (with contraction splits where the tiles are too few). Measured on
// the Qwen2.5-7B decode shapes at 128 rows: lm_head (594 wide tiles) 197 us against 210 us with narrow tiles;
// gate/up (148 wide tiles = one per SM) 57 us against 55 us.
static int skinny_bn(int M, int N, int swiglu, int num_sms) {
  const int num_m = (M + b200::GEMM_BM - 1) / b200::GEMM_BM;
  const int out_bn = swiglu ? 128 : 256;
  const int tiles256 = num_m * ((N + out_bn - 1) / out_bn);
  return tiles256 >= 2 * num_sms ? 256 : 128;
}

template <int BN, bool SWIGLU>
static int launch_skinny(const CUtensorMap& tmA, const CUtensorMap& tmB, const CUtensorMap& tmO, int M, int N, int K,
                         const b200::SkinnyParams& ep, uint32_t* status, int num_sms, cudaStream_t stream) {
  using namespace b200;
  using SM = GemmSmem<BN, SkinnyCfg<BN>::STAGES>;
  auto kern = gemm_skinny_kernel<BN, SWIGLU>;
  static bool attr_set = false;
  if (!attr_set) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SM::TOTAL_WITH_EPI) != cudaSuccess)
      return B200_ERR_LAUNCH;
    attr_set = true;
  }
  constexpr int OUT_BN = SWIGLU ? BN / 2 : BN;
  const int units = ((M + GEMM_BM - 1) / GEMM_BM) * ((N + OUT_BN - 1) / OUT_BN) * ep.splits;
  const int grid = units < num_sms ? units : num_sms;
  return launch_pdl(kern, dim3(grid), dim3(GEMM_THREADS), SM::TOTAL_WITH_EPI, stream, tmA, tmB, tmO, M, N, K, ep,
                    status) == cudaSuccess ? 0 : B200_ERR_LAUNCH;
}

extern "C" {

// How many contraction splits fill the machine for this shape (1 = the GEMM can write its result directly).
int b200_gemm_skinny_splits(int M, int N, int K, int swiglu, int num_sms) {
  using namespace b200;
  if (swiglu) return 1;
  const int bn = skinny_bn(M, N, 0, num_sms);
  const int tiles = ((M + GEMM_BM - 1) / GEMM_BM) * ((N + bn - 1) / bn);
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
  const int bn = skinny_bn(M, N, swiglu, num_sms);
  CUtensorMap tmA, tmB, tmO;
  if (make_tmap_2d(&tmA, x, M, K, ldx, GEMM_BM, GEMM_BK, 2)) return B200_ERR_TENSORMAP;
  if (make_tmap_2d(&tmB, W, n_rows_w, K, ldw, swiglu ? bn / 2 : bn, GEMM_BK, 2)) return B200_ERR_TENSORMAP;
  if (ws ? make_tmap_ws(&tmO, ws, splits, M, N) : make_tmap_out16(&tmO, out, M, N, ldo)) return B200_ERR_TENSORMAP;
  SkinnyParams ep{nullptr, ws ? nullptr : bias, bias_bf16, ws ? 1 : 0, M, N, splits, up_row0};
  if (bn == 256) {
    if (swiglu) return launch_skinny<256, true>(tmA, tmB, tmO, M, N, K, ep, status, num_sms, stream);
    return launch_skinny<256, false>(tmA, tmB, tmO, M, N, K, ep, status, num_sms, stream);
  }
  if (swiglu) return launch_skinny<128, true>(tmA, tmB, tmO, M, N, K, ep, status, num_sms, stream);
  return launch_skinny<128, false>(tmA, tmB, tmO, M, N, K, ep, status, num_sms, stream);
}

int b200_splitk_reduce(const float* ws, int splits, int M, int N, const void* bias, int bias_bf16, void* out,
                       long long ldo, cudaStream_t stream) {
  if (M <= 0 || N <= 0 || (N & 3) || (ldo & 3) || splits < 1) return B200_ERR_ARG;
  const long long n4 = (long long)M * (N / 4);
  const int grid = (int)((n4 + 255) / 256 < 2048 ? (n4 + 255) / 256 : 2048);
  return b200::launch_pdl(b200::splitk_reduce_kernel, dim3(grid), dim3(256), 0, stream, ws, splits, M, N, bias, bias_bf16,
                          (__nv_bfloat16*)out, ldo) == cudaSuccess ? 0 : B200_ERR_LAUNCH;
}

int b200_splitk_reduce_residual_rmsnorm(const float* ws, int splits, int M, int H, const void* res_in, const void* w,
                                        float eps, void* res_out, void* y, cudaStream_t stream) {
  using namespace b200;
  if (M <= 0 || H <= 0 || (H & 3) || H > RN_THREADS * RN_VPT * 4 || splits < 1) return B200_ERR_ARG;
  return launch_pdl(splitk_reduce_residual_rmsnorm_kernel, dim3(M), dim3(RN_THREADS), 0, stream, ws, splits, M, H,
                    (const __nv_bfloat16*)res_in, (const __nv_bfloat16*)w, eps, (__nv_bfloat16*)res_out,
                    (__nv_bfloat16*)y) == cudaSuccess ? 0 : B200_ERR_LAUNCH;
}

int b200_splitk_reduce_qkv_rope_append(const float* ws, int splits, int M, int hq, int hkv, int d, const void* bias,
                                       int bias_bf16, const long long* positions, const int* slot_mapping,
                                       float theta, void* q_out, void* cache, int page_size, int v_transposed,
                                       cudaStream_t stream) {
  if (M <= 0 || hq <= 0 || hkv <= 0 || d <= 0 || (d & 7) || splits < 1) return B200_ERR_ARG;
  return b200::launch_pdl(b200::splitk_reduce_qkv_rope_append_kernel, dim3(M), dim3(192), 0, stream, ws, splits, M, hq,
                          hkv, d, bias, bias_bf16, positions, slot_mapping, log2f(theta), (__nv_bfloat16*)q_out,
                          (__nv_bfloat16*)cache, page_size, v_transposed) == cudaSuccess ? 0 : B200_ERR_LAUNCH;
}

}  // extern "C"
