// Paged KV cache append and split-KV decode attention (GQA) for the rollout engine; the engine-side
// replacement for the paged-attention kernels the reference gets from vLLM
// (cosmos_rl/rollout/vllm_rollout/vllm_rollout.py:295-326).
//
// Cache layout: [num_pages, 2 (k|v), hkv, page_size, d] bf16, so that one (page, head) slab is a
// contiguous [page_size, d] tile. Decode: grid (hkv, B, nsplit); the G = hq/hkv query heads that share a
// KV head are processed together so K/V are read from HBM once per group. Each warp owns 32-token
// groups: lanes map to tokens for QK^T (K rows streamed with 16-byte loads, q broadcast from shared
// memory) and to head-dim slices for PV. Split partials (m, l, acc) go to a scratch buffer and a
// second kernel merges them.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "api.h"

namespace {

constexpr int PD_WARPS = 4;
constexpr int PD_MAXG = 8;
constexpr float LOG2E = 1.4426950408889634f;

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

__global__ void kv_append_kernel(const __nv_bfloat16* __restrict__ k, const __nv_bfloat16* __restrict__ v,
                                 __nv_bfloat16* __restrict__ cache, const int* __restrict__ slot_mapping, int T,
                                 int hkv, int d, long long k_stride, long long v_stride, int page_size) {
  const int vec_per_tok = hkv * d / 8;
  long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= (long long)T * vec_per_tok) return;
  const int t = (int)(idx / vec_per_tok);
  const int e = (int)(idx % vec_per_tok) * 8;
  const int slot = slot_mapping[t];
  if (slot < 0) return;
  const int page = slot / page_size, off = slot % page_size;
  const int h = e / d, c = e % d;
  const long long slab = (long long)page_size * d;
  __nv_bfloat16* kd = cache + ((long long)(page * 2 + 0) * hkv + h) * slab + (long long)off * d + c;
  __nv_bfloat16* vd = cache + ((long long)(page * 2 + 1) * hkv + h) * slab + (long long)off * d + c;
  *reinterpret_cast<uint4*>(kd) = *reinterpret_cast<const uint4*>(k + t * k_stride + e);
  *reinterpret_cast<uint4*>(vd) = *reinterpret_cast<const uint4*>(v + t * v_stride + e);
}

template <int D>
__global__ void __launch_bounds__(PD_WARPS * 32)
paged_decode_kernel(const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ cache,
                    const int* __restrict__ block_table, const int* __restrict__ seq_lens,
                    __nv_bfloat16* __restrict__ out, float* __restrict__ scratch, int hq, int hkv, int page_size,
                    int max_pages, int nsplit, float scale_log2) {
  constexpr int DV = D / 32;  // head-dim elements per lane in the PV phase
  const int h = blockIdx.x, b = blockIdx.y, split = blockIdx.z;
  const int G = hq / hkv;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int len = seq_lens[b];
  int chunk = (len + nsplit - 1) / nsplit;
  chunk = (chunk + 31) & ~31;
  const int t0 = split * chunk;
  const int t1 = min(len, t0 + chunk);

  __shared__ __align__(16) float q_sh[PD_MAXG][D];
  __shared__ float p_sh[PD_WARPS][PD_MAXG][32];
  __shared__ float red_m[PD_WARPS][PD_MAXG], red_l[PD_WARPS][PD_MAXG];
  __shared__ float red_acc[PD_WARPS][PD_MAXG][D];

  for (int i = threadIdx.x; i < G * D; i += blockDim.x) {
    int g = i / D, c = i % D;
    q_sh[g][c] = __bfloat162float(q[((long long)b * hq + h * G + g) * D + c]) * scale_log2;
  }
  __syncthreads();

  float m[PD_MAXG], l[PD_MAXG], acc[PD_MAXG][DV];
#pragma unroll
  for (int g = 0; g < PD_MAXG; ++g) {
    m[g] = -INFINITY;
    l[g] = 0.f;
#pragma unroll
    for (int j = 0; j < DV; ++j) acc[g][j] = 0.f;
  }
  const long long slab = (long long)page_size * D;
  const int* bt = block_table + (long long)b * max_pages;

  for (int base = t0 + warp * 32; base < t1; base += PD_WARPS * 32) {
    // ---- QK^T: lane <-> token ----
    const int t = base + lane;
    const bool valid = t < t1;
    float s[PD_MAXG];
#pragma unroll
    for (int g = 0; g < PD_MAXG; ++g) s[g] = 0.f;
    if (valid) {
      const int page = bt[t / page_size];
      const uint4* kr = reinterpret_cast<const uint4*>(cache + ((long long)(page * 2 + 0) * hkv + h) * slab +
                                                       (long long)(t % page_size) * D);
#pragma unroll 4
      for (int c = 0; c < D / 8; ++c) {
        uint4 u = kr[c];
        const __nv_bfloat162* p2 = reinterpret_cast<const __nv_bfloat162*>(&u);
        float kf[8];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          float2 f = __bfloat1622float2(p2[j]);
          kf[2 * j] = f.x;
          kf[2 * j + 1] = f.y;
        }
#pragma unroll
        for (int g = 0; g < PD_MAXG; ++g) {
          if (g < G) {
            float4 qa = *reinterpret_cast<const float4*>(&q_sh[g][c * 8]);
            float4 qb = *reinterpret_cast<const float4*>(&q_sh[g][c * 8 + 4]);
            s[g] += kf[0] * qa.x + kf[1] * qa.y + kf[2] * qa.z + kf[3] * qa.w + kf[4] * qb.x + kf[5] * qb.y +
                    kf[6] * qb.z + kf[7] * qb.w;
          }
        }
      }
    }
    // ---- online softmax (per warp) ----
#pragma unroll
    for (int g = 0; g < PD_MAXG; ++g) {
      if (g < G) {
        float sv = valid ? s[g] : -INFINITY;
        float nm = fmaxf(m[g], warp_max(sv));
        float corr = exp2f(m[g] - nm);
        float p = valid ? exp2f(sv - nm) : 0.f;
        l[g] = l[g] * corr + warp_sum(p);
        m[g] = nm;
#pragma unroll
        for (int j = 0; j < DV; ++j) acc[g][j] *= corr;
        p_sh[warp][g][lane] = p;
      }
    }
    __syncwarp();
    // ---- PV: lane <-> head-dim slice ----
    const int ntok = min(32, t1 - base);
    for (int i = 0; i < ntok; ++i) {
      const int tt = base + i;
      const int page = bt[tt / page_size];
      const __nv_bfloat16* vr = cache + ((long long)(page * 2 + 1) * hkv + h) * slab +
                                (long long)(tt % page_size) * D + lane * DV;
      float vf[DV];
      if (DV == 4) {
        uint2 u = *reinterpret_cast<const uint2*>(vr);
        float2 a = __bfloat1622float2(*reinterpret_cast<__nv_bfloat162*>(&u.x));
        float2 c2 = __bfloat1622float2(*reinterpret_cast<__nv_bfloat162*>(&u.y));
        vf[0] = a.x; vf[1] = a.y; vf[2] = c2.x; vf[3] = c2.y;
      } else {
#pragma unroll
        for (int j = 0; j < DV; ++j) vf[j] = __bfloat162float(vr[j]);
      }
#pragma unroll
      for (int g = 0; g < PD_MAXG; ++g) {
        if (g < G) {
          const float p = p_sh[warp][g][i];
#pragma unroll
          for (int j = 0; j < DV; ++j) acc[g][j] += p * vf[j];
        }
      }
    }
    __syncwarp();
  }

  // ---- merge the warps of this CTA ----
#pragma unroll
  for (int g = 0; g < PD_MAXG; ++g) {
    if (g < G) {
      if (lane == 0) { red_m[warp][g] = m[g]; red_l[warp][g] = l[g]; }
#pragma unroll
      for (int j = 0; j < DV; ++j) red_acc[warp][g][lane * DV + j] = acc[g][j];
    }
  }
  __syncthreads();
  for (int i = threadIdx.x; i < G * D; i += blockDim.x) {
    const int g = i / D, c = i % D;
    float M = -INFINITY;
#pragma unroll
    for (int w = 0; w < PD_WARPS; ++w) M = fmaxf(M, red_m[w][g]);
    float L = 0.f, A = 0.f;
#pragma unroll
    for (int w = 0; w < PD_WARPS; ++w) {
      float cw = (red_m[w][g] == -INFINITY) ? 0.f : exp2f(red_m[w][g] - M);
      L += red_l[w][g] * cw;
      A += red_acc[w][g][c] * cw;
    }
    const long long head = (long long)b * hq + h * G + g;
    if (nsplit == 1) {
      out[head * D + c] = __float2bfloat16(L > 0.f ? A / L : 0.f);
    } else {
      float* sp = scratch + (head * nsplit + split) * (D + 2);
      sp[c] = A;
      if (c == 0) { sp[D] = M; sp[D + 1] = L; }
    }
  }
}

template <int D>
__global__ void paged_decode_merge_kernel(const float* __restrict__ scratch, __nv_bfloat16* __restrict__ out,
                                          int nsplit) {
  const long long head = blockIdx.x;
  const int c = threadIdx.x;
  const float* sp = scratch + head * nsplit * (D + 2);
  float M = -INFINITY;
  for (int s = 0; s < nsplit; ++s) M = fmaxf(M, sp[s * (D + 2) + D]);
  float L = 0.f, A = 0.f;
  for (int s = 0; s < nsplit; ++s) {
    float ms = sp[s * (D + 2) + D];
    float cw = (ms == -INFINITY) ? 0.f : exp2f(ms - M);
    L += sp[s * (D + 2) + D + 1] * cw;
    A += sp[s * (D + 2) + c] * cw;
  }
  out[head * D + c] = __float2bfloat16(L > 0.f ? A / L : 0.f);
}

}  // namespace

extern "C" {

int b200_kv_append(const void* k, const void* v, void* cache, const int* slot_mapping, int T, int hkv, int d,
                   long long k_stride, long long v_stride, int page_size, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (d & 7) return B200_ERR_ARG;
  long long n = (long long)T * hkv * d / 8;
  kv_append_kernel<<<(unsigned)((n + 255) / 256), 256, 0, stream>>>((const __nv_bfloat16*)k, (const __nv_bfloat16*)v,
                                                                   (__nv_bfloat16*)cache, slot_mapping, T, hkv, d,
                                                                   k_stride, v_stride, page_size);
  return cudaGetLastError() == cudaSuccess ? 0 : B200_ERR_LAUNCH;
}

int b200_paged_decode(const void* q, const void* cache, const int* block_table, const int* seq_lens, void* out,
                      float* scratch, int B, int hq, int hkv, int d, int page_size, int max_pages, int nsplit,
                      float scale, cudaStream_t stream) {
  if (B <= 0) return 0;
  if (hkv <= 0 || hq % hkv || hq / hkv > PD_MAXG || nsplit <= 0 || (nsplit > 1 && !scratch)) return B200_ERR_ARG;
  dim3 grid(hkv, B, nsplit);
  if (d == 128) {
    paged_decode_kernel<128><<<grid, PD_WARPS * 32, 0, stream>>>(
        (const __nv_bfloat16*)q, (const __nv_bfloat16*)cache, block_table, seq_lens, (__nv_bfloat16*)out, scratch, hq,
        hkv, page_size, max_pages, nsplit, scale * LOG2E);
    if (nsplit > 1) paged_decode_merge_kernel<128><<<B * hq, 128, 0, stream>>>(scratch, (__nv_bfloat16*)out, nsplit);
  } else if (d == 64) {
    paged_decode_kernel<64><<<grid, PD_WARPS * 32, 0, stream>>>(
        (const __nv_bfloat16*)q, (const __nv_bfloat16*)cache, block_table, seq_lens, (__nv_bfloat16*)out, scratch, hq,
        hkv, page_size, max_pages, nsplit, scale * LOG2E);
    if (nsplit > 1) paged_decode_merge_kernel<64><<<B * hq, 64, 0, stream>>>(scratch, (__nv_bfloat16*)out, nsplit);
  } else {
    return B200_ERR_ARG;
  }
  return cudaGetLastError() == cudaSuccess ? 0 : B200_ERR_LAUNCH;
}

}  // extern "C"

// ---------------------------------------------------------------------------------------------------
// Split-KV decode attention for callers that cannot allocate device memory.
//
// Who needs this: a host program that embeds the rollout engine after it has already given the whole
// device to weights and KV cache (its memory budget is fixed at start-up, so a later cudaMalloc can
// fail or fragment the budget), or a caller written against the plain C ABI that has no device
// allocator of its own to obtain the split-merge scratch buffer from. For them the scratch lives in the
// library image: a file-scope __device__ array of PD_STATIC_SCRATCH_FLOATS floats (16 MiB). Every GPU
// on which this library is loaded holds that array from load until the process exits.
//
// Rules of use:
//  * The first call on a device looks up the array's device address (cudaGetSymbolAddress with that
//    device current) and remembers it; make that first call before any stream capture begins.
//  * B * hq * nsplit * (d + 2) must not exceed PD_STATIC_SCRATCH_FLOATS, else B200_ERR_TOO_LARGE is
//    returned and nothing is launched.
//  * All calls on a device share the one array. The first kernel writes every element the merge kernel
//    reads (empty splits included), so nothing has to be cleared and contents left by the previous call
//    are harmless; but two calls whose kernels overlap on the GPU (different streams) would race on it.
//  * No cudaMalloc, cudaFree or other allocating routine is called, here or in the kernels.
// ---------------------------------------------------------------------------------------------------
#include <mutex>

#define PD_STATIC_SCRATCH_FLOATS (4u * 1024u * 1024u)
#define PD_MAX_DEVICES 64

static __device__ __align__(256) float g_pd_static_scratch[PD_STATIC_SCRATCH_FLOATS];
static float* g_pd_scratch_addr[PD_MAX_DEVICES];  // device address of the array, per device
static std::mutex g_pd_scratch_mu;

extern "C" int b200_paged_decode_static(const void* q, const void* cache, const int* block_table,
                                        const int* seq_lens, void* out, int B, int hq, int hkv, int d,
                                        int page_size, int max_pages, int nsplit, float scale,
                                        cudaStream_t stream) {
  if (B <= 0) return 0;
  if (hkv <= 0 || hq % hkv || hq / hkv > PD_MAXG || nsplit <= 0 || (d != 128 && d != 64)) return B200_ERR_ARG;
  const unsigned long long need = (unsigned long long)B * hq * nsplit * (d + 2);
  if (need > PD_STATIC_SCRATCH_FLOATS) return B200_ERR_TOO_LARGE;
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= PD_MAX_DEVICES) return B200_ERR_RUNTIME;
  float* scratch = nullptr;
  {
    std::lock_guard<std::mutex> lock(g_pd_scratch_mu);
    if (g_pd_scratch_addr[dev] == nullptr) {
      // In host code the array's name is only a stand-in; the address the kernel may use comes from here.
      void* p = nullptr;
      if (cudaGetSymbolAddress(&p, g_pd_static_scratch) != cudaSuccess || p == nullptr) return B200_ERR_RUNTIME;
      g_pd_scratch_addr[dev] = static_cast<float*>(p);
    }
    scratch = g_pd_scratch_addr[dev];
  }
  dim3 grid(hkv, B, nsplit);
  if (d == 128) {
    paged_decode_kernel<128><<<grid, PD_WARPS * 32, 0, stream>>>(
        (const __nv_bfloat16*)q, (const __nv_bfloat16*)cache, block_table, seq_lens, (__nv_bfloat16*)out, scratch, hq,
        hkv, page_size, max_pages, nsplit, scale * LOG2E);
    if (nsplit > 1) paged_decode_merge_kernel<128><<<B * hq, 128, 0, stream>>>(scratch, (__nv_bfloat16*)out, nsplit);
  } else {
    paged_decode_kernel<64><<<grid, PD_WARPS * 32, 0, stream>>>(
        (const __nv_bfloat16*)q, (const __nv_bfloat16*)cache, block_table, seq_lens, (__nv_bfloat16*)out, scratch, hq,
        hkv, page_size, max_pages, nsplit, scale * LOG2E);
    if (nsplit > 1) paged_decode_merge_kernel<64><<<B * hq, 64, 0, stream>>>(scratch, (__nv_bfloat16*)out, nsplit);
  }
  return cudaGetLastError() == cudaSuccess ? 0 : B200_ERR_LAUNCH;
}
