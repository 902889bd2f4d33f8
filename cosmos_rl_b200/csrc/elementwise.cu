// Bandwidth-bound ops of the policy model and optimizer for sm_100a: RMSNorm (+ fused residual add)
// forward/backward, rotary embedding, SwiGLU forward/backward, fused AdamW with bf16 shadow write,
// gradient sum-of-squares and clip coefficient. All math in fp32, 16-byte vector accesses.
// Reference semantics: cosmos_rl/policy/kernel/norm.py:36-41, rope.py:33-57, fused.py:31-37,
// cosmos_rl/policy/trainer/optm/__init__.py:365-400, cosmos_rl/utils/distributed.py:306-407.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "api.h"

namespace {

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

template <int THREADS>
__device__ __forceinline__ float block_sum(float v, float* sh) {
  v = warp_sum(v);
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31;
  __syncthreads();
  if (l == 0) sh[w] = v;
  __syncthreads();
  float r = (threadIdx.x < THREADS / 32) ? sh[threadIdx.x] : 0.f;
  if (w == 0) {
    r = warp_sum(r);
    if (l == 0) sh[0] = r;
  }
  __syncthreads();
  return sh[0];
}

__device__ __forceinline__ void unpack8(const uint4& u, float (&f)[8]) {
  const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    float2 t = __bfloat1622float2(p[i]);
    f[2 * i] = t.x;
    f[2 * i + 1] = t.y;
  }
}
__device__ __forceinline__ uint4 pack8(const float (&f)[8]) {
  uint4 u;
  __nv_bfloat162* p = reinterpret_cast<__nv_bfloat162*>(&u);
#pragma unroll
  for (int i = 0; i < 4; ++i) p[i] = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
  return u;
}

// ------------------------------------------------------------------------------------------------
// RMSNorm forward: one CTA per row, row cached in registers (H <= 256*8*MAXV)
// ------------------------------------------------------------------------------------------------
constexpr int NORM_THREADS = 256;
constexpr int NORM_MAXV = 4;

__global__ void __launch_bounds__(NORM_THREADS)
rmsnorm_fwd_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ res,
                   const __nv_bfloat16* __restrict__ w, __nv_bfloat16* __restrict__ y,
                   __nv_bfloat16* __restrict__ res_out, float* __restrict__ rstd_out, int H, float eps) {
  __shared__ float sh[32];
  const long long row = blockIdx.x;
  const int nvec = H >> 3;
  const uint4* xr = reinterpret_cast<const uint4*>(x + row * H);
  const uint4* rr = res ? reinterpret_cast<const uint4*>(res + row * H) : nullptr;
  uint4* ro = res_out ? reinterpret_cast<uint4*>(res_out + row * H) : nullptr;
  float cache[NORM_MAXV][8];
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < NORM_MAXV; ++i) {
    int v = threadIdx.x + i * NORM_THREADS;
    if (v < nvec) {
      float f[8];
      unpack8(xr[v], f);
      if (rr) {
        float g[8];
        unpack8(rr[v], g);
#pragma unroll
        for (int j = 0; j < 8; ++j) f[j] += g[j];
        uint4 h = pack8(f);
        unpack8(h, f);  // the norm sees the bf16-rounded residual stream
        if (ro) ro[v] = h;
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        cache[i][j] = f[j];
        ss += f[j] * f[j];
      }
    }
  }
  ss = block_sum<NORM_THREADS>(ss, sh);
  const float rstd = rsqrtf(ss / (float)H + eps);
  if (threadIdx.x == 0 && rstd_out) rstd_out[row] = rstd;
  const uint4* wr = reinterpret_cast<const uint4*>(w);
  uint4* yr = reinterpret_cast<uint4*>(y + row * H);
#pragma unroll
  for (int i = 0; i < NORM_MAXV; ++i) {
    int v = threadIdx.x + i * NORM_THREADS;
    if (v < nvec) {
      float g[8], o[8];
      unpack8(wr[v], g);
#pragma unroll
      for (int j = 0; j < 8; ++j) o[j] = cache[i][j] * rstd * g[j];
      yr[v] = pack8(o);
    }
  }
}

// RMSNorm backward. CTA b handles rows b, b+grid, ...; dw partial sums stay in registers.
__global__ void __launch_bounds__(NORM_THREADS)
rmsnorm_bwd_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ x,
                   const __nv_bfloat16* __restrict__ w, const float* __restrict__ rstd,
                   const __nv_bfloat16* __restrict__ dres, __nv_bfloat16* __restrict__ dx,
                   float* __restrict__ dw_partial, int T, int H) {
  __shared__ float sh[32];
  const int nvec = H >> 3;
  float dw[NORM_MAXV][8];
  float wv[NORM_MAXV][8];
#pragma unroll
  for (int i = 0; i < NORM_MAXV; ++i) {
    int v = threadIdx.x + i * NORM_THREADS;
#pragma unroll
    for (int j = 0; j < 8; ++j) dw[i][j] = 0.f;
    if (v < nvec) unpack8(reinterpret_cast<const uint4*>(w)[v], wv[i]);
  }
  for (long long row = blockIdx.x; row < T; row += gridDim.x) {
    const uint4* dyr = reinterpret_cast<const uint4*>(dy + row * H);
    const uint4* xr = reinterpret_cast<const uint4*>(x + row * H);
    const float rs = rstd[row];
    float xh[NORM_MAXV][8], dxh[NORM_MAXV][8];
    float dot = 0.f;
#pragma unroll
    for (int i = 0; i < NORM_MAXV; ++i) {
      int v = threadIdx.x + i * NORM_THREADS;
      if (v < nvec) {
        float a[8], b[8];
        unpack8(dyr[v], a);
        unpack8(xr[v], b);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          xh[i][j] = b[j] * rs;
          dxh[i][j] = a[j] * wv[i][j];
          dw[i][j] += a[j] * xh[i][j];
          dot += dxh[i][j] * xh[i][j];
        }
      }
    }
    dot = block_sum<NORM_THREADS>(dot, sh) / (float)H;
    uint4* dxr = reinterpret_cast<uint4*>(dx + row * H);
    const uint4* drr = dres ? reinterpret_cast<const uint4*>(dres + row * H) : nullptr;
#pragma unroll
    for (int i = 0; i < NORM_MAXV; ++i) {
      int v = threadIdx.x + i * NORM_THREADS;
      if (v < nvec) {
        float o[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) o[j] = rs * (dxh[i][j] - xh[i][j] * dot);
        if (drr) {
          float r[8];
          unpack8(drr[v], r);
#pragma unroll
          for (int j = 0; j < 8; ++j) o[j] += r[j];
        }
        dxr[v] = pack8(o);
      }
    }
  }
  float* out = dw_partial + (long long)blockIdx.x * H;
#pragma unroll
  for (int i = 0; i < NORM_MAXV; ++i) {
    int v = threadIdx.x + i * NORM_THREADS;
    if (v < nvec) {
#pragma unroll
      for (int j = 0; j < 8; ++j) out[v * 8 + j] = dw[i][j];
    }
  }
}

// ---- RMSNorm backward, split in two bandwidth-shaped kernels ---------------------------------------------
// dx: fully parallel over rows (one CTA per row for wide rows, one warp per row for narrow rows such as the
// per-head q/k norms), no weight-gradient state in registers. dw: column strips, each warp streams a strip of
// rows for 256 columns and the strips meet in one fp32 atomicAdd per column.
__global__ void __launch_bounds__(NORM_THREADS)
rmsnorm_dx_row_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ x,
                      const __nv_bfloat16* __restrict__ w, const float* __restrict__ rstd,
                      const __nv_bfloat16* __restrict__ dres, __nv_bfloat16* __restrict__ dx, int H) {
  __shared__ float sh[32];
  const long long row = blockIdx.x;
  const int nvec = H >> 3;
  const uint4* dyr = reinterpret_cast<const uint4*>(dy + row * H);
  const uint4* xr = reinterpret_cast<const uint4*>(x + row * H);
  const uint4* wr = reinterpret_cast<const uint4*>(w);
  const float rs = rstd[row];
  float xh[NORM_MAXV][8], dxh[NORM_MAXV][8];
  float dot = 0.f;
#pragma unroll
  for (int i = 0; i < NORM_MAXV; ++i) {
    int v = threadIdx.x + i * NORM_THREADS;
    if (v < nvec) {
      float a[8], b[8], g[8];
      unpack8(dyr[v], a);
      unpack8(xr[v], b);
      unpack8(wr[v], g);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        xh[i][j] = b[j] * rs;
        dxh[i][j] = a[j] * g[j];
        dot += dxh[i][j] * xh[i][j];
      }
    }
  }
  dot = block_sum<NORM_THREADS>(dot, sh) / (float)H;
  uint4* dxr = reinterpret_cast<uint4*>(dx + row * H);
  const uint4* drr = dres ? reinterpret_cast<const uint4*>(dres + row * H) : nullptr;
#pragma unroll
  for (int i = 0; i < NORM_MAXV; ++i) {
    int v = threadIdx.x + i * NORM_THREADS;
    if (v < nvec) {
      float o[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) o[j] = rs * (dxh[i][j] - xh[i][j] * dot);
      if (drr) {
        float r[8];
        unpack8(drr[v], r);
#pragma unroll
        for (int j = 0; j < 8; ++j) o[j] += r[j];
      }
      dxr[v] = pack8(o);
    }
  }
}

// narrow rows (H <= 1024, H % 8 == 0): one warp per row, up to 4 vectors per lane
__global__ void __launch_bounds__(256)
rmsnorm_dx_warp_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ x,
                       const __nv_bfloat16* __restrict__ w, const float* __restrict__ rstd,
                       const __nv_bfloat16* __restrict__ dres, __nv_bfloat16* __restrict__ dx, long long T, int H) {
  const long long row = (long long)blockIdx.x * 8 + (threadIdx.x >> 5);
  if (row >= T) return;
  const int lane = threadIdx.x & 31, nvec = H >> 3;
  const uint4* dyr = reinterpret_cast<const uint4*>(dy + row * H);
  const uint4* xr = reinterpret_cast<const uint4*>(x + row * H);
  const uint4* wr = reinterpret_cast<const uint4*>(w);
  const float rs = rstd[row];
  float xh[4][8], dxh[4][8];
  float dot = 0.f;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    int v = lane + 32 * i;
    if (v < nvec) {
      float a[8], b[8], g[8];
      unpack8(dyr[v], a);
      unpack8(xr[v], b);
      unpack8(wr[v], g);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        xh[i][j] = b[j] * rs;
        dxh[i][j] = a[j] * g[j];
        dot += dxh[i][j] * xh[i][j];
      }
    }
  }
  dot = warp_sum(dot) / (float)H;
  uint4* dxr = reinterpret_cast<uint4*>(dx + row * H);
  const uint4* drr = dres ? reinterpret_cast<const uint4*>(dres + row * H) : nullptr;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    int v = lane + 32 * i;
    if (v < nvec) {
      float o[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) o[j] = rs * (dxh[i][j] - xh[i][j] * dot);
      if (drr) {
        float r[8];
        unpack8(drr[v], r);
#pragma unroll
        for (int j = 0; j < 8; ++j) o[j] += r[j];
      }
      dxr[v] = pack8(o);
    }
  }
}

// dw[c] += sum_t dy[t,c] * x[t,c] * rstd[t]; grid (ceil(H/256), row strips), 8 warps per CTA split the strip
__global__ void __launch_bounds__(256)
rmsnorm_dw_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ x,
                  const float* __restrict__ rstd, float* __restrict__ dw, long long T, int H) {
  __shared__ float sh[8][256];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int c0 = blockIdx.x * 256 + lane * 8;
  const long long rows_per_cta = (T + gridDim.y - 1) / gridDim.y;
  const long long r0 = blockIdx.y * rows_per_cta, r1 = min(T, r0 + rows_per_cta);
  float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
  if (c0 < H) {
    for (long long r = r0 + warp; r < r1; r += 8) {
      float a[8], b[8];
      unpack8(*reinterpret_cast<const uint4*>(dy + r * H + c0), a);
      unpack8(*reinterpret_cast<const uint4*>(x + r * H + c0), b);
      const float rs = rstd[r];
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[j] += a[j] * b[j] * rs;
    }
  }
#pragma unroll
  for (int j = 0; j < 8; ++j) sh[warp][lane * 8 + j] = acc[j];
  __syncthreads();
  const int c = blockIdx.x * 256 + threadIdx.x;
  if (c < H) {
    float s = 0.f;
#pragma unroll
    for (int wv = 0; wv < 8; ++wv) s += sh[wv][threadIdx.x];
    atomicAdd(&dw[c], s);
  }
}

__global__ void colsum_kernel(const float* __restrict__ partial, float* __restrict__ out, int rows, int cols,
                              int accumulate) {
  int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= cols) return;
  float s = 0.f;
  for (int r = 0; r < rows; ++r) s += partial[(long long)r * cols + c];
  out[c] = accumulate ? out[c] + s : s;
}

// ------------------------------------------------------------------------------------------------
// RoPE (rotate-half convention), in place, cos/sin evaluated in fp32 from the integer position
// ------------------------------------------------------------------------------------------------
__global__ void rope_kernel(__nv_bfloat16* __restrict__ q, __nv_bfloat16* __restrict__ k,
                            const long long* __restrict__ pos, int T, int hq, int hkv, int d, long long q_stride,
                            long long k_stride, float log2_theta, float sign) {
  const int half = d >> 1;
  long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= (long long)T * half) return;
  const int i = (int)(idx % half);
  const long long t = idx / half;
  const float inv_freq = exp2f(-(2.0f * (float)i / (float)d) * log2_theta);
  float s, c;
  sincosf((float)pos[t] * inv_freq, &s, &c);
  s *= sign;
  __nv_bfloat16* qp = q + t * q_stride;
  for (int h = 0; h < hq; ++h) {
    float a = __bfloat162float(qp[h * d + i]), b = __bfloat162float(qp[h * d + i + half]);
    qp[h * d + i] = __float2bfloat16(a * c - b * s);
    qp[h * d + i + half] = __float2bfloat16(b * c + a * s);
  }
  if (k) {
    __nv_bfloat16* kp = k + t * k_stride;
    for (int h = 0; h < hkv; ++h) {
      float a = __bfloat162float(kp[h * d + i]), b = __bfloat162float(kp[h * d + i + half]);
      kp[h * d + i] = __float2bfloat16(a * c - b * s);
      kp[h * d + i + half] = __float2bfloat16(b * c + a * s);
    }
  }
}

// Vectorised variant: one thread per (token, group of ROPE_HPT heads, 8 rotation pairs); 16-byte loads and stores.
// The eight sin/cos pairs are evaluated once per thread and reused for the heads of its group (evaluating them
// per head made the kernel ALU-bound: 92 % issue-active at 0.46 of the copy bandwidth). Needs d % 16 == 0 and
// strides that keep 16-byte alignment.
constexpr int ROPE_HPT = 4;
__global__ void rope_vec_kernel(__nv_bfloat16* __restrict__ q, __nv_bfloat16* __restrict__ k,
                                const long long* __restrict__ pos, int T, int hq, int hkv, int d, long long q_stride,
                                long long k_stride, float log2_theta, float sign) {
  const int half = d >> 1, vecs = half >> 3, heads = hq + (k ? hkv : 0);
  const int groups = (heads + ROPE_HPT - 1) / ROPE_HPT;
  long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= (long long)T * groups * vecs) return;
  const int v = (int)(idx % vecs);
  const int g = (int)((idx / vecs) % groups);
  const long long t = idx / ((long long)vecs * groups);
  const float p = (float)pos[t];
  float sn[8], cs[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    const float inv_freq = exp2f(-(2.0f * (float)(v * 8 + j) / (float)d) * log2_theta);
    sincosf(p * inv_freq, &sn[j], &cs[j]);
    sn[j] *= sign;
  }
#pragma unroll
  for (int hh = 0; hh < ROPE_HPT; ++hh) {
    const int h = g * ROPE_HPT + hh;
    if (h >= heads) break;
    __nv_bfloat16* base = h < hq ? q + t * q_stride + (long long)h * d : k + t * k_stride + (long long)(h - hq) * d;
    const uint4 lo = *reinterpret_cast<const uint4*>(base + v * 8);
    const uint4 hi = *reinterpret_cast<const uint4*>(base + half + v * 8);
    float a[8], b[8], oa[8], ob[8];
    unpack8(lo, a);
    unpack8(hi, b);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      oa[j] = a[j] * cs[j] - b[j] * sn[j];
      ob[j] = b[j] * cs[j] + a[j] * sn[j];
    }
    *reinterpret_cast<uint4*>(base + v * 8) = pack8(oa);
    *reinterpret_cast<uint4*>(base + half + v * 8) = pack8(ob);
  }
}

// ------------------------------------------------------------------------------------------------
// SwiGLU on a fused [T, 2I] gate|up projection
// ------------------------------------------------------------------------------------------------
__global__ void swiglu_fwd_kernel(const __nv_bfloat16* __restrict__ gu, __nv_bfloat16* __restrict__ out, long long T,
                                  int I) {
  const int nvec = I >> 3;
  long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= T * nvec) return;
  const long long t = idx / nvec;
  const int v = (int)(idx % nvec);
  const uint4* g = reinterpret_cast<const uint4*>(gu + t * 2 * I);
  const uint4* u = reinterpret_cast<const uint4*>(gu + t * 2 * I + I);
  float a[8], b[8], o[8];
  unpack8(g[v], a);
  unpack8(u[v], b);
#pragma unroll
  for (int j = 0; j < 8; ++j) o[j] = a[j] / (1.f + __expf(-a[j])) * b[j];
  reinterpret_cast<uint4*>(out + t * I)[v] = pack8(o);
}

__global__ void swiglu_bwd_kernel(const __nv_bfloat16* __restrict__ dout, const __nv_bfloat16* __restrict__ gu,
                                  __nv_bfloat16* __restrict__ dgu, long long T, int I) {
  const int nvec = I >> 3;
  long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= T * nvec) return;
  const long long t = idx / nvec;
  const int v = (int)(idx % nvec);
  float a[8], b[8], d[8], dg[8], du[8];
  unpack8(reinterpret_cast<const uint4*>(gu + t * 2 * I)[v], a);
  unpack8(reinterpret_cast<const uint4*>(gu + t * 2 * I + I)[v], b);
  unpack8(reinterpret_cast<const uint4*>(dout + t * I)[v], d);
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    float s = 1.f / (1.f + __expf(-a[j]));
    float silu = a[j] * s;
    dg[j] = d[j] * b[j] * (s + silu * (1.f - s));
    du[j] = d[j] * silu;
  }
  reinterpret_cast<uint4*>(dgu + t * 2 * I)[v] = pack8(dg);
  reinterpret_cast<uint4*>(dgu + t * 2 * I + I)[v] = pack8(du);
}

// ------------------------------------------------------------------------------------------------
// AdamW on flat buffers
// ------------------------------------------------------------------------------------------------
template <bool GRAD_FP32>
__global__ void __launch_bounds__(256)
adamw_kernel(float* __restrict__ master, float* __restrict__ m, float* __restrict__ v, const void* __restrict__ grad,
             __nv_bfloat16* __restrict__ shadow, long long n, float lr, float b1, float b2, float eps, float wd,
             float bias1, float bias2, const float* __restrict__ gscale) {
  const float gs = gscale ? *gscale : 1.f;
  const float step = lr / bias1;
  const float inv_sqrt_b2 = rsqrtf(bias2);
  long long i = ((long long)blockIdx.x * blockDim.x + threadIdx.x) * 4;
  const long long stride = (long long)gridDim.x * blockDim.x * 4;
  for (; i + 3 < n; i += stride) {
    float4 p = *reinterpret_cast<float4*>(master + i);
    float4 mm = *reinterpret_cast<float4*>(m + i);
    float4 vv = *reinterpret_cast<float4*>(v + i);
    float g[4];
    if (GRAD_FP32) {
      float4 t = *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(grad) + i);
      g[0] = t.x; g[1] = t.y; g[2] = t.z; g[3] = t.w;
    } else {
      uint2 t = *reinterpret_cast<const uint2*>(reinterpret_cast<const __nv_bfloat16*>(grad) + i);
      float2 lo = __bfloat1622float2(*reinterpret_cast<__nv_bfloat162*>(&t.x));
      float2 hi = __bfloat1622float2(*reinterpret_cast<__nv_bfloat162*>(&t.y));
      g[0] = lo.x; g[1] = lo.y; g[2] = hi.x; g[3] = hi.y;
    }
    float pp[4] = {p.x, p.y, p.z, p.w}, pm[4] = {mm.x, mm.y, mm.z, mm.w}, pv[4] = {vv.x, vv.y, vv.z, vv.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      float gj = g[j] * gs;
      pp[j] *= (1.f - lr * wd);
      pm[j] = b1 * pm[j] + (1.f - b1) * gj;
      pv[j] = b2 * pv[j] + (1.f - b2) * gj * gj;
      pp[j] -= step * pm[j] / (sqrtf(pv[j]) * inv_sqrt_b2 + eps);
    }
    *reinterpret_cast<float4*>(master + i) = make_float4(pp[0], pp[1], pp[2], pp[3]);
    *reinterpret_cast<float4*>(m + i) = make_float4(pm[0], pm[1], pm[2], pm[3]);
    *reinterpret_cast<float4*>(v + i) = make_float4(pv[0], pv[1], pv[2], pv[3]);
    if (shadow) {
      uint2 o;
      *reinterpret_cast<__nv_bfloat162*>(&o.x) = __floats2bfloat162_rn(pp[0], pp[1]);
      *reinterpret_cast<__nv_bfloat162*>(&o.y) = __floats2bfloat162_rn(pp[2], pp[3]);
      *reinterpret_cast<uint2*>(shadow + i) = o;
    }
  }
  // tail (n not a multiple of 4): handled by the first thread
  if (blockIdx.x == 0 && threadIdx.x == 0) {
    for (long long t = n & ~3ll; t < n; ++t) {
      float gj = (GRAD_FP32 ? reinterpret_cast<const float*>(grad)[t]
                            : __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(grad)[t])) * gs;
      float p = master[t] * (1.f - lr * wd);
      float mm = b1 * m[t] + (1.f - b1) * gj;
      float vv = b2 * v[t] + (1.f - b2) * gj * gj;
      p -= step * mm / (sqrtf(vv) * inv_sqrt_b2 + eps);
      master[t] = p; m[t] = mm; v[t] = vv;
      if (shadow) shadow[t] = __float2bfloat16(p);
    }
  }
}

template <bool FP32>
__global__ void __launch_bounds__(256) sumsq_kernel(const void* __restrict__ x, long long n, float* __restrict__ out) {
  __shared__ float sh[32];
  float s = 0.f;
  long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const long long stride = (long long)gridDim.x * blockDim.x;
  if (FP32) {
    const float* p = reinterpret_cast<const float*>(x);
    for (; i < n; i += stride) { float t = p[i]; s += t * t; }
  } else {
    const __nv_bfloat16* p = reinterpret_cast<const __nv_bfloat16*>(x);
    const long long nvec = n >> 3;
    const uint4* pv = reinterpret_cast<const uint4*>(p);
    for (long long v = i; v < nvec; v += stride) {
      float f[8];
      unpack8(pv[v], f);
#pragma unroll
      for (int j = 0; j < 8; ++j) s += f[j] * f[j];
    }
    for (long long t = (nvec << 3) + i; t < n; t += stride) { float f = __bfloat162float(p[t]); s += f * f; }
  }
  s = block_sum<256>(s, sh);
  if (threadIdx.x == 0) atomicAdd(out, s);
}

__global__ void clip_coef_kernel(const float* sumsq, float max_norm, float* coef, float* norm_out) {
  float n = sqrtf(*sumsq);
  if (norm_out) *norm_out = n;
  float c = max_norm > 0.f ? max_norm / (n + 1e-6f) : 1.f;
  *coef = c < 1.f ? c : 1.f;
}

inline int ok() { return cudaGetLastError() == cudaSuccess ? 0 : B200_ERR_LAUNCH; }

}  // namespace

extern "C" {

int b200_rmsnorm_fwd(const void* x, const void* residual, const void* w, void* y, void* residual_out, float* rstd,
                     int T, int H, float eps, cudaStream_t stream) {
  if (T <= 0) return 0;
  if ((H & 7) || H > NORM_THREADS * 8 * NORM_MAXV) return B200_ERR_ARG;
  rmsnorm_fwd_kernel<<<T, NORM_THREADS, 0, stream>>>(
      (const __nv_bfloat16*)x, (const __nv_bfloat16*)residual, (const __nv_bfloat16*)w, (__nv_bfloat16*)y,
      (__nv_bfloat16*)residual_out, rstd, H, eps);
  return ok();
}

int b200_rmsnorm_bwd(const void* dy, const void* x, const void* w, const float* rstd, const void* dres, void* dx,
                     float* dw_partial, int n_partial, int T, int H, cudaStream_t stream) {
  if (T <= 0) return 0;
  if ((H & 7) || H > NORM_THREADS * 8 * NORM_MAXV || n_partial <= 0) return B200_ERR_ARG;
  rmsnorm_bwd_kernel<<<n_partial, NORM_THREADS, 0, stream>>>(
      (const __nv_bfloat16*)dy, (const __nv_bfloat16*)x, (const __nv_bfloat16*)w, rstd, (const __nv_bfloat16*)dres,
      (__nv_bfloat16*)dx, dw_partial, T, H);
  return ok();
}

// dx (+ dres) and dw (fp32, ACCUMULATED into dw_accum, which the caller zeroes or reuses across micro-batches)
int b200_rmsnorm_bwd2(const void* dy, const void* x, const void* w, const float* rstd, const void* dres, void* dx,
                      float* dw_accum, long long T, int H, cudaStream_t stream) {
  if (T <= 0) return 0;
  if ((H & 7) || H > NORM_THREADS * 8 * NORM_MAXV) return B200_ERR_ARG;
  if (H <= 1024)
    rmsnorm_dx_warp_kernel<<<(unsigned)((T + 7) / 8), 256, 0, stream>>>(
        (const __nv_bfloat16*)dy, (const __nv_bfloat16*)x, (const __nv_bfloat16*)w, rstd, (const __nv_bfloat16*)dres,
        (__nv_bfloat16*)dx, T, H);
  else
    rmsnorm_dx_row_kernel<<<(unsigned)T, NORM_THREADS, 0, stream>>>(
        (const __nv_bfloat16*)dy, (const __nv_bfloat16*)x, (const __nv_bfloat16*)w, rstd, (const __nv_bfloat16*)dres,
        (__nv_bfloat16*)dx, H);
  if (dw_accum) {
    const int col_blocks = (H + 255) / 256;
    long long strips = (148 * 8 + col_blocks - 1) / col_blocks;
    if (strips > (T + 63) / 64) strips = (T + 63) / 64;
    if (strips < 1) strips = 1;
    dim3 grid(col_blocks, (unsigned)strips);
    rmsnorm_dw_kernel<<<grid, 256, 0, stream>>>((const __nv_bfloat16*)dy, (const __nv_bfloat16*)x, rstd, dw_accum, T,
                                                H);
  }
  return ok();
}

int b200_colsum_f32(const float* partial, float* out, int rows, int cols, int accumulate, cudaStream_t stream) {
  colsum_kernel<<<(cols + 255) / 256, 256, 0, stream>>>(partial, out, rows, cols, accumulate);
  return ok();
}

int b200_rope_inplace(void* q, void* k, const long long* positions, int T, int hq, int hkv, int d, long long q_stride,
                      long long k_stride, float theta, int backward, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (d & 1) return B200_ERR_ARG;
  const bool aligned = !(d & 15) && !(q_stride & 7) && !(k_stride & 7) && !((uintptr_t)q & 15) && !((uintptr_t)k & 15);
  if (aligned) {
    long long nv = (long long)T * ((hq + (k ? hkv : 0) + ROPE_HPT - 1) / ROPE_HPT) * (d / 16);
    rope_vec_kernel<<<(unsigned)((nv + 255) / 256), 256, 0, stream>>>((__nv_bfloat16*)q, (__nv_bfloat16*)k, positions,
                                                                     T, hq, hkv, d, q_stride, k_stride,
                                                                     log2f(theta), backward ? -1.f : 1.f);
    return ok();
  }
  long long n = (long long)T * (d / 2);
  rope_kernel<<<(unsigned)((n + 255) / 256), 256, 0, stream>>>((__nv_bfloat16*)q, (__nv_bfloat16*)k, positions, T, hq,
                                                              hkv, d, q_stride, k_stride, log2f(theta),
                                                              backward ? -1.f : 1.f);
  return ok();
}

int b200_swiglu_fwd(const void* gate_up, void* out, long long T, int I, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (I & 7) return B200_ERR_ARG;
  long long n = T * (I / 8);
  swiglu_fwd_kernel<<<(unsigned)((n + 255) / 256), 256, 0, stream>>>((const __nv_bfloat16*)gate_up,
                                                                    (__nv_bfloat16*)out, T, I);
  return ok();
}

int b200_swiglu_bwd(const void* dout, const void* gate_up, void* dgate_up, long long T, int I, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (I & 7) return B200_ERR_ARG;
  long long n = T * (I / 8);
  swiglu_bwd_kernel<<<(unsigned)((n + 255) / 256), 256, 0, stream>>>(
      (const __nv_bfloat16*)dout, (const __nv_bfloat16*)gate_up, (__nv_bfloat16*)dgate_up, T, I);
  return ok();
}

int b200_adamw(float* master, float* m, float* v, const void* grad, int grad_fp32, void* param_bf16, long long n,
               float lr, float beta1, float beta2, float eps, float weight_decay, float bias1, float bias2,
               const float* grad_scale_dev, cudaStream_t stream) {
  if (n <= 0) return 0;
  long long want = (n / 4 + 255) / 256;
  int grid = (int)(want < 148 * 16 ? (want > 0 ? want : 1) : 148 * 16);
  if (grad_fp32)
    adamw_kernel<true><<<grid, 256, 0, stream>>>(master, m, v, grad, (__nv_bfloat16*)param_bf16, n, lr, beta1, beta2,
                                                 eps, weight_decay, bias1, bias2, grad_scale_dev);
  else
    adamw_kernel<false><<<grid, 256, 0, stream>>>(master, m, v, grad, (__nv_bfloat16*)param_bf16, n, lr, beta1,
                                                  beta2, eps, weight_decay, bias1, bias2, grad_scale_dev);
  return ok();
}

int b200_sumsq(const void* x, int is_fp32, long long n, float* out_accum, cudaStream_t stream) {
  if (n <= 0) return 0;
  long long want = (n / 8 + 255) / 256;
  int grid = (int)(want < 148 * 8 ? (want > 0 ? want : 1) : 148 * 8);
  if (is_fp32)
    sumsq_kernel<true><<<grid, 256, 0, stream>>>(x, n, out_accum);
  else
    sumsq_kernel<false><<<grid, 256, 0, stream>>>(x, n, out_accum);
  return ok();
}

int b200_clip_coef(const float* sumsq, float max_norm, float* coef_out, float* norm_out, cudaStream_t stream) {
  clip_coef_kernel<<<1, 1, 0, stream>>>(sumsq, max_norm, coef_out, norm_out);
  return ok();
}

}  // extern "C"
