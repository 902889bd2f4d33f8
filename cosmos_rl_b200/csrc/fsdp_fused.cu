// Data-parallel gradient reduction and weight publication fused with the optimizer, over NVLink peer memory.
//
// The reference runs FSDP2: an NCCL reduce-scatter of fp32-cast gradients per block, a foreach/fused AdamW on
// DTensor shards, and NCCL all-gathers of the parameters (cosmos_rl/policy/model/gpt/parallelize.py:366-423,
// cosmos_rl/policy/trainer/optm/__init__.py:365-400, gradient clipping cosmos_rl/utils/distributed.py:306-407).
// Here every rank keeps the full bf16 weights and gradients in one flat, peer-mapped buffer and owns a
// contiguous shard of the fp32 optimizer state. One step is two bandwidth-bound kernels:
//   1. reduce_scatter_sumsq: read this rank's shard range from EVERY rank's bf16 gradient buffer (plain 16-byte
//      peer loads over NVLink), average in fp32, write the fp32 gradient shard and accumulate its sum of
//      squares (for the global clip coefficient) in the same pass;
//   2. adamw_publish: AdamW on the shard (fp32 master, m, v) with the clip coefficient read from the device,
//      writing the updated bf16 weights straight into EVERY rank's parameter buffer (peer stores), i.e. the
//      all-gather is the optimizer's store.
// Ordering between ranks (gradients complete before 1, all of 1 finished before gradients are cleared, all of
// 2 finished before the next forward) is provided by the caller with stream-ordered barriers.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "api.h"

namespace {

constexpr int MAX_PEERS = 8;
struct PeerPtrs {
  void* p[MAX_PEERS];
  int n;
};

__device__ __forceinline__ uint4 ld_peer(const void* p) {
  uint4 v;
  asm volatile("ld.global.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}

__global__ void __launch_bounds__(256)
reduce_scatter_sumsq_kernel(PeerPtrs grads, long long lo, long long n, float* __restrict__ out,
                            float* __restrict__ sumsq, float scale) {
  __shared__ float sh[8];
  float ss = 0.f;
  const long long nvec = n >> 3;
  for (long long v = (long long)blockIdx.x * blockDim.x + threadIdx.x; v < nvec; v += (long long)gridDim.x * blockDim.x) {
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    uint4 u[MAX_PEERS];
#pragma unroll
    for (int r = 0; r < MAX_PEERS; ++r)
      if (r < grads.n) u[r] = ld_peer(reinterpret_cast<const __nv_bfloat16*>(grads.p[r]) + lo + v * 8);
#pragma unroll
    for (int r = 0; r < MAX_PEERS; ++r) {
      if (r < grads.n) {
        const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&u[r]);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          float2 f = __bfloat1622float2(h[i]);
          acc[2 * i] += f.x;
          acc[2 * i + 1] += f.y;
        }
      }
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) { acc[i] *= scale; ss += acc[i] * acc[i]; }
    float4* o = reinterpret_cast<float4*>(out + v * 8);
    o[0] = make_float4(acc[0], acc[1], acc[2], acc[3]);
    o[1] = make_float4(acc[4], acc[5], acc[6], acc[7]);
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
  if ((threadIdx.x & 31) == 0) sh[threadIdx.x >> 5] = ss;
  __syncthreads();
  if (threadIdx.x == 0) {
    float t = 0.f;
    for (int w = 0; w < 8; ++w) t += sh[w];
    atomicAdd(sumsq, t);
  }
}

__global__ void __launch_bounds__(256)
adamw_publish_kernel(float* __restrict__ master, float* __restrict__ m, float* __restrict__ v,
                     const float* __restrict__ grad, PeerPtrs params, long long lo, long long n, float lr, float b1,
                     float b2, float eps, float wd, float bias1, float bias2, const float* __restrict__ gscale) {
  const float gs = gscale ? *gscale : 1.f;
  const float step = lr / bias1;
  const float inv_sqrt_b2 = rsqrtf(bias2);
  const long long nvec = n >> 3;
  for (long long q = (long long)blockIdx.x * blockDim.x + threadIdx.x; q < nvec; q += (long long)gridDim.x * blockDim.x) {
    const long long i = q * 8;
    float p[8], mm[8], vv[8], g[8];
    *reinterpret_cast<float4*>(p) = *reinterpret_cast<const float4*>(master + i);
    *reinterpret_cast<float4*>(p + 4) = *reinterpret_cast<const float4*>(master + i + 4);
    *reinterpret_cast<float4*>(mm) = *reinterpret_cast<const float4*>(m + i);
    *reinterpret_cast<float4*>(mm + 4) = *reinterpret_cast<const float4*>(m + i + 4);
    *reinterpret_cast<float4*>(vv) = *reinterpret_cast<const float4*>(v + i);
    *reinterpret_cast<float4*>(vv + 4) = *reinterpret_cast<const float4*>(v + i + 4);
    *reinterpret_cast<float4*>(g) = *reinterpret_cast<const float4*>(grad + i);
    *reinterpret_cast<float4*>(g + 4) = *reinterpret_cast<const float4*>(grad + i + 4);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float gj = g[j] * gs;
      p[j] *= (1.f - lr * wd);
      mm[j] = b1 * mm[j] + (1.f - b1) * gj;
      vv[j] = b2 * vv[j] + (1.f - b2) * gj * gj;
      p[j] -= step * mm[j] / (sqrtf(vv[j]) * inv_sqrt_b2 + eps);
    }
    *reinterpret_cast<float4*>(master + i) = *reinterpret_cast<float4*>(p);
    *reinterpret_cast<float4*>(master + i + 4) = *reinterpret_cast<float4*>(p + 4);
    *reinterpret_cast<float4*>(m + i) = *reinterpret_cast<float4*>(mm);
    *reinterpret_cast<float4*>(m + i + 4) = *reinterpret_cast<float4*>(mm + 4);
    *reinterpret_cast<float4*>(v + i) = *reinterpret_cast<float4*>(vv);
    *reinterpret_cast<float4*>(v + i + 4) = *reinterpret_cast<float4*>(vv + 4);
    uint4 o;
    __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
    for (int j = 0; j < 4; ++j) h[j] = __floats2bfloat162_rn(p[2 * j], p[2 * j + 1]);
#pragma unroll
    for (int r = 0; r < MAX_PEERS; ++r)
      if (r < params.n) *reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(params.p[r]) + lo + i) = o;
  }
}

// Two-shot all-reduce in ONE launch and in place: this rank owns elements [lo, lo + n) of the flat buffer, reads
// them from every rank (peer loads), averages in fp32 and stores the bf16 result into every rank's buffer (peer
// stores). A rank only ever writes its own range, and only the owner reads that range, so no barrier is needed
// between the reduce and the gather halves; the caller orders whole calls with stream barriers. This is the
// on-box form of the inter-replica gradient all-reduce (cosmos_rl/policy/trainer/llm_trainer/grpo_trainer.py:2112-2147).
__global__ void __launch_bounds__(256)
peer_all_reduce_kernel(PeerPtrs bufs, long long lo, long long n, float scale) {
  const long long stride = (long long)gridDim.x * blockDim.x * 8;
  for (long long i = ((long long)blockIdx.x * blockDim.x + threadIdx.x) * 8; i < n; i += stride) {
    float acc[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[j] = 0.f;
#pragma unroll
    for (int r = 0; r < MAX_PEERS; ++r) {
      if (r < bufs.n) {
        const uint4 u = *reinterpret_cast<const uint4*>(reinterpret_cast<const __nv_bfloat16*>(bufs.p[r]) + lo + i);
        const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 f = __bfloat1622float2(h[j]);
          acc[2 * j] += f.x;
          acc[2 * j + 1] += f.y;
        }
      }
    }
    uint4 o;
    __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
    for (int j = 0; j < 4; ++j) h[j] = __floats2bfloat162_rn(acc[2 * j] * scale, acc[2 * j + 1] * scale);
#pragma unroll
    for (int r = 0; r < MAX_PEERS; ++r)
      if (r < bufs.n) *reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(bufs.p[r]) + lo + i) = o;
  }
}

}  // namespace

extern "C" {

// bufs[r]: base of rank r's flat bf16 buffer; [lo, lo + n) is the range this rank reduces and republishes.
int b200_peer_all_reduce(void* const* bufs, int n_ranks, long long lo, long long n, float scale, cudaStream_t stream) {
  if (n <= 0) return 0;
  if (n_ranks <= 0 || n_ranks > MAX_PEERS || (n & 7) || (lo & 7)) return B200_ERR_ARG;
  PeerPtrs pp;
  pp.n = n_ranks;
  for (int r = 0; r < n_ranks; ++r) pp.p[r] = bufs[r];
  long long want = (n / 8 + 255) / 256;
  int grid = (int)(want < 148 * 16 ? want : 148 * 16);
  peer_all_reduce_kernel<<<grid, 256, 0, stream>>>(pp, lo, n, scale);
  return cudaGetLastError() == cudaSuccess ? 0 : B200_ERR_LAUNCH;
}

// grads[r]: base of rank r's flat bf16 gradient buffer (this rank's own included). Shard = [lo, lo + n), n % 8 == 0.
int b200_reduce_scatter_sumsq(void* const* grads, int n_ranks, long long lo, long long n, float* out_shard,
                              float* sumsq_accum, float scale, cudaStream_t stream) {
  if (n <= 0) return 0;
  if (n_ranks <= 0 || n_ranks > MAX_PEERS || (n & 7) || (lo & 7)) return B200_ERR_ARG;
  PeerPtrs pp;
  pp.n = n_ranks;
  for (int r = 0; r < n_ranks; ++r) pp.p[r] = grads[r];
  long long want = (n / 8 + 255) / 256;
  int grid = (int)(want < 148 * 16 ? want : 148 * 16);
  reduce_scatter_sumsq_kernel<<<grid, 256, 0, stream>>>(pp, lo, n, out_shard, sumsq_accum, scale);
  return cudaGetLastError() == cudaSuccess ? 0 : B200_ERR_LAUNCH;
}

// params[r]: base of rank r's flat bf16 parameter buffer; the updated shard is stored into every one of them.
int b200_adamw_publish(float* master, float* m, float* v, const float* grad_shard, void* const* params, int n_ranks,
                       long long lo, long long n, float lr, float beta1, float beta2, float eps, float weight_decay,
                       float bias1, float bias2, const float* grad_scale_dev, cudaStream_t stream) {
  if (n <= 0) return 0;
  if (n_ranks <= 0 || n_ranks > MAX_PEERS || (n & 7) || (lo & 7)) return B200_ERR_ARG;
  PeerPtrs pp;
  pp.n = n_ranks;
  for (int r = 0; r < n_ranks; ++r) pp.p[r] = params[r];
  long long want = (n / 8 + 255) / 256;
  int grid = (int)(want < 148 * 16 ? want : 148 * 16);
  adamw_publish_kernel<<<grid, 256, 0, stream>>>(master, m, v, grad_shard, pp, lo, n, lr, beta1, beta2, eps,
                                                 weight_decay, bias1, bias2, grad_scale_dev);
  return cudaGetLastError() == cudaSuccess ? 0 : B200_ERR_LAUNCH;
}

}  // extern "C"
