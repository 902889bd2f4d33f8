// Fused sampling for the rollout engine: temperature, top-k, top-p and the chosen token's log-prob in
// one kernel per decode step (one CTA per sequence). Replaces the sampler the reference gets from
// vLLM (cosmos_rl/rollout/vllm_rollout/vllm_rollout.py:593-730, SamplingParams built from
// cosmos_rl/policy/config/__init__.py:1477-1560).
//
// Pass 1 computes max / min / log-sum-exp of logits/T. With top-k / top-p active, the cut-off logit is
// found by bisection on the value axis (count and probability mass above the cut-off per pass; the row
// stays in L2 between passes). The draw is Gumbel-max over the kept set with a counter-based RNG keyed
// by (seed, offset, row, token), so a replay with the same keys reproduces the sample.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "api.h"

namespace {

constexpr int S_THREADS = 1024;

__device__ __forceinline__ float ld_logit(const void* p, int bf16, long long i) {
  return bf16 ? __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(p)[i]) : reinterpret_cast<const float*>(p)[i];
}

__device__ __forceinline__ uint64_t mix64(uint64_t z) {
  z += 0x9E3779B97F4A7C15ull;
  z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
  z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
  return z ^ (z >> 31);
}
__device__ __forceinline__ float uniform01(uint64_t seed, uint64_t offset, uint32_t row, uint32_t i) {
  uint64_t h = mix64(mix64(seed ^ (offset * 0xD6E8FEB86659FD93ull)) ^ (((uint64_t)row << 32) | i));
  return ((float)(h >> 40) + 0.5f) * (1.0f / 16777216.0f);  // (0, 1)
}

template <class T, class Op>
__device__ __forceinline__ T block_reduce(T v, T* sh, Op op, T identity) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = op(v, __shfl_xor_sync(0xffffffffu, v, o));
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31;
  __syncthreads();
  if (l == 0) sh[w] = v;
  __syncthreads();
  T r = (threadIdx.x < S_THREADS / 32) ? sh[threadIdx.x] : identity;
  if (w == 0) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) r = op(r, __shfl_xor_sync(0xffffffffu, r, o));
    if (l == 0) sh[0] = r;
  }
  __syncthreads();
  return sh[0];
}

struct MaxOp { __device__ float operator()(float a, float b) const { return fmaxf(a, b); } };
struct MinOp { __device__ float operator()(float a, float b) const { return fminf(a, b); } };
struct SumOp { __device__ float operator()(float a, float b) const { return a + b; } };

__global__ void __launch_bounds__(S_THREADS)
sample_kernel(const void* __restrict__ logits, int bf16, long long ld, int V, const float* __restrict__ temperature,
              const float* __restrict__ top_p, const int* __restrict__ top_k, uint64_t seed, uint64_t offset,
              const unsigned long long* __restrict__ offset_dev, long long* __restrict__ tokens,
              float* __restrict__ logprobs) {
  if (offset_dev) offset += *offset_dev;  // step counter living on the device (CUDA-graph replays)
  __shared__ float shf[32];
  __shared__ float sh_key[32];
  __shared__ int sh_idx[32];
  const int row = blockIdx.x;
  const long long base = (long long)row * ld;
  const float temp = temperature ? temperature[row] : 1.f;
  const bool greedy = temp <= 0.f;
  const float invT = greedy ? 1.f : 1.f / temp;
  const float tp = top_p ? top_p[row] : 1.f;
  const int tk = top_k ? top_k[row] : -1;

  // pass 1: max, min
  float mx = -INFINITY, mn = INFINITY;
  for (int i = threadIdx.x; i < V; i += S_THREADS) {
    float x = ld_logit(logits, bf16, base + i) * invT;
    mx = fmaxf(mx, x);
    mn = fminf(mn, x);
  }
  mx = block_reduce(mx, shf, MaxOp(), -INFINITY);
  mn = block_reduce(mn, shf, MinOp(), INFINITY);
  float se = 0.f;
  for (int i = threadIdx.x; i < V; i += S_THREADS) se += __expf(ld_logit(logits, bf16, base + i) * invT - mx);
  se = block_reduce(se, shf, SumOp(), 0.f);
  const float lse = mx + logf(se);

  float cut = -INFINITY;
  if (!greedy && ((tk > 0 && tk < V) || tp < 1.f)) {
    float mass_k = 1.f;
    if (tk > 0 && tk < V) {
      // largest cut with count(x >= cut) >= k
      float lo = mn, hi = mx;  // invariant: count(lo) >= k
      for (int it = 0; it < 32; ++it) {
        float mid = 0.5f * (lo + hi);
        float c = 0.f;
        for (int i = threadIdx.x; i < V; i += S_THREADS) c += (ld_logit(logits, bf16, base + i) * invT >= mid) ? 1.f : 0.f;
        c = block_reduce(c, shf, SumOp(), 0.f);
        if (c >= (float)tk) lo = mid; else hi = mid;
      }
      cut = lo;
      float s = 0.f;
      for (int i = threadIdx.x; i < V; i += S_THREADS) {
        float x = ld_logit(logits, bf16, base + i) * invT;
        s += (x >= cut) ? __expf(x - lse) : 0.f;
      }
      mass_k = block_reduce(s, shf, SumOp(), 0.f);
    }
    if (tp < 1.f) {
      // largest cut >= current cut with mass(x >= cut) >= top_p * mass_k
      const float want = tp * mass_k;
      float lo = (cut == -INFINITY) ? mn : cut, hi = mx;
      for (int it = 0; it < 32; ++it) {
        float mid = 0.5f * (lo + hi);
        float s = 0.f;
        for (int i = threadIdx.x; i < V; i += S_THREADS) {
          float x = ld_logit(logits, bf16, base + i) * invT;
          s += (x >= mid) ? __expf(x - lse) : 0.f;
        }
        s = block_reduce(s, shf, SumOp(), 0.f);
        if (s >= want) lo = mid; else hi = mid;
      }
      cut = lo;
    }
  }

  // draw: Gumbel-max over the kept set (plain argmax when greedy)
  float best = -INFINITY;
  int best_i = 0;
  for (int i = threadIdx.x; i < V; i += S_THREADS) {
    float x = ld_logit(logits, bf16, base + i) * invT;
    if (x < cut) continue;
    float key = x;
    if (!greedy) {
      float u = uniform01(seed, offset, (uint32_t)row, (uint32_t)i);
      key = x - __logf(-__logf(u));
    }
    if (key > best) { best = key; best_i = i; }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    float ob = __shfl_xor_sync(0xffffffffu, best, o);
    int oi = __shfl_xor_sync(0xffffffffu, best_i, o);
    if (ob > best || (ob == best && oi < best_i)) { best = ob; best_i = oi; }
  }
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31;
  if (l == 0) { sh_key[w] = best; sh_idx[w] = best_i; }
  __syncthreads();
  if (w == 0) {
    best = sh_key[l];
    best_i = sh_idx[l];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      float ob = __shfl_xor_sync(0xffffffffu, best, o);
      int oi = __shfl_xor_sync(0xffffffffu, best_i, o);
      if (ob > best || (ob == best && oi < best_i)) { best = ob; best_i = oi; }
    }
    if (l == 0) {
      tokens[row] = best_i;
      if (logprobs) {
        // log-prob under softmax(logits / temperature); for greedy rows temperature 1 is reported
        logprobs[row] = ld_logit(logits, bf16, base + best_i) * invT - lse;
      }
    }
  }
}

}  // namespace

extern "C" int b200_sample(const void* logits, int logits_bf16, long long ld, int B, int V, const float* temperature,
                           const float* top_p, const int* top_k, unsigned long long seed, unsigned long long offset,
                           const unsigned long long* offset_dev, long long* tokens, float* logprobs,
                           cudaStream_t stream) {
  if (B <= 0) return 0;
  if (V <= 0) return B200_ERR_ARG;
  sample_kernel<<<B, S_THREADS, 0, stream>>>(logits, logits_bf16, ld, V, temperature, top_p, top_k, seed, offset,
                                             offset_dev, tokens, logprobs);
  return cudaGetLastError() == cudaSuccess ? 0 : B200_ERR_LAUNCH;
}
