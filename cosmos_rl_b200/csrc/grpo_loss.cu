// Fused per-token GRPO objective: one pass over the scored tokens computes the clipped / dual-clipped / AIPO
// surrogate, the k3 KL penalty, the decoupled behaviour weight, and the analytic derivative of the per-token
// term with respect to the current log-prob, plus three reductions used for metrics. Replaces ~25 elementwise
// launches and 4 reductions of the op-by-op formulation (cosmos_rl/policy/trainer/llm_trainer/grpo_trainer.py:113-353).
//
// Tie rules follow torch autograd so the two paths agree bit-for-bit in the gradient's support:
// clamp passes gradient on the closed interval; minimum splits the gradient evenly on a tie.
#include <cuda_runtime.h>
#include <stdint.h>
#include "api.h"

namespace {

struct GrpoParams {
    float eps_lo, eps_hi, lower_bound, kl_beta, aipo_rho, behav_cap;
    int unbiased_kl, use_aipo, use_dual_clip, decoupled, use_cap;
};

__global__ void __launch_bounds__(256)
grpo_loss_kernel(const float* __restrict__ lp, const float* __restrict__ old_lp, const float* __restrict__ ref_lp,
                 const float* __restrict__ roll_lp, const float* __restrict__ adv, const float* __restrict__ mask,
                 int n, GrpoParams p, float* __restrict__ per_tok, float* __restrict__ dlp, float* __restrict__ kl_out,
                 float* __restrict__ stats) {
    float s_clip = 0.f, s_ratio = 0.f, s_kl = 0.f;
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x) {
        const float l = lp[i], o = old_lp[i], A = adv[i];
        const float diff = l - o;
        const float c = fminf(fmaxf(diff, -20.f), 20.f);
        const float ratio = expf(c);
        const float dratio = (diff >= -20.f && diff <= 20.f) ? ratio : 0.f;
        float per, d;
        if (p.use_aipo) {
            per = -fminf(ratio, p.aipo_rho) * A;
            d = (ratio <= p.aipo_rho) ? -dratio * A : 0.f;
            s_clip += (ratio > p.aipo_rho) ? 1.f : 0.f;
        } else {
            const float lo = 1.f - p.eps_lo, hi = 1.f + p.eps_hi;
            const float rc = fminf(fmaxf(ratio, lo), hi);
            const float l1 = ratio * A, l2 = rc * A;
            const float d1 = dratio * A, d2 = (ratio >= lo && ratio <= hi) ? dratio * A : 0.f;
            float clip1 = -fminf(l1, l2);
            float dclip = (l1 < l2) ? -d1 : ((l2 < l1) ? -d2 : -0.5f * (d1 + d2));
            s_clip += (l2 < l1) ? 1.f : 0.f;
            per = clip1;
            d = dclip;
            if (p.use_dual_clip && A < 0.f) {
                const float l3 = -p.lower_bound * A;
                if (l3 < clip1) { per = l3; d = 0.f; }
                else if (l3 == clip1) { d = 0.5f * dclip; }
            }
        }
        if (p.decoupled) {
            float w = expf(o - roll_lp[i]);
            if (p.use_cap && w > p.behav_cap) w = 0.f;
            per *= w;
            d *= w;
        }
        // off-policy sequence masking drops the surrogate of a masked sequence, never its KL penalty
        const float m = mask ? mask[i] : 1.f;
        per *= m;
        d *= m;
        float kl = 0.f;
        if (ref_lp != nullptr) {
            const float rd = ref_lp[i] - l;
            const float r = fminf(fmaxf(rd, -20.f), 20.f);
            const float e = expf(r);
            const float raw = e - r - 1.f;
            const float draw = (rd >= -20.f && rd <= 20.f) ? -(e - 1.f) : 0.f;
            float dkl;
            if (p.unbiased_kl) {
                // importance-weighted k3: the weight exp(lp - old) is differentiable and the PRODUCT is clamped
                const float w = expf(diff);
                const float prod = w * raw;
                kl = fminf(fmaxf(prod, -10.f), 10.f);
                dkl = (prod >= -10.f && prod <= 10.f) ? w * raw + w * draw : 0.f;
            } else {
                kl = fminf(fmaxf(raw, -10.f), 10.f);
                dkl = (raw >= -10.f && raw <= 10.f) ? draw : 0.f;
            }
            per += p.kl_beta * kl;
            d += p.kl_beta * dkl;
        }
        per_tok[i] = per;
        dlp[i] = d;
        kl_out[i] = kl;
        s_ratio += ratio;
        s_kl += kl;
    }
    __shared__ float red[3][8];
    #pragma unroll
    for (int off = 16; off > 0; off >>= 1) {
        s_clip += __shfl_xor_sync(0xffffffffu, s_clip, off);
        s_ratio += __shfl_xor_sync(0xffffffffu, s_ratio, off);
        s_kl += __shfl_xor_sync(0xffffffffu, s_kl, off);
    }
    const int w = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (lane == 0) { red[0][w] = s_clip; red[1][w] = s_ratio; red[2][w] = s_kl; }
    __syncthreads();
    if (threadIdx.x < 3) {
        float t = 0.f;
        for (int k = 0; k < 8; ++k) t += red[threadIdx.x][k];
        atomicAdd(&stats[threadIdx.x], t);
    }
}

}  // namespace

extern "C" int b200_grpo_loss(const float* lp, const float* old_lp, const float* ref_lp, const float* roll_lp,
                              const float* adv, const float* mask, int n, float eps_lo, float eps_hi,
                              float lower_bound, int use_dual_clip, float kl_beta, int unbiased_kl, int use_aipo,
                              float aipo_rho, int decoupled, int use_cap, float behav_cap, float* per_tok, float* dlp,
                              float* kl_out, float* stats, cudaStream_t stream) {
    if (n <= 0) return 0;
    if (decoupled && roll_lp == nullptr) return 1;
    GrpoParams p{eps_lo, eps_hi, lower_bound, kl_beta, aipo_rho, behav_cap, unbiased_kl, use_aipo, use_dual_clip,
                 decoupled, use_cap};
    cudaError_t e = cudaMemsetAsync(stats, 0, 3 * sizeof(float), stream);
    if (e != cudaSuccess) return (int)e;
    int blocks = (n + 255) / 256;
    if (blocks > 148 * 8) blocks = 148 * 8;
    grpo_loss_kernel<<<blocks, 256, 0, stream>>>(lp, old_lp, ref_lp, roll_lp, adv, mask, n, p, per_tok, dlp, kl_out,
                                                 stats);
    return (int)cudaGetLastError();
}
