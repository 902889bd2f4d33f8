// Fused lm_head GEMM + per-token log-probability / entropy on tcgen05, without ever writing the
// [T, V] logits to memory. Replaces the eager row-loop log_softmax+gather and chunked entropy of the
// reference (cosmos_rl/utils/util.py:314-366, 899-994) and feeds the GRPO loss
// (cosmos_rl/policy/trainer/llm_trainer/grpo_trainer.py:113-353).
//
// Forward: work unit = (128-row block of tokens, vocabulary split). The CTA that owns a unit walks its
// vocabulary tiles; each epilogue thread owns one token row and keeps an online-softmax state
// (running max, sum of exp, label logit, sum exp*logit) in registers across tiles, written once per unit
// to a [T, nsplit, 4] fp32 scratch that b200_logprob_combine reduces.
// Backward: the logits tile is recomputed on the tensor cores and the epilogue emits
// d(loss)/d(logits) in bf16 for a vocabulary chunk; the two remaining GEMMs are plain ones.
#include "gemm_core.cuh"
#include "api.h"

namespace b200 {

constexpr int LP_BN = 256;
constexpr int LP_STAGES = 4;
constexpr float LOG2E = 1.4426950408889634f;
constexpr float LN2 = 0.6931471805599453f;

struct LogprobEpilogue {
  struct Params {
    const long long* labels;
    float* partial;  // [T, nsplit, 4]
    int T, V, nsplit, tps;
    float scale_log2;  // inv_temperature * log2(e): logits are tracked in the log2 domain
  };
  float m, l, z, e;
  int cur_unit_m = -1, cur_split = -1;
  long long label;

  __device__ __forceinline__ void flush(const Params& p, int row) {
    if (cur_unit_m < 0) return;
    long long r = (long long)cur_unit_m * GEMM_BM + row;
    if (r < p.T) {
      float4 o = make_float4(m, l, z, e);
      *reinterpret_cast<float4*>(p.partial + (r * p.nsplit + cur_split) * 4) = o;
    }
  }
  __device__ __forceinline__ void tile_begin(const Params& p, const TileInfo& t, int row) {
    const int m_blk = t.m_blk, n_blk = t.n_blk;
    int split = n_blk / p.tps;
    if (m_blk != cur_unit_m || split != cur_split) {
      flush(p, row);
      cur_unit_m = m_blk;
      cur_split = split;
      m = -INFINITY; l = 0.f; z = -INFINITY; e = 0.f;
      long long r = (long long)m_blk * GEMM_BM + row;
      label = r < p.T ? p.labels[r] : -1;
    }
  }
  __device__ __forceinline__ void chunk(const Params& p, const TileInfo& t, int row, int col0,
                                        const float (&v)[32]) {
    const int c = t.n_blk * LP_BN + col0;
    if (c >= p.V) return;
    float x[32];
    float cmax = -INFINITY;
#pragma unroll
    for (int i = 0; i < 32; ++i) {
      x[i] = (c + i < p.V) ? v[i] * p.scale_log2 : -INFINITY;
      cmax = fmaxf(cmax, x[i]);
    }
    const float nm = fmaxf(m, cmax);
    const float corr = exp2f(m - nm);  // m = -inf on the first chunk -> 0
    float sl = 0.f, se = 0.f;
#pragma unroll
    for (int i = 0; i < 32; ++i) {
      float pexp = exp2f(x[i] - nm);
      sl += pexp;
      se += (c + i < p.V) ? pexp * x[i] : 0.f;
    }
    l = l * corr + sl;
    e = e * corr + se;
    m = nm;
    const long long off = label - c;
    if (off >= 0 && off < 32) {
#pragma unroll
      for (int i = 0; i < 32; ++i)
        if (i == (int)off) z = x[i];
    }
  }
  __device__ __forceinline__ void tile_end(const Params&, const TileInfo&, int) {}
  __device__ __forceinline__ void finish(const Params& p) {
    const int quad = (threadIdx.x >> 5) & 3;
    flush(p, quad * 32 + (threadIdx.x & 31));
  }
};

// Work unit u = (token block, vocabulary split); CTA b owns units b, b+grid, ... and walks the tps
// vocabulary tiles of each. n_blk may run past the last real tile in the final split: those tiles read
// zero-filled weights and the epilogue masks every column >= V.
struct LogprobSched {
  int num_m, tps, units, num_kb;
  __device__ __forceinline__ void init(int M, int, int K, int, const LogprobEpilogue::Params& p) {
    num_m = (M + GEMM_BM - 1) / GEMM_BM;
    tps = p.tps;
    units = num_m * p.nsplit;
    num_kb = (K + GEMM_BK - 1) / GEMM_BK;
  }
  __device__ __forceinline__ bool get(int it, TileInfo& t) const {
    int j = it / tps, i = it - j * tps;
    int u = blockIdx.x + j * gridDim.x;
    if (u >= units) return false;
    t.m_blk = u % num_m;
    t.n_blk = (u / num_m) * tps + i;
    t.a_mn0 = t.m_blk * GEMM_BM;
    t.b_mn0 = t.n_blk * LP_BN;
    t.k0 = 0;
    t.num_kb = num_kb;
    t.batch = 0;
    return true;
  }
};

__global__ void __launch_bounds__(GEMM_THREADS, 1)
lmhead_logprob_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, int T, int V,
                      int H, LogprobEpilogue::Params ep, uint32_t* status) {
  gemm_mainloop<LP_BN, LP_STAGES, LogprobEpilogue, LogprobSched>(&tmA, &tmB, T, V, H, ep, status);
}

__global__ void logprob_combine_kernel(const float* __restrict__ partial, const long long* __restrict__ labels,
                                       float* __restrict__ logprob, float* __restrict__ lse_out,
                                       float* __restrict__ entropy, int T, int nsplit) {
  int r = blockIdx.x * blockDim.x + threadIdx.x;
  if (r >= T) return;
  const float4* p = reinterpret_cast<const float4*>(partial) + (long long)r * nsplit;
  float M = -INFINITY;
  for (int s = 0; s < nsplit; ++s) M = fmaxf(M, p[s].x);
  float L = 0.f, E = 0.f, Z = -INFINITY;
  for (int s = 0; s < nsplit; ++s) {
    float4 q = p[s];
    float c = exp2f(q.x - M);
    L += q.y * c;
    E += q.w * c;
    Z = fmaxf(Z, q.z);
  }
  // convert from the log2 domain back to natural log
  const float lse2 = M + log2f(L);
  if (lse_out) lse_out[r] = lse2 * LN2;
  if (logprob) logprob[r] = (labels[r] >= 0) ? (Z - lse2) * LN2 : 0.f;
  if (entropy) entropy[r] = (lse2 - E / L) * LN2;
}

// ---------------------------------------------------------------------------------------------
// backward: dlogits chunk
// ---------------------------------------------------------------------------------------------
struct DlogitsEpilogue {
  struct Params {
    const long long* labels;
    const float* lse;
    const float* g_lp;
    const float* g_ent;   // may be null
    const float* ent;     // may be null
    __nv_bfloat16* out;
    long long ldd;
    int T, Vc, v0;
    float inv_temp;
  };
  float lse_r, glp, gent, ent_r;
  long long label;
  __device__ __forceinline__ void tile_begin(const Params& p, const TileInfo& t, int row) {
    long long r = (long long)t.m_blk * GEMM_BM + row;
    if (r < p.T) {
      lse_r = p.lse[r];
      glp = p.g_lp[r];
      gent = p.g_ent ? p.g_ent[r] : 0.f;
      ent_r = p.ent ? p.ent[r] : 0.f;
      label = p.labels[r];
      if (label < 0) { glp = 0.f; }
    }
  }
  __device__ __forceinline__ void chunk(const Params& p, const TileInfo& t, int row, int col0,
                                        const float (&v)[32]) {
    const long long r = (long long)t.m_blk * GEMM_BM + row;
    const int c = t.n_blk * LP_BN + col0;
    if (r >= p.T || c >= p.Vc) return;
    float o[32];
    const long long off = label - (long long)(p.v0 + c);
#pragma unroll
    for (int i = 0; i < 32; ++i) {
      float x = v[i] * p.inv_temp;
      float pr = __expf(x - lse_r);
      float g = -glp * pr - gent * pr * (x - lse_r + ent_r);
      if ((long long)i == off) g += glp;
      o[i] = g * p.inv_temp;
    }
    __nv_bfloat16* dst = p.out + r * p.ldd + c;
    if (c + 32 <= p.Vc && ((reinterpret_cast<uintptr_t>(dst) & 15) == 0)) {
#pragma unroll
      for (int i = 0; i < 32; i += 8) {
        uint4 u;
        u.x = pack_bf16x2(o[i], o[i + 1]);
        u.y = pack_bf16x2(o[i + 2], o[i + 3]);
        u.z = pack_bf16x2(o[i + 4], o[i + 5]);
        u.w = pack_bf16x2(o[i + 6], o[i + 7]);
        *reinterpret_cast<uint4*>(dst + i) = u;
      }
    } else {
      for (int i = 0; i < 32 && c + i < p.Vc; ++i) dst[i] = __float2bfloat16(o[i]);
    }
  }
  __device__ __forceinline__ void tile_end(const Params&, const TileInfo&, int) {}
  __device__ __forceinline__ void finish(const Params&) {}
};

__global__ void __launch_bounds__(GEMM_THREADS, 1)
lmhead_dlogits_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, int T, int Vc,
                      int H, DlogitsEpilogue::Params ep, uint32_t* status) {
  gemm_mainloop<LP_BN, LP_STAGES, DlogitsEpilogue, RasterSchedule>(&tmA, &tmB, T, Vc, H, ep, status);
}

}  // namespace b200

extern "C" {

int b200_lmhead_logprob_partial(const void* hidden, const void* weight, const long long* labels, float* partial,
                                int T, int V, int H, long long ldh, long long ldw, float inv_temperature,
                                int nsplit, uint32_t* status, int num_sms, cudaStream_t stream) {
  using namespace b200;
  if (T <= 0 || V <= 0 || H <= 0 || (H & 7) || nsplit <= 0) return B200_ERR_ARG;
  CUtensorMap tmA, tmB;
  if (make_tmap_2d(&tmA, hidden, T, H, ldh, GEMM_BM, GEMM_BK, 2)) return B200_ERR_TENSORMAP;
  if (make_tmap_2d(&tmB, weight, V, H, ldw, LP_BN, GEMM_BK, 2)) return B200_ERR_TENSORMAP;
  using SM = GemmSmem<LP_BN, LP_STAGES>;
  static bool attr_set = false;
  if (!attr_set) {
    if (cudaFuncSetAttribute(lmhead_logprob_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SM::TOTAL) !=
        cudaSuccess)
      return B200_ERR_LAUNCH;
    attr_set = true;
  }
  const int num_m = (T + GEMM_BM - 1) / GEMM_BM;
  const int num_n = (V + LP_BN - 1) / LP_BN;
  if (nsplit > num_n) return B200_ERR_ARG;
  LogprobEpilogue::Params ep{labels, partial, T, V, nsplit, (num_n + nsplit - 1) / nsplit, inv_temperature * LOG2E};
  int units = num_m * nsplit;
  int grid = units < num_sms ? units : num_sms;
  lmhead_logprob_kernel<<<grid, GEMM_THREADS, SM::TOTAL, stream>>>(tmA, tmB, T, V, H, ep, status);
  return cudaGetLastError() == cudaSuccess ? 0 : B200_ERR_LAUNCH;
}

int b200_logprob_combine(const float* partial, const long long* labels, float* logprob, float* lse, float* entropy,
                         int T, int nsplit, cudaStream_t stream) {
  if (T <= 0) return 0;
  b200::logprob_combine_kernel<<<(T + 127) / 128, 128, 0, stream>>>(partial, labels, logprob, lse, entropy, T, nsplit);
  return cudaGetLastError() == cudaSuccess ? 0 : B200_ERR_LAUNCH;
}

int b200_lmhead_dlogits(const void* hidden, const void* weight, const long long* labels, const float* lse,
                        const float* g_logprob, const float* g_entropy, const float* entropy, void* dlogits, int T,
                        int V, int H, long long ldh, long long ldw, int v0, int Vc, long long ldd,
                        float inv_temperature, uint32_t* status, int num_sms, cudaStream_t stream) {
  using namespace b200;
  if (T <= 0 || Vc <= 0 || H <= 0 || (H & 7) || v0 < 0 || v0 + Vc > V) return B200_ERR_ARG;
  CUtensorMap tmA, tmB;
  const __nv_bfloat16* wchunk = reinterpret_cast<const __nv_bfloat16*>(weight) + (long long)v0 * ldw;
  if (make_tmap_2d(&tmA, hidden, T, H, ldh, GEMM_BM, GEMM_BK, 2)) return B200_ERR_TENSORMAP;
  if (make_tmap_2d(&tmB, wchunk, Vc, H, ldw, LP_BN, GEMM_BK, 2)) return B200_ERR_TENSORMAP;
  using SM = GemmSmem<LP_BN, LP_STAGES>;
  static bool attr_set = false;
  if (!attr_set) {
    if (cudaFuncSetAttribute(lmhead_dlogits_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SM::TOTAL) !=
        cudaSuccess)
      return B200_ERR_LAUNCH;
    attr_set = true;
  }
  DlogitsEpilogue::Params ep{labels, lse, g_logprob, g_entropy, entropy, (__nv_bfloat16*)dlogits, ldd, T, Vc, v0,
                             inv_temperature};
  int tiles = ((T + GEMM_BM - 1) / GEMM_BM) * ((Vc + LP_BN - 1) / LP_BN);
  int grid = tiles < num_sms ? tiles : num_sms;
  lmhead_dlogits_kernel<<<grid, GEMM_THREADS, SM::TOTAL, stream>>>(tmA, tmB, T, Vc, H, ep, status);
  return cudaGetLastError() == cudaSuccess ? 0 : B200_ERR_LAUNCH;
}

}  // extern "C"
