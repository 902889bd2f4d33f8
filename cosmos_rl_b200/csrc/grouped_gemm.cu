// Grouped (per-expert) bf16 GEMMs for mixture-of-experts layers on tcgen05/TMEM, replacing the
// grouped_gemm / torch._grouped_mm library calls of the reference (cosmos_rl/policy/kernel/moe/moe.py:420-443,
// moe/grouped_gemm.py:33-165).
//
// Tokens routed to the local experts are stored sorted by expert in one [Mp, *] buffer in which every
// expert's block starts on a multiple of 128 rows (padding rows are zero). Then a 128-row output tile belongs
// to exactly one expert and a 64-row contraction block never straddles two experts, so all three GEMMs run on
// the dense pipeline of gemm_core.cuh with a different tile schedule and 3-D tensor maps over the stacked
// expert weights [E, N, K]:
//   forward  Y[Mp, N]   = X[Mp, K] . W[e]^T                      (A 2-D K-major, B 3-D K-major, z = expert)
//   dgrad    dX[Mp, K]  = dY[Mp, N] . W[e]                       (A 2-D K-major, B 3-D MN-major)
//   wgrad    dW[e][N,K] (+)= dY[rows of e]^T . X[rows of e]      (A, B 2-D MN-major, contraction = the expert's rows)
// Tile counts and expert boundaries are read from device memory (tile_expert / expert_offsets / n_tiles), so
// no host synchronisation sits between routing and the expert GEMMs.
#include "gemm_core.cuh"
#include "api.h"

namespace b200 {

struct GroupedParams {
  void* C;
  long long ldc;
  long long c_batch_stride;   // wgrad: elements between dW[e] and dW[e+1]
  int N;                      // output columns
  int rows_limit;             // fwd/dgrad: allocated rows of C; wgrad: output rows per expert
  int out_fp32, accumulate, bn;
  const int* tile_expert;     // [max_tiles] expert of each 128-row tile (fwd/dgrad)
  const int* expert_offsets;  // [E + 1] padded row offsets (wgrad)
  const int* n_tiles;         // [1] number of 128-row tiles in use
  int num_experts;
  int K;                      // contraction length (fwd/dgrad)
};

struct GroupedEpilogue {
  using Params = GroupedParams;
  __device__ __forceinline__ void tile_begin(const Params&, const TileInfo&, int) {}
  __device__ __forceinline__ void tile_end(const Params&, const TileInfo&, int) {}
  __device__ __forceinline__ void finish(const Params&) {}
  __device__ __forceinline__ void chunk(const Params& p, const TileInfo& t, int row, int col0, const float (&v)[32]) {
    // forward / dgrad: batch offset is zero and m_blk indexes the padded token rows;
    // wgrad: m_blk indexes rows of dW[e] and the expert selects the slice.
    char* base = reinterpret_cast<char*>(p.C) + (long long)(p.c_batch_stride ? t.batch : 0) * p.c_batch_stride *
                                                    (p.out_fp32 ? 4 : 2);
    StoreEpilogue_store(base, p.ldc, p.rows_limit, p.N, p.out_fp32, p.accumulate, (long long)t.m_blk * GEMM_BM + row,
                        t.n_blk * p.bn + col0, v);
  }
  static __device__ __forceinline__ void StoreEpilogue_store(void* C, long long ldc, long long M, int N, int out_fp32,
                                                             int accumulate, long long r, int c,
                                                             const float (&v)[32]) {
    if (r >= M || c >= N) return;
    if (out_fp32) {
      float* dst = reinterpret_cast<float*>(C) + r * ldc + c;
      for (int i = 0; i < 32 && c + i < N; ++i) dst[i] = accumulate ? dst[i] + v[i] : v[i];
    } else {
      __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(C) + r * ldc + c;
      if (c + 32 <= N && ((reinterpret_cast<uintptr_t>(dst) & 15) == 0)) {
#pragma unroll
        for (int i = 0; i < 32; i += 8) {
          float w[8];
#pragma unroll
          for (int j = 0; j < 8; ++j) w[j] = v[i + j];
          if (accumulate) {
            uint4 old = *reinterpret_cast<uint4*>(dst + i);
            const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&old);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              float2 f = __bfloat1622float2(h[j]);
              w[2 * j] += f.x;
              w[2 * j + 1] += f.y;
            }
          }
          uint4 o;
          o.x = pack_bf16x2(w[0], w[1]);
          o.y = pack_bf16x2(w[2], w[3]);
          o.z = pack_bf16x2(w[4], w[5]);
          o.w = pack_bf16x2(w[6], w[7]);
          *reinterpret_cast<uint4*>(dst + i) = o;
        }
      } else {
        for (int i = 0; i < 32 && c + i < N; ++i)
          dst[i] = __float2bfloat16(accumulate ? __bfloat162float(dst[i]) + v[i] : v[i]);
      }
    }
  }
};

// forward / dgrad: tiles = (128-row tile of the padded token buffer) x (BN-column tile)
struct TokenTileSchedule {
  int num_n, total, num_kb, bn;
  const int* tile_expert;
  __device__ __forceinline__ void init(int, int N, int K, int BN, const GroupedParams& p) {
    num_n = (N + BN - 1) / BN;
    total = p.n_tiles[0] * num_n;
    num_kb = (K + GEMM_BK - 1) / GEMM_BK;
    tile_expert = p.tile_expert;
    bn = BN;
  }
  __device__ __forceinline__ bool get(int it, TileInfo& t) const {
    int i = blockIdx.x + it * gridDim.x;
    if (i >= total) return false;
    // n fastest: CTAs running at the same time share the token tile's expert, i.e. the same weight slice in L2
    t.m_blk = i / num_n;
    t.n_blk = i - t.m_blk * num_n;
    t.a_mn0 = t.m_blk * GEMM_BM;
    t.b_mn0 = t.n_blk * bn;
    t.k0 = 0;
    t.num_kb = num_kb;
    t.batch = tile_expert[t.m_blk];
    return true;
  }
};

// wgrad: tiles = expert x (128-row tile of dW) x (BN-column tile of dW); contraction over the expert's rows
struct ExpertWgradSchedule {
  int num_m, num_n, per_expert, total, bn;
  const int* off;
  __device__ __forceinline__ void init(int M, int N, int, int BN, const GroupedParams& p) {
    num_m = (M + GEMM_BM - 1) / GEMM_BM;
    num_n = (N + BN - 1) / BN;
    per_expert = num_m * num_n;
    total = per_expert * p.num_experts;
    off = p.expert_offsets;
    bn = BN;
  }
  __device__ __forceinline__ bool get(int it, TileInfo& t) const {
    int i = blockIdx.x + it * gridDim.x;
    if (i >= total) return false;
    const int e = i / per_expert, r = i - e * per_expert;
    t.m_blk = r / num_n;
    t.n_blk = r - t.m_blk * num_n;
    t.a_mn0 = t.m_blk * GEMM_BM;
    t.b_mn0 = t.n_blk * bn;
    t.k0 = off[e];
    t.num_kb = (off[e + 1] - off[e]) / GEMM_BK;
    t.batch = e;
    return true;
  }
};

constexpr int GG_BN = 256, GG_STAGES = 4;

__global__ void __launch_bounds__(GEMM_THREADS, 1)
grouped_fwd_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, int M, int N,
                   int K, GroupedParams ep, uint32_t* status) {
  gemm_mainloop<GG_BN, GG_STAGES, GroupedEpilogue, TokenTileSchedule, GemmTraits<false, false, false, true>>(
      &tmA, &tmB, M, N, K, ep, status);
}
__global__ void __launch_bounds__(GEMM_THREADS, 1)
grouped_dgrad_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, int M, int N,
                     int K, GroupedParams ep, uint32_t* status) {
  gemm_mainloop<GG_BN, GG_STAGES, GroupedEpilogue, TokenTileSchedule, GemmTraits<false, true, false, true>>(
      &tmA, &tmB, M, N, K, ep, status);
}
__global__ void __launch_bounds__(GEMM_THREADS, 1)
grouped_wgrad_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, int M, int N,
                     int K, GroupedParams ep, uint32_t* status) {
  gemm_mainloop<GG_BN, GG_STAGES, GroupedEpilogue, ExpertWgradSchedule, GemmTraits<true, true>>(&tmA, &tmB, M, N, K,
                                                                                                  ep, status);
}

template <class Kern>
static int set_smem(Kern k, bool& done) {
  if (!done) {
    if (cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, GemmSmem<GG_BN, GG_STAGES>::TOTAL) !=
        cudaSuccess)
      return B200_ERR_LAUNCH;
    done = true;
  }
  return 0;
}

}  // namespace b200

extern "C" {

// mode 0: Y[Mp, N] = X[Mp, K] . W[e]^T with W [E, N, K]
// mode 1: dX[Mp, N] = dY[Mp, K] . W[e]   with W [E, K, N]   (K is the contraction = rows of W[e])
int b200_grouped_gemm(const void* X, const void* W, void* Y, int max_rows, int N, int K, int num_experts,
                      long long ldx, long long ldy, const int* tile_expert, const int* n_tiles, int mode,
                      int accumulate, uint32_t* status, int num_sms, cudaStream_t stream) {
  using namespace b200;
  if (max_rows <= 0 || N <= 0 || K <= 0 || (ldx & 7) || (max_rows % GEMM_BM)) return B200_ERR_ARG;
  CUtensorMap tmA, tmB;
  if (make_tmap_2d(&tmA, X, max_rows, K, ldx, GEMM_BM, GEMM_BK, 2)) return B200_ERR_TENSORMAP;
  static bool s0 = false, s1 = false;
  GroupedParams ep{Y, ldy, 0, N, max_rows, 0, accumulate, GG_BN, tile_expert, nullptr, n_tiles, num_experts, K};
  const int grid = num_sms;
  if (mode == 0) {
    if (make_tmap_3d(&tmB, W, num_experts, N, K, K, (uint64_t)N * K, GG_BN, GEMM_BK, 2)) return B200_ERR_TENSORMAP;
    if (set_smem(grouped_fwd_kernel, s0)) return B200_ERR_LAUNCH;
    grouped_fwd_kernel<<<grid, GEMM_THREADS, GemmSmem<GG_BN, GG_STAGES>::TOTAL, stream>>>(tmA, tmB, max_rows, N, K, ep,
                                                                                          status);
  } else {
    // W[e] stored [K(contraction), N(out)]: MN-major B, boxes of 64 contraction rows x 64 output columns
    if (make_tmap_3d(&tmB, W, num_experts, K, N, N, (uint64_t)N * K, 64, 64, 2)) return B200_ERR_TENSORMAP;
    if (set_smem(grouped_dgrad_kernel, s1)) return B200_ERR_LAUNCH;
    grouped_dgrad_kernel<<<grid, GEMM_THREADS, GemmSmem<GG_BN, GG_STAGES>::TOTAL, stream>>>(tmA, tmB, max_rows, N, K,
                                                                                            ep, status);
  }
  return cudaGetLastError() == cudaSuccess ? 0 : B200_ERR_LAUNCH;
}

// dW[e][N, K] (+)= dY[rows of e, N]^T . X[rows of e, K]; rows of e = [expert_offsets[e], expert_offsets[e+1])
int b200_grouped_wgrad(const void* dY, const void* X, void* dW, int max_rows, int N, int K, int num_experts,
                       long long lddy, long long ldx, const int* expert_offsets, int out_fp32, int accumulate,
                       uint32_t* status, int num_sms, cudaStream_t stream) {
  using namespace b200;
  if (max_rows <= 0 || N <= 0 || K <= 0 || (lddy & 7) || (ldx & 7)) return B200_ERR_ARG;
  CUtensorMap tmA, tmB;
  if (make_tmap_2d(&tmA, dY, max_rows, N, lddy, 64, 64, 2)) return B200_ERR_TENSORMAP;
  if (make_tmap_2d(&tmB, X, max_rows, K, ldx, 64, 64, 2)) return B200_ERR_TENSORMAP;
  static bool s2 = false;
  if (set_smem(grouped_wgrad_kernel, s2)) return B200_ERR_LAUNCH;
  GroupedParams ep{dW, K, (long long)N * K, K, N, out_fp32, accumulate, GG_BN, nullptr, expert_offsets, nullptr,
                   num_experts, 0};
  grouped_wgrad_kernel<<<num_sms, GEMM_THREADS, GemmSmem<GG_BN, GG_STAGES>::TOTAL, stream>>>(tmA, tmB, N, K, 0, ep,
                                                                                            status);
  return cudaGetLastError() == cudaSuccess ? 0 : B200_ERR_LAUNCH;
}

}  // extern "C"
