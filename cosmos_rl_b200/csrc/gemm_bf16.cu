// Dense bf16 GEMM on tcgen05/TMEM:  C[M,N] = A[M,K] * B[N,K]^T  (+ optional fp32 accumulate-into).
// A and B are row-major with K contiguous (the layout of activations x and nn.Linear weights),
// C is row-major bf16 or fp32. Building block for the fused kernels of this library; replaces
// the library GEMM the reference reaches through nn.Linear (cosmos_rl/policy/model/gpt/__init__.py:284-316).
#include "gemm_core.cuh"
#include "gemm_2cta.cuh"
#include "api.h"

namespace b200 {

struct StoreEpilogue {
  struct Params {
    void* C;
    long long ldc;
    int M, N;
    int out_fp32;     // 0: bf16, 1: fp32
    int accumulate;   // C += result
    int bn;
  };
  __device__ __forceinline__ void tile_begin(const Params&, const TileInfo&, int) {}
  __device__ __forceinline__ void tile_end(const Params&, const TileInfo&, int) {}
  __device__ __forceinline__ void finish(const Params&) {}
  __device__ __forceinline__ void chunk(const Params& p, const TileInfo& t, int row, int col0, const float (&v)[32]) {
    store_chunk(p.C, p.ldc, p.M, p.N, p.out_fp32, p.accumulate, (long long)t.m_blk * GEMM_BM + row,
                t.n_blk * p.bn + col0, v);
  }
  // shared with the grouped GEMM epilogue
  static __device__ __forceinline__ void store_chunk(void* C, long long ldc, long long M, int N, int out_fp32,
                                                     int accumulate, long long r, int c, const float (&v)[32]) {
    if (r >= M || c >= N) return;
    if (out_fp32) {
      float* dst = reinterpret_cast<float*>(C) + r * ldc + c;
      if (c + 32 <= N && ((reinterpret_cast<uintptr_t>(dst) & 15) == 0)) {
#pragma unroll
        for (int i = 0; i < 32; i += 4) {
          float4 o = make_float4(v[i], v[i + 1], v[i + 2], v[i + 3]);
          if (accumulate) {
            float4 old = *reinterpret_cast<float4*>(dst + i);
            o.x += old.x; o.y += old.y; o.z += old.z; o.w += old.w;
          }
          *reinterpret_cast<float4*>(dst + i) = o;
        }
      } else {
        for (int i = 0; i < 32 && c + i < N; ++i) dst[i] = accumulate ? dst[i] + v[i] : v[i];
      }
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

template <int BN, int STAGES, bool A_MN, bool B_MN>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
gemm_bf16_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, int M, int N, int K,
                 StoreEpilogue::Params ep, uint32_t* status) {
  gemm_mainloop<BN, STAGES, StoreEpilogue, RasterSchedule, GemmTraits<A_MN, B_MN>>(&tmA, &tmB, M, N, K, ep, status);
}

template <int BN, int STAGES, bool A_MN, bool B_MN>
static int launch_gemm(const void* A, const void* B, void* C, int M, int N, int K, long long lda, long long ldb,
                       long long ldc, int out_fp32, int accumulate, uint32_t* status, int num_sms,
                       cudaStream_t stream) {
  CUtensorMap tmA, tmB;
  // K-major operand: stored [MN, K], box = (tile rows) x 64 contraction elements.
  // MN-major operand: stored [K, MN], box = 64 contraction rows x 64 MN elements.
  if (A_MN ? make_tmap_2d(&tmA, A, K, M, lda, 64, 64, 2) : make_tmap_2d(&tmA, A, M, K, lda, GEMM_BM, GEMM_BK, 2))
    return B200_ERR_TENSORMAP;
  if (B_MN ? make_tmap_2d(&tmB, B, K, N, ldb, 64, 64, 2) : make_tmap_2d(&tmB, B, N, K, ldb, BN, GEMM_BK, 2))
    return B200_ERR_TENSORMAP;
  using SM = GemmSmem<BN, STAGES>;
  auto kern = gemm_bf16_kernel<BN, STAGES, A_MN, B_MN>;
  static bool attr_set = false;
  if (!attr_set) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SM::TOTAL) != cudaSuccess)
      return B200_ERR_LAUNCH;
    attr_set = true;
  }
  StoreEpilogue::Params ep{C, ldc, M, N, out_fp32, accumulate, BN};
  int tiles = ((M + GEMM_BM - 1) / GEMM_BM) * ((N + BN - 1) / BN);
  int grid = tiles < num_sms ? tiles : num_sms;
  kern<<<grid, GEMM_THREADS, SM::TOTAL, stream>>>(tmA, tmB, M, N, K, ep, status);
  return cudaGetLastError() == cudaSuccess ? 0 : B200_ERR_LAUNCH;
}

template <bool A_MN, bool B_MN>
static int dispatch_bn(const void* A, const void* B, void* C, int M, int N, int K, long long lda, long long ldb,
                       long long ldc, int out_fp32, int accumulate, uint32_t* status, int num_sms, cudaStream_t stream) {
  // Wide tiles amortise shared-memory traffic; narrow N uses the 128-wide tile.
  if (N >= 256)
    return launch_gemm<256, 4, A_MN, B_MN>(A, B, C, M, N, K, lda, ldb, ldc, out_fp32, accumulate, status, num_sms, stream);
  return launch_gemm<128, 6, A_MN, B_MN>(A, B, C, M, N, K, lda, ldb, ldc, out_fp32, accumulate, status, num_sms, stream);
}

// ---------------------------------------------------------------------------------------------------
// CTA-pair kernel (256 x BN tiles over two SMs); see gemm_2cta.cuh
// ---------------------------------------------------------------------------------------------------
template <int BN, int STAGES, bool A_MN, bool B_MN, int EPI>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(G2_THREADS, 1)
gemm2_bf16_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                  const __grid_constant__ CUtensorMap tmC, int M, int N, int K, Gemm2Params ep, uint32_t* status) {
  gemm2_mainloop<BN, STAGES, A_MN, B_MN, EPI>(&tmA, &tmB, &tmC, M, N, K, ep, status);
}

// How many CTA pairs can be resident at once (asked once per kernel and device; <= num_sms / 2).
template <class Kern>
static int max_pairs(Kern kern, int smem_bytes, int num_sms) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(2 * (num_sms / 2), 1, 1);
  cfg.blockDim = dim3(G2_THREADS, 1, 1);
  cfg.dynamicSmemBytes = smem_bytes;
  cudaLaunchAttribute at[1];
  at[0].id = cudaLaunchAttributeClusterDimension;
  at[0].val.clusterDim.x = 2;
  at[0].val.clusterDim.y = 1;
  at[0].val.clusterDim.z = 1;
  cfg.attrs = at;
  cfg.numAttrs = 1;
  int n = 0;
  if (cudaOccupancyMaxActiveClusters(&n, kern, &cfg) != cudaSuccess || n <= 0) {
    (void)cudaGetLastError();
    n = num_sms / 2;
  }
  return n < num_sms / 2 ? n : num_sms / 2;
}

template <int BN, int STAGES, bool A_MN, bool B_MN, int EPI>
static int launch_gemm2(const void* A, const void* B, void* C, int M, int N, int K, long long lda, long long ldb,
                        long long ldc, const Gemm2Params& ep, uint32_t* status, int num_sms, cudaStream_t stream) {
  CUtensorMap tmA, tmB, tmC;
  if (A_MN ? make_tmap_2d(&tmA, A, K, M, lda, 64, 64, 2) : make_tmap_2d(&tmA, A, M, K, lda, G2_BM_CTA, G2_BK, 2))
    return B200_ERR_TENSORMAP;
  if (B_MN ? make_tmap_2d(&tmB, B, K, N, ldb, 64, 64, 2) : make_tmap_2d(&tmB, B, N, K, ldb, BN / 2, G2_BK, 2))
    return B200_ERR_TENSORMAP;
  const int n_cols = EPI == G2_EPI_SWIGLU ? N / 2 : N;
  if (make_tmap_out(&tmC, C, M, n_cols, ldc, ep.out_fp32)) return B200_ERR_TENSORMAP;
  using SM = Gemm2Smem<BN, STAGES>;
  auto kern = gemm2_bf16_kernel<BN, STAGES, A_MN, B_MN, EPI>;
  static int pairs[16] = {0};  // per device
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 16) return B200_ERR_RUNTIME;
  if (pairs[dev] == 0) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SM::TOTAL) != cudaSuccess)
      return B200_ERR_LAUNCH;
    pairs[dev] = max_pairs(kern, SM::TOTAL, num_sms);
  }
  constexpr int OUT_BN = EPI == G2_EPI_SWIGLU ? BN / 2 : BN;
  const int tiles = ((M + G2_BM - 1) / G2_BM) * ((n_cols + OUT_BN - 1) / OUT_BN);
  int np = pairs[dev];
  if (num_sms / 2 < np) np = num_sms / 2;  // the caller may reserve SMs for kernels on other streams
  if (np < 1) np = 1;
  const int grid = 2 * (tiles < np ? tiles : np);
  kern<<<grid, G2_THREADS, SM::TOTAL, stream>>>(tmA, tmB, tmC, M, N, K, ep, status);
  return cudaGetLastError() == cudaSuccess ? 0 : B200_ERR_LAUNCH;
}

template <bool A_MN, bool B_MN>
static int dispatch_gemm2(const void* A, const void* B, void* C, int M, int N, int K, long long lda, long long ldb,
                          long long ldc, const Gemm2Params& ep, int epi, uint32_t* status, int num_sms,
                          cudaStream_t stream) {
  if (epi == G2_EPI_SWIGLU) {
    if constexpr (!A_MN && !B_MN)
      return launch_gemm2<256, 6, false, false, G2_EPI_SWIGLU>(A, B, C, M, N, K, lda, ldb, ldc, ep, status, num_sms, stream);
    else
      return B200_ERR_ARG;
  }
  if (N > 128)
    return launch_gemm2<256, 6, A_MN, B_MN, G2_EPI_STORE>(A, B, C, M, N, K, lda, ldb, ldc, ep, status, num_sms, stream);
  return launch_gemm2<128, 8, A_MN, B_MN, G2_EPI_STORE>(A, B, C, M, N, K, lda, ldb, ldc, ep, status, num_sms, stream);
}

static bool pair_kernel_usable(const void* C, int M, long long ldc, int out_fp32) {
  const int eb = out_fp32 ? 4 : 2;
  return M > 128 && (reinterpret_cast<uintptr_t>(C) & 15) == 0 && ((ldc * eb) & 15) == 0;
}

}  // namespace b200

// C[M,N] (+)= op(A) * op(B)^T with fp32 accumulation.
//   a_mn = 0: A stored [M, K] (lda = row stride)      a_mn = 1: A stored [K, M]
//   b_mn = 0: B stored [N, K] (ldb = row stride)      b_mn = 1: B stored [K, N]
// forward  y = x W^T      : a_mn 0, b_mn 0        dgrad dx = dy W : a_mn 0, b_mn 1 (W stored [N_contract, K_out])
// wgrad dW = dy^T x       : a_mn 1, b_mn 1 (both stored [tokens, features])
// (reason << 24) | CUresult of the last tensor-map encode that failed in this process (0: none); see gemm_core.cuh
extern "C" int b200_last_tmap_error() { return b200::last_tmap_error(); }

extern "C" int b200_gemm_bf16_ex(const void* A, const void* B, void* C, int M, int N, int K, long long lda,
                                 long long ldb, long long ldc, int a_mn, int b_mn, int out_fp32, int accumulate,
                                 const void* bias, int bias_bf16, int epilogue, int up_row0, int path,
                                 uint32_t* status, int num_sms, cudaStream_t stream) {
  if (M <= 0 || N <= 0 || K <= 0) return B200_ERR_ARG;
  // TMA needs 16-byte aligned row strides; MN-major tiles are fetched in 64-element columns
  if ((lda & 7) || (ldb & 7)) return B200_ERR_ARG;
  using namespace b200;
  const bool want_pair = path != 1 && pair_kernel_usable(C, M, ldc, out_fp32);
  if (epilogue == G2_EPI_SWIGLU || bias != nullptr || path == 2) {
    // epilogues that only the CTA-pair kernel has
    if (!pair_kernel_usable(C, 129, ldc, out_fp32)) return B200_ERR_ARG;
    if (epilogue == G2_EPI_SWIGLU && (a_mn || b_mn || (N & 1) || accumulate)) return B200_ERR_ARG;
  }
  if (want_pair || epilogue == G2_EPI_SWIGLU || bias != nullptr || path == 2) {
    Gemm2Params ep{bias, bias_bf16, out_fp32, accumulate, up_row0, 8};
    if (!a_mn && !b_mn) return dispatch_gemm2<false, false>(A, B, C, M, N, K, lda, ldb, ldc, ep, epilogue, status, num_sms, stream);
    if (!a_mn && b_mn) return dispatch_gemm2<false, true>(A, B, C, M, N, K, lda, ldb, ldc, ep, epilogue, status, num_sms, stream);
    if (a_mn && b_mn) return dispatch_gemm2<true, true>(A, B, C, M, N, K, lda, ldb, ldc, ep, epilogue, status, num_sms, stream);
    return dispatch_gemm2<true, false>(A, B, C, M, N, K, lda, ldb, ldc, ep, epilogue, status, num_sms, stream);
  }
  if (!a_mn && !b_mn) return dispatch_bn<false, false>(A, B, C, M, N, K, lda, ldb, ldc, out_fp32, accumulate, status, num_sms, stream);
  if (!a_mn && b_mn) return dispatch_bn<false, true>(A, B, C, M, N, K, lda, ldb, ldc, out_fp32, accumulate, status, num_sms, stream);
  if (a_mn && b_mn) return dispatch_bn<true, true>(A, B, C, M, N, K, lda, ldb, ldc, out_fp32, accumulate, status, num_sms, stream);
  return dispatch_bn<true, false>(A, B, C, M, N, K, lda, ldb, ldc, out_fp32, accumulate, status, num_sms, stream);
}

extern "C" int b200_gemm_bf16(const void* A, const void* B, void* C, int M, int N, int K, long long lda,
                              long long ldb, long long ldc, int a_mn, int b_mn, int out_fp32, int accumulate,
                              uint32_t* status, int num_sms, cudaStream_t stream) {
  return b200_gemm_bf16_ex(A, B, C, M, N, K, lda, ldb, ldc, a_mn, b_mn, out_fp32, accumulate, nullptr, 0, 0, 0, 0,
                           status, num_sms, stream);
}

extern "C" int b200_gemm_bf16_nt(const void* A, const void* B, void* C, int M, int N, int K, long long lda,
                                 long long ldb, long long ldc, int out_fp32, int accumulate, uint32_t* status,
                                 int num_sms, cudaStream_t stream) {
  return b200_gemm_bf16(A, B, C, M, N, K, lda, ldb, ldc, 0, 0, out_fp32, accumulate, status, num_sms, stream);
}
