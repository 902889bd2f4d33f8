// Dense bf16 GEMM on tcgen05/TMEM:  C[M,N] = A[M,K] * B[N,K]^T  (+ optional fp32 accumulate-into).
// A and B are row-major with K contiguous (the layout of activations x and nn.Linear weights),
// C is row-major bf16 or fp32. Building block for the fused kernels of this library; replaces
// the library GEMM the reference reaches through nn.Linear (cosmos_rl/policy/model/gpt/__init__.py:284-316).
#include "gemm_core.cuh"
#include "api.h"

namespace b200 {

struct StoreEpilogue {
  struct Params {
    void* C;
    long long ldc;
    int M, N;
    int out_fp32;     // 0: bf16, 1: fp32
    int accumulate;   // C += result (fp32 output only)
    int bn;
  };
  __device__ __forceinline__ void tile_begin(const Params&, int, int, int) {}
  __device__ __forceinline__ void tile_end(const Params&, int, int, int) {}
  __device__ __forceinline__ void finish(const Params&) {}
  __device__ __forceinline__ void chunk(const Params& p, int m_blk, int n_blk, int row, int col0,
                                        const float (&v)[32]) {
    const long long r = (long long)m_blk * GEMM_BM + row;
    const int c = n_blk * p.bn + col0;
    if (r >= p.M || c >= p.N) return;
    if (p.out_fp32) {
      float* dst = reinterpret_cast<float*>(p.C) + r * p.ldc + c;
      if (c + 32 <= p.N && ((reinterpret_cast<uintptr_t>(dst) & 15) == 0)) {
#pragma unroll
        for (int i = 0; i < 32; i += 4) {
          float4 o = make_float4(v[i], v[i + 1], v[i + 2], v[i + 3]);
          if (p.accumulate) {
            float4 old = *reinterpret_cast<float4*>(dst + i);
            o.x += old.x; o.y += old.y; o.z += old.z; o.w += old.w;
          }
          *reinterpret_cast<float4*>(dst + i) = o;
        }
      } else {
        for (int i = 0; i < 32 && c + i < p.N; ++i) dst[i] = p.accumulate ? dst[i] + v[i] : v[i];
      }
    } else {
      __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(p.C) + r * p.ldc + c;
      if (c + 32 <= p.N && ((reinterpret_cast<uintptr_t>(dst) & 15) == 0)) {
#pragma unroll
        for (int i = 0; i < 32; i += 8) {
          uint4 o;
          o.x = pack_bf16x2(v[i], v[i + 1]);
          o.y = pack_bf16x2(v[i + 2], v[i + 3]);
          o.z = pack_bf16x2(v[i + 4], v[i + 5]);
          o.w = pack_bf16x2(v[i + 6], v[i + 7]);
          *reinterpret_cast<uint4*>(dst + i) = o;
        }
      } else {
        for (int i = 0; i < 32 && c + i < p.N; ++i) dst[i] = __float2bfloat16(v[i]);
      }
    }
  }
};

template <int BN, int STAGES>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
gemm_bf16_nt_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, int M, int N,
                    int K, StoreEpilogue::Params ep, uint32_t* status) {
  gemm_mainloop<BN, STAGES, StoreEpilogue, RasterSchedule>(&tmA, &tmB, M, N, K, ep, status);
}

template <int BN, int STAGES>
static int launch_gemm(const void* A, const void* B, void* C, int M, int N, int K, long long lda, long long ldb,
                       long long ldc, int out_fp32, int accumulate, uint32_t* status, int num_sms,
                       cudaStream_t stream) {
  CUtensorMap tmA, tmB;
  if (make_tmap_2d(&tmA, A, M, K, lda, GEMM_BM, GEMM_BK, 2)) return B200_ERR_TENSORMAP;
  if (make_tmap_2d(&tmB, B, N, K, ldb, BN, GEMM_BK, 2)) return B200_ERR_TENSORMAP;
  using SM = GemmSmem<BN, STAGES>;
  auto kern = gemm_bf16_nt_kernel<BN, STAGES>;
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

}  // namespace b200

extern "C" int b200_gemm_bf16_nt(const void* A, const void* B, void* C, int M, int N, int K, long long lda,
                                 long long ldb, long long ldc, int out_fp32, int accumulate, uint32_t* status,
                                 int num_sms, cudaStream_t stream) {
  if (M <= 0 || N <= 0 || K <= 0 || (K & 7)) return B200_ERR_ARG;
  if (accumulate && !out_fp32) return B200_ERR_ARG;
  // Wide tiles amortise shared-memory traffic; narrow N (decode-time projections) uses the 128-wide tile.
  if (N >= 256)
    return b200::launch_gemm<256, 4>(A, B, C, M, N, K, lda, ldb, ldc, out_fp32, accumulate, status, num_sms, stream);
  return b200::launch_gemm<128, 6>(A, B, C, M, N, K, lda, ldb, ldc, out_fp32, accumulate, status, num_sms, stream);
}
