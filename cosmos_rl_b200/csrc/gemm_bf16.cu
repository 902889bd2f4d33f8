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

}  // namespace b200

// C[M,N] (+)= op(A) * op(B)^T with fp32 accumulation.
//   a_mn = 0: A stored [M, K] (lda = row stride)      a_mn = 1: A stored [K, M]
//   b_mn = 0: B stored [N, K] (ldb = row stride)      b_mn = 1: B stored [K, N]
// forward  y = x W^T      : a_mn 0, b_mn 0        dgrad dx = dy W : a_mn 0, b_mn 1 (W stored [N_contract, K_out])
// wgrad dW = dy^T x       : a_mn 1, b_mn 1 (both stored [tokens, features])
extern "C" int b200_gemm_bf16(const void* A, const void* B, void* C, int M, int N, int K, long long lda,
                              long long ldb, long long ldc, int a_mn, int b_mn, int out_fp32, int accumulate,
                              uint32_t* status, int num_sms, cudaStream_t stream) {
  if (M <= 0 || N <= 0 || K <= 0) return B200_ERR_ARG;
  // TMA needs 16-byte aligned row strides; MN-major tiles are fetched in 64-element columns
  if ((lda & 7) || (ldb & 7)) return B200_ERR_ARG;
  using namespace b200;
  if (!a_mn && !b_mn) return dispatch_bn<false, false>(A, B, C, M, N, K, lda, ldb, ldc, out_fp32, accumulate, status, num_sms, stream);
  if (!a_mn && b_mn) return dispatch_bn<false, true>(A, B, C, M, N, K, lda, ldb, ldc, out_fp32, accumulate, status, num_sms, stream);
  if (a_mn && b_mn) return dispatch_bn<true, true>(A, B, C, M, N, K, lda, ldb, ldc, out_fp32, accumulate, status, num_sms, stream);
  return dispatch_bn<true, false>(A, B, C, M, N, K, lda, ldb, ldc, out_fp32, accumulate, status, num_sms, stream);
}

extern "C" int b200_gemm_bf16_nt(const void* A, const void* B, void* C, int M, int N, int K, long long lda,
                                 long long ldb, long long ldc, int out_fp32, int accumulate, uint32_t* status,
                                 int num_sms, cudaStream_t stream) {
  return b200_gemm_bf16(A, B, C, M, N, K, lda, ldb, ldc, 0, 0, out_fp32, accumulate, status, num_sms, stream);
}
