// Block-scaled fp8 (e4m3) GEMM on tcgen05:  C[M,N] = sum_kb  sa[m, kb] * sb[n / 128, kb] * (A_kb * B_kb^T)
// with A [M,K] e4m3 + one fp32 scale per 1 x 128 block (activations), B [N,K] e4m3 + one fp32 scale per
// 128 x 128 block (weights), fp32 accumulation, bf16 output. This is the scaling scheme of the reference's
// DeepSeek-style fp8 path (cosmos_rl/policy/kernel/moe/moe.py block-scaled grouped GEMM,
// cosmos_rl/utils/fp8/fp8_util.py:21-153 for dense layers).
//
// The tensor core cannot apply a different fp32 scale per 128-wide slice of K inside one accumulation, so the
// kernel accumulates in two levels: each 128-deep k-block (four kind::f8f6f4 MMAs of K = 32 on a 128 x 128 tile)
// goes into one of two TMEM buffers with accumulate = 0; eight promotion warps (two per TMEM lane quadrant, 64
// columns each) read the finished buffer, multiply by the block's scale product and add into fp32 registers while
// the tensor core is already filling the other buffer. Operands arrive by TMA (128-byte swizzle, a 128-byte row =
// 128 fp8 elements) through a 6-stage ring. Persistent CTAs, bounded waits.
#include "gemm_core.cuh"
#include "api.h"

namespace b200 {

constexpr int F8_BM = 128, F8_BN = 128, F8_BK = 128;
constexpr int F8_STAGES = 6;
constexpr int F8_STAGE_BYTES = (F8_BM + F8_BN) * F8_BK;     // 32 KiB
constexpr int F8_SMEM = F8_STAGES * F8_STAGE_BYTES + 256 + 1024;
constexpr int F8_THREADS = 64 + 256;                         // TMA warp, MMA warp, 8 promotion warps

struct F8Params {
  const float* sa;       // [M, ldsa]  (ldsa >= ceil(K / 128))
  const float* sb;       // [ceil(N / 128), ldsb]
  __nv_bfloat16* C;
  long long ldc;
  int M, N, K, ldsa, ldsb;
  uint32_t* status;
};

__global__ void __launch_bounds__(F8_THREADS, 1)
gemm_fp8_block_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, F8Params p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + F8_STAGES * F8_STAGE_BYTES);
  uint64_t* empty_bar = full_bar + F8_STAGES;
  uint64_t* pfull = empty_bar + F8_STAGES;    // [2] partial accumulator ready
  uint64_t* pempty = pfull + 2;               // [2] partial accumulator consumed (8 warps)
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(pempty + 2);
  volatile uint32_t* abort_flag = tmem_slot + 1;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    for (int s = 0; s < F8_STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&pfull[a], 1);
      mbar_init(&pempty[a], 8);
    }
    *abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmB);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, 256);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  const int num_m = (p.M + F8_BM - 1) / F8_BM, num_n = (p.N + F8_BN - 1) / F8_BN;
  const int total = num_m * num_n;
  const int num_kb = (p.K + F8_BK - 1) / F8_BK;
  auto tile_of = [&](int i, int& m_blk, int& n_blk) {
    constexpr int G = 8;
    const int group = i / (G * num_n), first_m = group * G;
    const int gsz = min(num_m - first_m, G);
    const int r = i - group * G * num_n;
    m_blk = first_m + r % gsz;
    n_blk = r / gsz;
  };

  if (warp == 0) {
    if (lane == 0) {
      uint32_t stage = 0, phase = 0;
      for (int i = blockIdx.x; i < total && !*abort_flag; i += gridDim.x) {
        int m_blk, n_blk;
        tile_of(i, m_blk, n_blk);
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(&empty_bar[stage], phase ^ 1)) { atomicCAS(p.status, ST_OK, ST_TIMEOUT_EMPTY); *abort_flag = 1; break; }
          uint8_t* sa = smem + stage * F8_STAGE_BYTES;
          mbar_arrive_expect_tx(&full_bar[stage], F8_STAGE_BYTES);
          tma_load_2d(sa, &tmA, &full_bar[stage], kb * F8_BK, m_blk * F8_BM);
          tma_load_2d(sa + F8_BM * F8_BK, &tmB, &full_bar[stage], kb * F8_BK, n_blk * F8_BN);
          if (++stage == F8_STAGES) { stage = 0; phase ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc = umma_idesc_e4m3_f32(F8_BM, F8_BN);
      uint32_t stage = 0, phase = 0, it = 0;
      bool ok = true;
      for (int i = blockIdx.x; i < total && ok && !*abort_flag; i += gridDim.x) {
        for (int kb = 0; kb < num_kb; ++kb, ++it) {
          const uint32_t buf = it & 1, bph = (it >> 1) & 1;
          if (!mbar_wait(&pempty[buf], bph ^ 1)) { atomicCAS(p.status, ST_OK, ST_TIMEOUT_TMEM_EMPTY); *abort_flag = 1; ok = false; break; }
          if (!mbar_wait(&full_bar[stage], phase)) { atomicCAS(p.status, ST_OK, ST_TIMEOUT_FULL); *abort_flag = 1; ok = false; break; }
          tc_fence_after_sync();
          const uint32_t sa = smem_u32(smem + stage * F8_STAGE_BYTES), sb = sa + F8_BM * F8_BK;
#pragma unroll
          for (int k = 0; k < F8_BK / 32; ++k)
            umma_f8_ss(tmem_base + buf * F8_BN, umma_desc_kmajor_sw128(sa + k * 32), umma_desc_kmajor_sw128(sb + k * 32),
                       idesc, k > 0 ? 1u : 0u);
          tc_commit(&empty_bar[stage]);
          tc_commit(&pfull[buf]);
          if (++stage == F8_STAGES) { stage = 0; phase ^= 1; }
        }
      }
    }
  } else {
    // promotion warps: quadrant = warp % 4 (TMEM lanes), column half = (warp - 2) / 4
    const int quad = warp & 3, chalf = (warp - 2) >> 2;
    const int row = quad * 32 + lane;
    const uint32_t lane_addr = (uint32_t)(quad * 32) << 16;
    uint32_t it = 0;
    bool ok = true;
    for (int i = blockIdx.x; i < total && ok; i += gridDim.x) {
      int m_blk, n_blk;
      tile_of(i, m_blk, n_blk);
      const long long grow = (long long)m_blk * F8_BM + row;
      const float* sa_row = p.sa + (grow < p.M ? grow : 0) * p.ldsa;
      const float* sb_row = p.sb + (long long)n_blk * p.ldsb;
      float acc[64];
#pragma unroll
      for (int c = 0; c < 64; ++c) acc[c] = 0.f;
      float s_next = sa_row[0] * sb_row[0];
      for (int kb = 0; kb < num_kb; ++kb, ++it) {
        const uint32_t buf = it & 1, bph = (it >> 1) & 1;
        const float s = s_next;
        if (kb + 1 < num_kb) s_next = sa_row[kb + 1] * sb_row[kb + 1];
        if (!mbar_wait(&pfull[buf], bph)) { atomicCAS(p.status, ST_OK, ST_TIMEOUT_TMEM_FULL); *abort_flag = 1; ok = false; }
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        tc_fence_after_sync();
#pragma unroll
        for (int c = 0; c < 64; c += 32) {
          uint32_t r[32];
          tmem_ld_32x32b_x32(tmem_base + buf * F8_BN + lane_addr + chalf * 64 + c, r);
          tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 32; ++j) acc[c + j] = fmaf(s, __uint_as_float(r[j]), acc[c + j]);
        }
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive(&pempty[buf]);
      }
      if (!ok) break;
      if (grow < p.M) {
        const int col0 = n_blk * F8_BN + chalf * 64;
        __nv_bfloat16* dst = p.C + grow * p.ldc + col0;
#pragma unroll
        for (int c = 0; c < 64; c += 8) {
          if (col0 + c + 8 <= p.N) {
            uint4 o;
            o.x = pack_bf16x2(acc[c], acc[c + 1]);
            o.y = pack_bf16x2(acc[c + 2], acc[c + 3]);
            o.z = pack_bf16x2(acc[c + 4], acc[c + 5]);
            o.w = pack_bf16x2(acc[c + 6], acc[c + 7]);
            *reinterpret_cast<uint4*>(dst + c) = o;
          } else {
            for (int j = 0; j < 8 && col0 + c + j < p.N; ++j) dst[c + j] = __float2bfloat16(acc[c + j]);
          }
        }
      }
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (*abort_flag && threadIdx.x == 0) {
    for (int i = 0; i < 100; ++i) __nanosleep(1000);
  }
  __syncthreads();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, 256);
  }
}

}  // namespace b200

// A [M,K] e4m3 (row stride lda bytes = elements), sa [M, ldsa] fp32; B [N,K] e4m3, sb [ceil(N/128), ldsb] fp32;
// C [M,N] bf16. K, lda, ldb multiples of 16; ldc multiple of 8.
extern "C" int b200_gemm_fp8_block(const void* A, const float* sa, const void* B, const float* sb, void* C, int M,
                                   int N, int K, long long lda, long long ldb, long long ldc, int ldsa, int ldsb,
                                   uint32_t* status, int num_sms, cudaStream_t stream) {
  using namespace b200;
  if (M <= 0 || N <= 0 || K <= 0 || (lda & 15) || (ldb & 15) || (ldc & 7) || (K & 15)) return B200_ERR_ARG;
  const int nkb = (K + F8_BK - 1) / F8_BK;
  if (ldsa < nkb || ldsb < nkb) return B200_ERR_ARG;
  CUtensorMap tmA, tmB;
  if (make_tmap_2d(&tmA, A, M, K, lda, F8_BM, F8_BK, 1)) return B200_ERR_TENSORMAP;
  if (make_tmap_2d(&tmB, B, N, K, ldb, F8_BN, F8_BK, 1)) return B200_ERR_TENSORMAP;
  static bool attr_set = false;
  if (!attr_set) {
    if (cudaFuncSetAttribute(gemm_fp8_block_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, F8_SMEM) != cudaSuccess)
      return B200_ERR_LAUNCH;
    attr_set = true;
  }
  F8Params p{sa, sb, (__nv_bfloat16*)C, ldc, M, N, K, ldsa, ldsb, status};
  const int tiles = ((M + F8_BM - 1) / F8_BM) * ((N + F8_BN - 1) / F8_BN);
  const int grid = tiles < num_sms ? tiles : num_sms;
  gemm_fp8_block_kernel<<<grid, F8_THREADS, F8_SMEM, stream>>>(tmA, tmB, p);
  return cudaGetLastError() == cudaSuccess ? 0 : B200_ERR_LAUNCH;
}
