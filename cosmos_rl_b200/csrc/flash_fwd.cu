// Varlen (packed) causal flash-attention forward on tcgen05 / TMEM / TMA for head_dim 128, GQA.
//
// One CTA = one (sequence, 128-query block, query head). Per 128-key block j:
//     S_j = Q K_j^T            tcgen05.mma M=128 (queries) N=128 (keys) K=128 (d), both operands K-major (TMA, SW128)
//     P_j = exp2(S_j*c - m)    softmax warps: one thread per query row (TMEM lane), no shuffles; P -> smem (bf16)
//     O  += P_j V_j            tcgen05.mma M=128 N=128 (d) K=128 (keys); V is the MN-major B operand, so the
//                              [token, d] layout of the packed activations is used as stored (no transpose)
// S is double-buffered in TMEM so the tensor core computes S_{j+1} while the softmax warps work on S_j; O stays
// in TMEM for the whole item and is rescaled lazily: the running maximum only moves when it grows by more than
// 2^8, so the TMEM read-modify-write of O is rare. Roles: warp 0 TMA producer, warp 1 MMA issuer, warps 2-9
// softmax + epilogue. K and V have separate 2-deep rings (a K tile is released right after its S MMA).
// Outputs O [T, hq, d] bf16 and LSE [hq, T] fp32 (natural log of the softmax denominator of the scaled scores).
// Queries are aligned to the END of the keys of their sequence (len_k >= len_q: prefill with a prefix cache,
// context-parallel chunks); with cu_q == cu_k this is ordinary causal self-attention.
// Replaces flash_attn_varlen_func (cosmos_rl/policy/kernel/modeling_utils.py:65-173). Every wait is bounded.
#include "sm100.cuh"
#include "gemm_core.cuh"
#include "api.h"

namespace b200 {

constexpr int FA_B = 128;                         // block of queries / keys
constexpr int FA_D = 128;
constexpr int FA_TILE = FA_B * FA_D * 2;          // 32 KiB
constexpr int FA_SMEM = 6 * FA_TILE + 256 + 3072 + 1024; // Q, K x2, V x2, P, barriers, row statistics, alignment
constexpr int FA_THREADS = 320;   // TMA warp, MMA warp, 8 softmax warps (two per TMEM lane quadrant)
constexpr float FA_LOG2E = 1.4426950408889634f;
constexpr float FA_LN2 = 0.6931471805599453f;
constexpr float FA_RESCALE_TAU = 8.0f;

struct FaParams {
  const int* cu_q;
  const int* cu_k;
  __nv_bfloat16* out;
  float* lse;
  long long ldo;      // elements between tokens of out
  int hq, hkv, Tq, causal;
  float scale_log2;
  uint32_t* status;
};

__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

#define FA_FAIL(code)                         \
  {                                           \
    atomicCAS(p.status, ST_OK, code);         \
    *abort_flag = 1;                          \
    break;                                    \
  }

__global__ void __launch_bounds__(FA_THREADS, 1)
flash_fwd_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                 const __grid_constant__ CUtensorMap tm_v, FaParams p) {
  const int b = blockIdx.z, h = blockIdx.y;
  const int q_beg = p.cu_q[b], len_q = p.cu_q[b + 1] - q_beg;
  const int k_beg = p.cu_k[b], len_k = p.cu_k[b + 1] - k_beg;
  const int qb = (len_q + FA_B - 1) / FA_B - 1 - (int)blockIdx.x;   // heavy (late) query blocks first
  if (qb < 0) return;
  const int q0 = qb * FA_B;
  const int shift = len_k - len_q;
  int kv_end = p.causal ? min(len_k, q0 + FA_B + shift) : len_k;
  if (kv_end < 0) kv_end = 0;
  const int n = (kv_end + FA_B - 1) / FA_B;
  const int hk = h / (p.hq / p.hkv);

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* q_sh = smem;
  uint8_t* k_sh = smem + FA_TILE;          // [2]
  uint8_t* v_sh = smem + 3 * FA_TILE;      // [2]
  uint8_t* p_sh = smem + 5 * FA_TILE;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + 6 * FA_TILE);
  uint64_t* qfull = bars;
  uint64_t* kfull = bars + 1;    // [2]
  uint64_t* kempty = bars + 3;   // [2]
  uint64_t* vfull = bars + 5;    // [2]
  uint64_t* vempty = bars + 7;   // [2]
  uint64_t* s_ready = bars + 9;  // [2]
  uint64_t* p_ready = bars + 11;
  uint64_t* o_done = bars + 12;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 13);
  volatile uint32_t* abort_flag = tmem_slot + 1;
  float* max_sh = reinterpret_cast<float*>(smem + 6 * FA_TILE + 256);   // [2 buffers][2 column halves][128 rows]
  float* l_sh = max_sh + 512;                                            // [2][128]

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    mbar_init(qfull, 1);
    for (int s = 0; s < 2; ++s) {
      mbar_init(&kfull[s], 1);
      mbar_init(&kempty[s], 1);
      mbar_init(&vfull[s], 1);
      mbar_init(&vempty[s], 1);
      mbar_init(&s_ready[s], 1);
    }
    mbar_init(p_ready, 8);
    mbar_init(o_done, 1);
    *abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tm_q);
    tma_prefetch_desc(&tm_k);
    tma_prefetch_desc(&tm_v);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tmem_o = tmem_base + 256;

  if (warp == 0) {
    // ------------------------------------------------ TMA producer
    if (lane == 0 && n > 0) {
      mbar_arrive_expect_tx(qfull, FA_TILE);
      tma_load_2d(q_sh, &tm_q, qfull, h * FA_D, q_beg + q0);
      tma_load_2d(q_sh + FA_TILE / 2, &tm_q, qfull, h * FA_D + 64, q_beg + q0);
      for (int j = 0; j < n && !*abort_flag; ++j) {
        const int s = j & 1;
        const uint32_t ph = (j >> 1) & 1;
        const int row = k_beg + j * FA_B;
        if (!mbar_wait(&kempty[s], ph ^ 1)) FA_FAIL(ST_TIMEOUT_EMPTY)
        mbar_arrive_expect_tx(&kfull[s], FA_TILE);
        tma_load_2d(k_sh + s * FA_TILE, &tm_k, &kfull[s], hk * FA_D, row);
        tma_load_2d(k_sh + s * FA_TILE + FA_TILE / 2, &tm_k, &kfull[s], hk * FA_D + 64, row);
        if (!mbar_wait(&vempty[s], ph ^ 1)) FA_FAIL(ST_TIMEOUT_EMPTY)
        mbar_arrive_expect_tx(&vfull[s], FA_TILE);
        // per 64-key block: two boxes of 64 keys x 64 head-dim elements
#pragma unroll
        for (int kb = 0; kb < 2; ++kb)
#pragma unroll
          for (int i = 0; i < 2; ++i)
            tma_load_2d(v_sh + s * FA_TILE + kb * 16384 + i * 8192, &tm_v, &vfull[s], hk * FA_D + i * 64, row + kb * 64);
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------ MMA issuer
    if (lane == 0 && n > 0) {
      constexpr uint32_t idesc_s = umma_idesc_bf16_f32(FA_B, FA_B);
      constexpr uint32_t idesc_o = umma_idesc_bf16_f32(FA_B, FA_D) | (1u << 16);   // B (= V) is MN-major
      const uint32_t q_addr = smem_u32(q_sh), p_addr = smem_u32(p_sh);
      auto mma_s = [&](int j) -> bool {
        const int s = j & 1;
        if (!mbar_wait(&kfull[s], (j >> 1) & 1)) return false;
        tc_fence_after_sync();
        const uint32_t ks = smem_u32(k_sh + s * FA_TILE);
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          const uint32_t off = (k >> 2) * (FA_TILE / 2) + (k & 3) * 32;
          umma_bf16_ss(tmem_base + s * FA_B, umma_desc_kmajor_sw128(q_addr + off), umma_desc_kmajor_sw128(ks + off),
                       idesc_s, k > 0 ? 1u : 0u);
        }
        tc_commit(&kempty[s]);
        tc_commit(&s_ready[s]);
        return true;
      };
      do {
        if (!mbar_wait(qfull, 0)) FA_FAIL(ST_TIMEOUT_FULL)
        tc_fence_after_sync();
        if (!mma_s(0)) FA_FAIL(ST_TIMEOUT_FULL)
        if (n > 1 && !mma_s(1)) FA_FAIL(ST_TIMEOUT_FULL)
        for (int j = 0; j < n; ++j) {
          const int s = j & 1;
          if (!mbar_wait(p_ready, j & 1)) FA_FAIL(ST_TIMEOUT_TMEM_EMPTY)
          if (!mbar_wait(&vfull[s], (j >> 1) & 1)) FA_FAIL(ST_TIMEOUT_FULL)
          tc_fence_after_sync();
          const uint32_t vs = smem_u32(v_sh + s * FA_TILE);
#pragma unroll
          for (int k = 0; k < 8; ++k) {
            const uint32_t a_off = (k >> 2) * (FA_TILE / 2) + (k & 3) * 32;
            const uint32_t b_off = (k >> 2) * 16384 + (k & 3) * 2048;
            umma_bf16_ss(tmem_o, umma_desc_kmajor_sw128(p_addr + a_off), umma_desc_mnmajor_sw128(vs + b_off, 8192),
                         idesc_o, (j > 0 || k > 0) ? 1u : 0u);
          }
          tc_commit(&vempty[s]);
          tc_commit(o_done);
          if (j + 2 < n && !mma_s(j + 2)) FA_FAIL(ST_TIMEOUT_FULL)
        }
      } while (false);
    }
  } else {
    // ------------------------------------------------ softmax + epilogue (warps 2..9)
    // Two warps share a TMEM lane quadrant and split the 128 columns of a row; they exchange their partial row
    // maxima through shared memory (one named barrier per key block) and keep partial row sums. A failed wait
    // never leaves the loop early: all eight warps meet at the barrier and leave together.
    const int quad = warp & 3;
    const int chalf = (warp - 2) >> 2;
    const int c_lo = chalf * 64;
    const int row = quad * 32 + lane;
    const uint32_t lane_addr = (uint32_t)(quad * 32) << 16;
    const int q_idx = q0 + row;                    // position inside the sequence's queries
    const int k_limit = p.causal ? min(len_k, q_idx + shift + 1) : len_k;   // keys [0, k_limit) are visible
    float m_run = -INFINITY, l_run = 0.f;
    bool ok = true;
    for (int j = 0; j < n; ++j) {
      const int s = j & 1;
      if (ok && !mbar_wait(&s_ready[s], (j >> 1) & 1)) { atomicCAS(p.status, ST_OK, ST_TIMEOUT_TMEM_FULL); *abort_flag = 1; ok = false; }
      ok = __all_sync(0xffffffffu, ok);
      tc_fence_after_sync();
      const uint32_t ts = tmem_base + s * FA_B + lane_addr;
      const int kbase = j * FA_B;
      const bool need_mask = kbase + FA_B > k_limit;
      // pass 1: maximum over this warp's half of the row
      float mx = -INFINITY;
      if (ok) {
#pragma unroll 1
        for (int c = c_lo; c < c_lo + 64; c += 32) {
          uint32_t r[32];
          tmem_ld_32x32b_x32(ts + c, r);
          tmem_ld_wait();
          if (!need_mask) {
#pragma unroll
            for (int i = 0; i < 32; ++i) mx = fmaxf(mx, __uint_as_float(r[i]));
          } else {
#pragma unroll
            for (int i = 0; i < 32; ++i)
              if (kbase + c + i < k_limit) mx = fmaxf(mx, __uint_as_float(r[i]));
          }
        }
      }
      max_sh[s * 256 + chalf * 128 + row] = mx;
      asm volatile("bar.sync 1, 256;" ::: "memory");
      // never leave the loop early (the barrier count must match in all eight warps): after a failure a warp
      // only skips its work, and every warp sits out at most one timed-out wait
      if (*abort_flag) ok = false;
      ok = __all_sync(0xffffffffu, ok);
      mx = fmaxf(mx, max_sh[s * 256 + (chalf ^ 1) * 128 + row]) * p.scale_log2;   // scale > 0
      // lazy rescale of the running state (identical decision in both warps of a row)
      float corr = 1.f;
      const bool grow = mx > m_run + FA_RESCALE_TAU || (m_run == -INFINITY && mx != -INFINITY);
      if (grow) {
        corr = (m_run == -INFINITY) ? 0.f : exp2f(m_run - mx);
        m_run = mx;
        l_run *= corr;
      }
      if (j > 0) {
        // PV_{j-1} must have finished reading P and updating O before either is touched
        if (!mbar_wait(o_done, (j - 1) & 1)) { atomicCAS(p.status, ST_OK, ST_TIMEOUT_TMEM_FULL); *abort_flag = 1; ok = false; }
        ok = __all_sync(0xffffffffu, ok);
        tc_fence_after_sync();
        if (ok && __any_sync(0xffffffffu, grow)) {
#pragma unroll 1
          for (int c = c_lo; c < c_lo + 64; c += 16) {
            uint32_t r[16];
            tmem_ld_32x32b_x16(tmem_o + lane_addr + c, r);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 16; ++i) r[i] = __float_as_uint(__uint_as_float(r[i]) * corr);
            tmem_st_32x32b_x16(tmem_o + lane_addr + c, r);
          }
          tmem_st_wait();
        }
      }
      if (!ok) continue;                            // meet the others at the next barrier
      // pass 2: probabilities of this warp's 64 keys -> shared memory (K-major, 128-byte swizzle)
      float sum = 0.f;
      const float mref = (m_run == -INFINITY) ? 0.f : m_run;
#pragma unroll 1
      for (int c = c_lo; c < c_lo + 64; c += 32) {
        uint32_t r[32];
        tmem_ld_32x32b_x32(ts + c, r);
        tmem_ld_wait();
        float e[32];
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          float v = fast_exp2(fmaf(__uint_as_float(r[i]), p.scale_log2, -mref));
          if (need_mask && kbase + c + i >= k_limit) v = 0.f;
          e[i] = v;
          sum += v;
        }
        uint8_t* dst = p_sh + (c >> 6) * (FA_TILE / 2) + row * 128;
        const int chunk0 = (c & 63) >> 3;
#pragma unroll
        for (int g = 0; g < 4; ++g) {
          uint4 o;
          o.x = pack_bf16x2(e[8 * g + 0], e[8 * g + 1]);
          o.y = pack_bf16x2(e[8 * g + 2], e[8 * g + 3]);
          o.z = pack_bf16x2(e[8 * g + 4], e[8 * g + 5]);
          o.w = pack_bf16x2(e[8 * g + 6], e[8 * g + 7]);
          *reinterpret_cast<uint4*>(dst + (((chunk0 + g) ^ (row & 7)) << 4)) = o;
        }
      }
      l_run += sum;
      fence_proxy_async_smem();
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(p_ready);
    }
    // ---- epilogue: combine the two partial row sums, O / l -> bf16, LSE
    l_sh[chalf * 128 + row] = l_run;
    asm volatile("bar.sync 1, 256;" ::: "memory");
    if (*abort_flag) ok = false;
    l_run += l_sh[(chalf ^ 1) * 128 + row];
    if (ok && n > 0) {
      if (!mbar_wait(o_done, (n - 1) & 1)) { atomicCAS(p.status, ST_OK, ST_TIMEOUT_TMEM_FULL); *abort_flag = 1; ok = false; }
    }
    ok = __all_sync(0xffffffffu, ok);               // tcgen05.ld below is warp-collective
    if (ok) {
      tc_fence_after_sync();
      const bool live = q_idx < len_q;
      const float inv = l_run > 0.f ? 1.f / l_run : 0.f;
      __nv_bfloat16* orow = p.out + (long long)(q_beg + q_idx) * p.ldo + h * FA_D;
#pragma unroll 1
      for (int c = c_lo; c < c_lo + 64; c += 32) {
        uint32_t r[32];
        if (n > 0) {
          tmem_ld_32x32b_x32(tmem_o + lane_addr + c, r);
          tmem_ld_wait();
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) r[i] = 0u;
        }
        if (live) {
#pragma unroll
          for (int g = 0; g < 4; ++g) {
            uint4 o;
            o.x = pack_bf16x2(__uint_as_float(r[8 * g + 0]) * inv, __uint_as_float(r[8 * g + 1]) * inv);
            o.y = pack_bf16x2(__uint_as_float(r[8 * g + 2]) * inv, __uint_as_float(r[8 * g + 3]) * inv);
            o.z = pack_bf16x2(__uint_as_float(r[8 * g + 4]) * inv, __uint_as_float(r[8 * g + 5]) * inv);
            o.w = pack_bf16x2(__uint_as_float(r[8 * g + 6]) * inv, __uint_as_float(r[8 * g + 7]) * inv);
            *reinterpret_cast<uint4*>(orow + c + 8 * g) = o;
          }
        }
      }
      if (live && chalf == 0)
        p.lse[(long long)h * p.Tq + q_beg + q_idx] = l_run > 0.f ? (m_run + log2f(l_run)) * FA_LN2 : INFINITY;
    }
    tc_fence_before_sync();
  }

  tc_fence_before_sync();
  __syncthreads();
  if (*abort_flag && threadIdx.x == 0) {
    for (int i = 0; i < 100; ++i) __nanosleep(1000);
  }
  __syncthreads();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, 512);
  }
}

}  // namespace b200

// q [Tq, hq, 128], k / v [Tk, hkv, 128] bf16 with token strides ldq / ldk / ldv (elements, multiples of 8);
// out [Tq, hq, 128] with token stride ldo; lse [hq, Tq] fp32. cu_q / cu_k: int32 [B + 1] on the device.
// max_q: longest query segment (bounds the grid). Sequences need len_k >= len_q when causal.
extern "C" int b200_flash_fwd(const void* q, const void* k, const void* v, void* out, float* lse, const int* cu_q,
                              const int* cu_k, int B, int Tq, int Tk, int hq, int hkv, int d, long long ldq,
                              long long ldk, long long ldv, long long ldo, int max_q, int causal, float scale,
                              uint32_t* status, cudaStream_t stream) {
  using namespace b200;
  if (B <= 0 || Tq <= 0) return 0;
  if (d != FA_D || hkv <= 0 || hq % hkv || (ldq & 7) || (ldk & 7) || (ldv & 7) || (ldo & 7) || max_q <= 0)
    return B200_ERR_ARG;
  CUtensorMap tm_q, tm_k, tm_v;
  if (make_tmap_2d(&tm_q, q, Tq, (uint64_t)hq * FA_D, ldq, FA_B, 64, 2)) return B200_ERR_TENSORMAP;
  if (make_tmap_2d(&tm_k, k, Tk, (uint64_t)hkv * FA_D, ldk, FA_B, 64, 2)) return B200_ERR_TENSORMAP;
  if (make_tmap_2d(&tm_v, v, Tk, (uint64_t)hkv * FA_D, ldv, 64, 64, 2)) return B200_ERR_TENSORMAP;
  static bool attr_set = false;
  if (!attr_set) {
    if (cudaFuncSetAttribute(flash_fwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, FA_SMEM) != cudaSuccess)
      return B200_ERR_LAUNCH;
    attr_set = true;
  }
  FaParams p{cu_q, cu_k, (__nv_bfloat16*)out, lse, ldo, hq, hkv, Tq, causal, scale * FA_LOG2E, status};
  dim3 grid((max_q + FA_B - 1) / FA_B, hq, B);
  flash_fwd_kernel<<<grid, FA_THREADS, FA_SMEM, stream>>>(tm_q, tm_k, tm_v, p);
  return cudaGetLastError() == cudaSuccess ? 0 : B200_ERR_LAUNCH;
}
