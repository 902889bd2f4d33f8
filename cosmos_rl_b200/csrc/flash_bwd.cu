// Varlen causal flash-attention backward on tcgen05 / TMEM / TMA (head_dim 128, GQA, packed sequences).
//
// One CTA owns one (sequence, 128-key block, kv head): K and V tiles stay in shared memory, dK and dV accumulate
// in TMEM over every query head of the GQA group and every 64-query block that can see the key block, and are
// written once as bf16 (no atomics, no per-head partial sums). Per (query head, 64-query block) iteration i:
//     S^T  = K Q^T                 M=keys(128) N=queries(64) K=d     TMEM S[i&1]   (64 columns)
//     dP^T = V dO^T                M=keys      N=queries     K=d     TMEM dP[i&1]  (64 columns)
//     P^T  = exp2(S^T c - lse),  dS^T = P^T o (dP^T - delta) * scale   8 softmax warps, thread = key row x 32 queries;
//                                                                      both written to smem as bf16 [keys x queries]
//     dV  += P^T dO                M=keys N=d K=queries(64)          dO tile re-read as MN-major B
//     dK  += dS^T Q                M=keys N=d K=queries              Q  tile re-read as MN-major B
//     dQ^T = K^T dS^T              M=d N=queries K=keys              K tile as MN-major A, dS^T smem as MN-major B;
//                                                                    written over dP[i&1], which is dead by then
// Q/dO tiles and the S/dP accumulators are double-buffered: the TMA loads and the first two MMAs of iteration i+1
// run while the softmax warps work on iteration i, and the dQ^T drain of iteration i-1 (coalesced fp32 atomics:
// a warp adds 32 consecutive head-dim elements of one query) runs while the tensor core does the three MMAs of
// iteration i. A tile loaded by TMA as rows of 128 bytes (SW128) serves both as a K-major operand (rows = M/N) and
// as an MN-major operand (rows = contraction), so nothing is transposed or loaded twice.
// delta = rowsum(O o dO) comes from a small pre-pass. All waits are bounded; a failed wait never leaves a loop that
// contains a named barrier early.
// Replaces flash_attn's varlen backward (cosmos_rl/policy/kernel/modeling_utils.py:65-173).
#include "sm100.cuh"
#include "gemm_core.cuh"
#include "api.h"

namespace b200 {

constexpr int FB_BK = 128;                           // keys per CTA
constexpr int FB_BQ = 64;                            // queries per iteration
constexpr int FB_D = 128;
constexpr int FB_KV_TILE = FB_BK * FB_D * 2;         // 32 KiB
constexpr int FB_Q_TILE = FB_BQ * FB_D * 2;          // 16 KiB
constexpr int FB_P_TILE = FB_BK * FB_BQ * 2;         // 16 KiB
constexpr int FB_SMEM = 2 * FB_KV_TILE + 4 * FB_Q_TILE + 2 * FB_P_TILE + 1024 /*lse, delta x2*/ + 256 + 1024;
constexpr int FB_THREADS = 320;                      // TMA warp, MMA warp, 8 softmax warps (two per TMEM lane quadrant)
constexpr float FB_LOG2E = 1.4426950408889634f;

struct FbParams {
  const int* cu_q;
  const int* cu_k;
  const float* lse;      // [hq, Tq]
  const float* delta;    // [hq, Tq]
  float* dq_accum;       // [Tq, hq, d] fp32, zero-initialised
  __nv_bfloat16* dk;     // [Tk, hkv, d]
  __nv_bfloat16* dv;
  long long lddk, lddv;  // token strides (elements)
  int hq, hkv, Tq, causal;
  float scale, scale_log2;
  uint32_t* status;
};

__device__ __forceinline__ float fb_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

#define FB_FAIL(code)                         \
  {                                           \
    atomicCAS(p.status, ST_OK, code);         \
    *abort_flag = 1;                          \
    break;                                    \
  }

__global__ void __launch_bounds__(FB_THREADS, 1)
flash_bwd_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                 const __grid_constant__ CUtensorMap tm_v, const __grid_constant__ CUtensorMap tm_do, FbParams p) {
  const int b = blockIdx.z, hk = blockIdx.y, kb = blockIdx.x;
  const int q_beg = p.cu_q[b], len_q = p.cu_q[b + 1] - q_beg;
  const int k_beg = p.cu_k[b], len_k = p.cu_k[b + 1] - k_beg;
  const int kv0 = kb * FB_BK;
  if (kv0 >= len_k) return;
  const int shift = len_k - len_q;
  const int G = p.hq / p.hkv;
  const int nqb = (len_q + FB_BQ - 1) / FB_BQ;
  int qb_first = 0;
  if (p.causal && kv0 - shift > 0) qb_first = (kv0 - shift) / FB_BQ;
  const int per_head = nqb > qb_first ? nqb - qb_first : 0;
  const int n_iter = per_head * G;

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* k_sh = smem;
  uint8_t* v_sh = smem + FB_KV_TILE;
  uint8_t* q_sh = smem + 2 * FB_KV_TILE;                    // [2]
  uint8_t* do_sh = q_sh + 2 * FB_Q_TILE;                    // [2]
  uint8_t* pt_sh = do_sh + 2 * FB_Q_TILE;
  uint8_t* ds_sh = pt_sh + FB_P_TILE;
  float* lse_sh = reinterpret_cast<float*>(ds_sh + FB_P_TILE);   // [2][64] lse * log2(e)
  float* dlt_sh = lse_sh + 2 * FB_BQ;                             // [2][64]
  uint64_t* bars = reinterpret_cast<uint64_t*>(reinterpret_cast<uint8_t*>(lse_sh) + 1024);
  uint64_t* kv_full = bars;
  uint64_t* qdo_full = bars + 1;     // [2]
  uint64_t* qdo_empty = bars + 3;    // [2]
  uint64_t* sdp_ready = bars + 5;    // [2]
  uint64_t* pds_ready = bars + 7;
  uint64_t* mma3_done = bars + 8;
  uint64_t* dq_drained = bars + 9;   // [2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 11);
  volatile uint32_t* abort_flag = tmem_slot + 1;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    mbar_init(kv_full, 1);
    for (int s = 0; s < 2; ++s) {
      mbar_init(&qdo_full[s], 1);
      mbar_init(&qdo_empty[s], 1);
      mbar_init(&sdp_ready[s], 1);
      mbar_init(&dq_drained[s], 8);
    }
    mbar_init(pds_ready, 8);
    mbar_init(mma3_done, 1);
    *abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tm_q);
    tma_prefetch_desc(&tm_k);
    tma_prefetch_desc(&tm_v);
    tma_prefetch_desc(&tm_do);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  // columns: S[2] 0..127, dP[2] (later dQ^T) 128..255, dV 256..383, dK 384..511
  const uint32_t tm_dv = tmem_base + 256, tm_dk = tmem_base + 384;

  if (warp == 0) {
    // ------------------------------------------------ TMA producer
    if (lane == 0 && n_iter > 0) {
      mbar_arrive_expect_tx(kv_full, 2 * FB_KV_TILE);
      tma_load_2d(k_sh, &tm_k, kv_full, hk * FB_D, k_beg + kv0);
      tma_load_2d(k_sh + FB_KV_TILE / 2, &tm_k, kv_full, hk * FB_D + 64, k_beg + kv0);
      tma_load_2d(v_sh, &tm_v, kv_full, hk * FB_D, k_beg + kv0);
      tma_load_2d(v_sh + FB_KV_TILE / 2, &tm_v, kv_full, hk * FB_D + 64, k_beg + kv0);
      for (int i = 0; i < n_iter && !*abort_flag; ++i) {
        const int s = i & 1;
        const int h = hk * G + i / per_head, qb = qb_first + i % per_head;
        if (!mbar_wait(&qdo_empty[s], ((i >> 1) & 1) ^ 1)) FB_FAIL(ST_TIMEOUT_EMPTY)
        const int row = q_beg + qb * FB_BQ;
        mbar_arrive_expect_tx(&qdo_full[s], 2 * FB_Q_TILE);
        tma_load_2d(q_sh + s * FB_Q_TILE, &tm_q, &qdo_full[s], h * FB_D, row);
        tma_load_2d(q_sh + s * FB_Q_TILE + FB_Q_TILE / 2, &tm_q, &qdo_full[s], h * FB_D + 64, row);
        tma_load_2d(do_sh + s * FB_Q_TILE, &tm_do, &qdo_full[s], h * FB_D, row);
        tma_load_2d(do_sh + s * FB_Q_TILE + FB_Q_TILE / 2, &tm_do, &qdo_full[s], h * FB_D + 64, row);
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------ MMA issuer
    if (lane == 0 && n_iter > 0) {
      constexpr uint32_t id_s = umma_idesc_bf16_f32(128, FB_BQ);                                 // both K-major
      constexpr uint32_t id_dkv = umma_idesc_bf16_f32(128, FB_D) | (1u << 16);                   // B MN-major
      constexpr uint32_t id_dq = umma_idesc_bf16_f32(128, FB_BQ) | (1u << 15) | (1u << 16);      // A, B MN-major
      const uint32_t k_a = smem_u32(k_sh), v_a = smem_u32(v_sh), pt_a = smem_u32(pt_sh), ds_a = smem_u32(ds_sh);
      auto issue_sdp = [&](int i) -> bool {   // S^T(i), dP^T(i)
        const int s = i & 1;
        if (!mbar_wait(&qdo_full[s], (i >> 1) & 1)) return false;
        // dP[s] still holds dQ^T of iteration i-2 until the softmax warps have drained it
        if (i >= 2 && !mbar_wait(&dq_drained[s], ((i - 2) >> 1) & 1)) return false;
        tc_fence_after_sync();
        const uint32_t q_a = smem_u32(q_sh + s * FB_Q_TILE), do_a = smem_u32(do_sh + s * FB_Q_TILE);
#pragma unroll
        for (int k = 0; k < 8; ++k)
          umma_bf16_ss(tmem_base + s * FB_BQ, umma_desc_kmajor_sw128(k_a + (k >> 2) * (FB_KV_TILE / 2) + (k & 3) * 32),
                       umma_desc_kmajor_sw128(q_a + (k >> 2) * (FB_Q_TILE / 2) + (k & 3) * 32), id_s, k > 0 ? 1u : 0u);
#pragma unroll
        for (int k = 0; k < 8; ++k)
          umma_bf16_ss(tmem_base + 128 + s * FB_BQ,
                       umma_desc_kmajor_sw128(v_a + (k >> 2) * (FB_KV_TILE / 2) + (k & 3) * 32),
                       umma_desc_kmajor_sw128(do_a + (k >> 2) * (FB_Q_TILE / 2) + (k & 3) * 32), id_s, k > 0 ? 1u : 0u);
        tc_commit(&sdp_ready[s]);
        return true;
      };
      do {
        if (!mbar_wait(kv_full, 0)) FB_FAIL(ST_TIMEOUT_FULL)
        if (!issue_sdp(0)) FB_FAIL(ST_TIMEOUT_FULL)
        for (int i = 0; i < n_iter; ++i) {
          const int s = i & 1;
          if (i + 1 < n_iter && !issue_sdp(i + 1)) FB_FAIL(ST_TIMEOUT_FULL)
          if (!mbar_wait(pds_ready, i & 1)) FB_FAIL(ST_TIMEOUT_TMEM_EMPTY)
          tc_fence_after_sync();
          const uint32_t q_a = smem_u32(q_sh + s * FB_Q_TILE), do_a = smem_u32(do_sh + s * FB_Q_TILE);
#pragma unroll
          for (int k = 0; k < 4; ++k)   // dV += P^T dO      (K = 64 queries)
            umma_bf16_ss(tm_dv, umma_desc_kmajor_sw128(pt_a + k * 32), umma_desc_mnmajor_sw128(do_a + k * 2048, FB_Q_TILE / 2),
                         id_dkv, (i > 0 || k > 0) ? 1u : 0u);
#pragma unroll
          for (int k = 0; k < 4; ++k)   // dK += dS^T Q
            umma_bf16_ss(tm_dk, umma_desc_kmajor_sw128(ds_a + k * 32), umma_desc_mnmajor_sw128(q_a + k * 2048, FB_Q_TILE / 2),
                         id_dkv, (i > 0 || k > 0) ? 1u : 0u);
#pragma unroll
          for (int k = 0; k < 8; ++k)   // dQ^T = K^T dS^T   (K = 128 keys), over dP[s]
            umma_bf16_ss(tmem_base + 128 + s * FB_BQ, umma_desc_mnmajor_sw128(k_a + k * 2048, FB_KV_TILE / 2),
                         umma_desc_mnmajor_sw128(ds_a + k * 2048, FB_P_TILE), id_dq, k > 0 ? 1u : 0u);
          tc_commit(&qdo_empty[s]);
          tc_commit(mma3_done);
        }
      } while (false);
    }
  } else {
    // ------------------------------------------------ softmax / dS / drains (warps 2..9)
    // warp -> (TMEM lane quadrant, half of the 64 query columns). S^T / dP^T rows are keys, dQ^T rows are head-dim.
    const int quad = warp & 3;
    const int chalf = (warp - 2) >> 2;
    const int row = quad * 32 + lane;
    const uint32_t lane_addr = (uint32_t)(quad * 32) << 16;
    const int c0 = chalf * 32;                           // first query column of this warp
    const int key = kv0 + row;
    const bool key_ok = key < len_k;
    const int q_min = p.causal ? key - shift : -(1 << 30);   // visible iff q >= key - shift
    const int tid = threadIdx.x - 64;                    // 0..255
    bool ok = true;
    auto load_stats = [&](int i, float& l, float& dl) {  // threads 0..63: statistics of query (i, tid)
      const int ph = per_head > 0 ? per_head : 1;
      const int h = hk * G + i / ph, qi = (qb_first + i % ph) * FB_BQ + tid;
      const long long o = (long long)h * p.Tq + q_beg + qi;
      const bool live = tid < FB_BQ && i < n_iter && qi < len_q;
      l = live ? p.lse[o] * FB_LOG2E : INFINITY;
      dl = live ? p.delta[o] : 0.f;
    };
    auto drain_dq = [&](int j) {                         // dQ^T of iteration j: lanes = head-dim, columns = queries
      const int s = j & 1;
      const int h = hk * G + j / per_head, q0 = (qb_first + j % per_head) * FB_BQ;
      uint32_t r[32];
      tmem_ld_32x32b_x32(tmem_base + 128 + s * FB_BQ + lane_addr + c0, r);
      tmem_ld_wait();
      float* dst = p.dq_accum + ((long long)(q_beg + q0 + c0) * p.hq + h) * FB_D + row;
#pragma unroll
      for (int c = 0; c < 32; ++c)
        if (q0 + c0 + c < len_q) atomicAdd(dst + (long long)c * p.hq * FB_D, __uint_as_float(r[c]));
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&dq_drained[s]);
    };
    float l_next, d_next;
    load_stats(0, l_next, d_next);
    for (int i = 0; i < n_iter; ++i) {                   // never left early (named barrier inside)
      const int s = i & 1;
      const int q0 = (qb_first + i % per_head) * FB_BQ;
      if (tid < FB_BQ) { lse_sh[s * FB_BQ + tid] = l_next; dlt_sh[s * FB_BQ + tid] = d_next; }
      asm volatile("bar.sync 1, 256;" ::: "memory");
      if (*abort_flag) ok = false;
      load_stats(i + 1, l_next, d_next);                 // prefetch for the next iteration
      if (ok && !mbar_wait(&sdp_ready[s], (i >> 1) & 1)) { atomicCAS(p.status, ST_OK, ST_TIMEOUT_TMEM_FULL); *abort_flag = 1; ok = false; }
      ok = __all_sync(0xffffffffu, ok);                  // tcgen05.ld below is warp-collective
      uint32_t pp[16], dd[16];
      if (ok) {
        tc_fence_after_sync();
        uint32_t rs[32], rd[32];
        tmem_ld_32x32b_x32(tmem_base + s * FB_BQ + lane_addr + c0, rs);
        tmem_ld_32x32b_x32(tmem_base + 128 + s * FB_BQ + lane_addr + c0, rd);
        tmem_ld_wait();
        const bool need_mask = !key_ok || (q0 < q_min) || (q0 + FB_BQ > len_q);
#pragma unroll
        for (int c = 0; c < 32; c += 2) {
          float pv[2], dv2[2];
#pragma unroll
          for (int u = 0; u < 2; ++u) {
            const int qc = c0 + c + u;
            float pe = fb_exp2(fmaf(__uint_as_float(rs[c + u]), p.scale_log2, -lse_sh[s * FB_BQ + qc]));
            if (need_mask && (!key_ok || q0 + qc < q_min || q0 + qc >= len_q)) pe = 0.f;
            pv[u] = pe;
            dv2[u] = pe * (__uint_as_float(rd[c + u]) - dlt_sh[s * FB_BQ + qc]) * p.scale;
          }
          pp[c >> 1] = pack_bf16x2(pv[0], pv[1]);
          dd[c >> 1] = pack_bf16x2(dv2[0], dv2[1]);
        }
        tc_fence_before_sync();
      }
      // P^T / dS^T of the previous iteration are still being read by its three MMAs until mma3_done(i-1)
      if (ok && i > 0 && !mbar_wait(mma3_done, (i - 1) & 1)) { atomicCAS(p.status, ST_OK, ST_TIMEOUT_TMEM_FULL); *abort_flag = 1; ok = false; }
      ok = __all_sync(0xffffffffu, ok);
      if (ok) {
        const int off = row * 128;
        const int chunk0 = c0 >> 3;
#pragma unroll
        for (int g = 0; g < 4; ++g) {
          const int sw = ((chunk0 + g) ^ (row & 7)) << 4;
          *reinterpret_cast<uint4*>(pt_sh + off + sw) = make_uint4(pp[4 * g], pp[4 * g + 1], pp[4 * g + 2], pp[4 * g + 3]);
          *reinterpret_cast<uint4*>(ds_sh + off + sw) = make_uint4(dd[4 * g], dd[4 * g + 1], dd[4 * g + 2], dd[4 * g + 3]);
        }
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) mbar_arrive(pds_ready);
        // while the tensor core runs the three MMAs of iteration i: drain dQ^T of iteration i-1
        if (i > 0) {
          tc_fence_after_sync();
          drain_dq(i - 1);
        }
      }
    }
    // ---- last dQ^T, then dK, dV of the key block
    if (n_iter > 0) {
      if (ok && !mbar_wait(mma3_done, (n_iter - 1) & 1)) { atomicCAS(p.status, ST_OK, ST_TIMEOUT_TMEM_FULL); *abort_flag = 1; ok = false; }
      ok = __all_sync(0xffffffffu, ok);
      if (ok) {
        tc_fence_after_sync();
        drain_dq(n_iter - 1);
      }
    }
    if (ok) {                                            // loads by every lane, stores by rows inside the sequence
      __nv_bfloat16* dkr = p.dk + (long long)(k_beg + key) * p.lddk + hk * FB_D;
      __nv_bfloat16* dvr = p.dv + (long long)(k_beg + key) * p.lddv + hk * FB_D;
#pragma unroll 1
      for (int c = chalf * 64; c < chalf * 64 + 64; c += 32) {
        uint32_t a[32], bb[32];
        if (n_iter > 0) {
          tmem_ld_32x32b_x32(tm_dk + lane_addr + c, a);
          tmem_ld_32x32b_x32(tm_dv + lane_addr + c, bb);
          tmem_ld_wait();
        } else {
#pragma unroll
          for (int j = 0; j < 32; ++j) { a[j] = 0u; bb[j] = 0u; }
        }
#pragma unroll
        for (int g = 0; g < 4; ++g) {
          uint4 o;
          o.x = pack_bf16x2(__uint_as_float(a[8 * g + 0]), __uint_as_float(a[8 * g + 1]));
          o.y = pack_bf16x2(__uint_as_float(a[8 * g + 2]), __uint_as_float(a[8 * g + 3]));
          o.z = pack_bf16x2(__uint_as_float(a[8 * g + 4]), __uint_as_float(a[8 * g + 5]));
          o.w = pack_bf16x2(__uint_as_float(a[8 * g + 6]), __uint_as_float(a[8 * g + 7]));
          if (key_ok) *reinterpret_cast<uint4*>(dkr + c + 8 * g) = o;
          o.x = pack_bf16x2(__uint_as_float(bb[8 * g + 0]), __uint_as_float(bb[8 * g + 1]));
          o.y = pack_bf16x2(__uint_as_float(bb[8 * g + 2]), __uint_as_float(bb[8 * g + 3]));
          o.z = pack_bf16x2(__uint_as_float(bb[8 * g + 4]), __uint_as_float(bb[8 * g + 5]));
          o.w = pack_bf16x2(__uint_as_float(bb[8 * g + 6]), __uint_as_float(bb[8 * g + 7]));
          if (key_ok) *reinterpret_cast<uint4*>(dvr + c + 8 * g) = o;
        }
      }
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

// delta[h, t] = sum_d O[t, h, d] * dO[t, h, d]; one warp per (t, h)
__global__ void flash_delta_kernel(const __nv_bfloat16* __restrict__ o, const __nv_bfloat16* __restrict__ dout,
                                   float* __restrict__ delta, int T, int hq, long long ldo, long long lddo) {
  const long long w = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (w >= (long long)T * hq) return;
  const int t = (int)(w / hq), h = (int)(w % hq);
  const uint2 a = *reinterpret_cast<const uint2*>(o + t * ldo + h * FB_D + lane * 4);
  const uint2 b = *reinterpret_cast<const uint2*>(dout + t * lddo + h * FB_D + lane * 4);
  const __nv_bfloat162* ah = reinterpret_cast<const __nv_bfloat162*>(&a);
  const __nv_bfloat162* bh = reinterpret_cast<const __nv_bfloat162*>(&b);
  float s = 0.f;
#pragma unroll
  for (int j = 0; j < 2; ++j) {
    const float2 x = __bfloat1622float2(ah[j]), y = __bfloat1622float2(bh[j]);
    s += x.x * y.x + x.y * y.y;
  }
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) s += __shfl_xor_sync(0xffffffffu, s, off);
  if (lane == 0) delta[(long long)h * T + t] = s;
}

}  // namespace b200

// Gradients of b200_flash_fwd. dq_accum [Tq, hq, 128] fp32 must be zero on entry and holds dQ on return;
// dk / dv [Tk, hkv, 128] bf16 are overwritten; delta [hq, Tq] fp32 is scratch. max_k bounds the grid.
extern "C" int b200_flash_bwd(const void* q, const void* k, const void* v, const void* out, const void* dout,
                              const float* lse, float* dq_accum, void* dk, void* dv, float* delta, const int* cu_q,
                              const int* cu_k, int B, int Tq, int Tk, int hq, int hkv, int d, long long ldq,
                              long long ldk, long long ldv, long long ldo, long long lddo, long long lddk,
                              long long lddv, int max_k, int causal, float scale, uint32_t* status,
                              cudaStream_t stream) {
  using namespace b200;
  if (B <= 0 || Tq <= 0 || Tk <= 0) return 0;
  if (d != FB_D || hkv <= 0 || hq % hkv || (ldq & 7) || (ldk & 7) || (ldv & 7) || (ldo & 3) || (lddo & 7) ||
      (lddk & 7) || (lddv & 7) || max_k <= 0)
    return B200_ERR_ARG;
  CUtensorMap tm_q, tm_k, tm_v, tm_do;
  if (make_tmap_2d(&tm_q, q, Tq, (uint64_t)hq * FB_D, ldq, FB_BQ, 64, 2)) return B200_ERR_TENSORMAP;
  if (make_tmap_2d(&tm_k, k, Tk, (uint64_t)hkv * FB_D, ldk, FB_BK, 64, 2)) return B200_ERR_TENSORMAP;
  if (make_tmap_2d(&tm_v, v, Tk, (uint64_t)hkv * FB_D, ldv, FB_BK, 64, 2)) return B200_ERR_TENSORMAP;
  if (make_tmap_2d(&tm_do, dout, Tq, (uint64_t)hq * FB_D, lddo, FB_BQ, 64, 2)) return B200_ERR_TENSORMAP;
  static bool attr_set = false;
  if (!attr_set) {
    if (cudaFuncSetAttribute(flash_bwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, FB_SMEM) != cudaSuccess)
      return B200_ERR_LAUNCH;
    attr_set = true;
  }
  const long long warps = (long long)Tq * hq;
  flash_delta_kernel<<<(unsigned)((warps * 32 + 255) / 256), 256, 0, stream>>>(
      (const __nv_bfloat16*)out, (const __nv_bfloat16*)dout, delta, Tq, hq, ldo, lddo);
  FbParams p{cu_q, cu_k, lse, delta, dq_accum, (__nv_bfloat16*)dk, (__nv_bfloat16*)dv, lddk, lddv, hq, hkv, Tq, causal,
             scale, scale * FB_LOG2E, status};
  dim3 grid((max_k + FB_BK - 1) / FB_BK, hkv, B);
  flash_bwd_kernel<<<grid, FB_THREADS, FB_SMEM, stream>>>(tm_q, tm_k, tm_v, tm_do, p);
  return cudaGetLastError() == cudaSuccess ? 0 : B200_ERR_LAUNCH;
}
