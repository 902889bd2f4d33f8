// Paged decode attention on the 5th-generation tensor cores (tcgen05 + TMEM), fed by TMA.
//
// Decode attention is bound by reading the KV cache once; the job of the kernel is to keep HBM busy while
// spending almost no issue slots on arithmetic. A CUDA-core kernel needs ~2300 instructions per 32 cached
// tokens for a GQA group of 7 heads; here the two contractions are eight `tcgen05.mma` each per 128 tokens.
//
// Cache layout (per layer): [pages, 2, hkv, 128 x 128] bf16 with page_size = 128 tokens and d = 128:
//   slab (page, 0, h) = K   as [token, d]      (row = token, d contiguous)
//   slab (page, 1, h) = V^T as [d, token]      (row = d, tokens contiguous)
// so both contractions take K-major operands straight from TMA (128-byte swizzle):
//   S^T[token, head] = K[token, :] . Q[head, :]        M = 128 tokens, N = 16 (G <= 8 heads, padded), K = d
//   O^T[d, head]    += V^T[d, token] . P[head, token]   M = 128 (d),    N = 16,                        K = tokens
// One work item = (sequence, kv head, split). Persistent CTAs (one per SM) walk the items.
//   warp 0   : TMA producer (Q tile per item, K / V^T slabs per page through a 3-stage ring)
//   warp 1   : MMA issuer (one thread), owns the TMEM allocation (S^T: 16 columns, O^T: 16 columns)
//   warps 2-5: softmax. Thread <-> TMEM lane: a token row of S^T, a head-dim row of O^T. Column (head)
//              maxima / sums over the 128 tokens go through warp shuffles and a small shared array; P is
//              written to shared memory in the swizzled K-major layout the second MMA reads; O^T is
//              rescaled in TMEM (tcgen05.ld / st) when the running maximum moves.
// Every mbarrier wait is bounded; on a timeout the kernel records a status code, frees TMEM and returns.
#include "sm100.cuh"
#include "gemm_core.cuh"
#include "api.h"

namespace b200 {

constexpr int PDT_PAGE = 128;
constexpr int PDT_D = 128;
constexpr int PDT_N = 16;       // padded head count (MMA N)
constexpr int PDT_STAGES = 3;
constexpr int PDT_SLAB_BYTES = PDT_PAGE * PDT_D * 2;        // 32 KiB
constexpr int PDT_STAGE_BYTES = 2 * PDT_SLAB_BYTES;         // K + V^T
constexpr int PDT_Q_BYTES = 2 * PDT_N * 64 * 2;             // two 16 x 64 boxes
constexpr int PDT_P_BYTES = 2 * PDT_N * 64 * 2;             // two 16 x 64-token halves
constexpr int PDT_SMEM = PDT_STAGES * PDT_STAGE_BYTES + 2 * PDT_Q_BYTES + 2 * PDT_P_BYTES + 1024 /*barriers, reductions*/ + 1024;
constexpr int PDT_THREADS = 192;
constexpr float PDT_LOG2E = 1.4426950408889634f;

struct PdtParams {
  const int* block_table;
  const int* seq_lens;
  __nv_bfloat16* out;      // [B, hq, d]
  float* scratch;          // [B*hq, nsplit, d + 2] when nsplit > 1
  int B, hq, hkv, max_pages, nsplit;
  float scale_log2;
  uint32_t* status;
  // shared-prefix mode (prefix_pages != nullptr): the first prefix_pages[b] pages of sequence b are handled by
  // paged_prefix_tc_kernel; this kernel covers the remaining tokens and writes split (max_shared + split) of ns_total
  const int* prefix_pages;
  int max_shared, ns_total;
};

__device__ __forceinline__ void softmax_bar() { asm volatile("bar.sync 1, 128;" ::: "memory"); }

__global__ void __launch_bounds__(PDT_THREADS, 1)
paged_decode_tc_kernel(const __grid_constant__ CUtensorMap tm_cache, const __grid_constant__ CUtensorMap tm_q,
                       PdtParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* q_sh = smem + PDT_STAGES * PDT_STAGE_BYTES;     // [2] query tiles (current / next work item)
  uint8_t* p_sh = q_sh + 2 * PDT_Q_BYTES;                  // [2] probability tiles (even / odd key tile)
  uint64_t* bars = reinterpret_cast<uint64_t*>(p_sh + 2 * PDT_P_BYTES);
  uint64_t* kfull = bars;                    // [STAGES]
  uint64_t* vfull = kfull + PDT_STAGES;      // [STAGES]
  uint64_t* kvempty = vfull + PDT_STAGES;    // [STAGES]  also "PV of this tile is done" for the softmax warps
  uint64_t* qfull = kvempty + PDT_STAGES;    // [2]
  uint64_t* qempty = qfull + 2;              // [2]
  uint64_t* s_ready = qempty + 2;            // [2]
  uint64_t* p_ready = s_ready + 2;           // [2]
  uint64_t* o_ready = p_ready + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(o_ready + 1);
  volatile uint32_t* abort_flag = tmem_slot + 1;
  float* red = reinterpret_cast<float*>(tmem_slot + 2);  // [2][4 warps][8 heads]

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int G = p.hq / p.hkv;
  const int n_items = p.B * p.hkv * p.nsplit;

  pdl_launch_dependents();
  if (threadIdx.x == 0) {
    for (int s = 0; s < PDT_STAGES; ++s) {
      mbar_init(&kfull[s], 1);
      mbar_init(&vfull[s], 1);
      mbar_init(&kvempty[s], 1);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(&qfull[s], 1);
      mbar_init(&qempty[s], 1);
      mbar_init(&s_ready[s], 1);
      mbar_init(&p_ready[s], 4);
    }
    mbar_init(o_ready, 1);
    *abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tm_cache);
    tma_prefetch_desc(&tm_q);
  }
  // rows G..15 of both P tiles stay zero for the whole kernel
  for (int i = threadIdx.x; i < 2 * PDT_P_BYTES / 4; i += blockDim.x) reinterpret_cast<uint32_t*>(p_sh)[i] = 0;
  if (warp == 1) {
    tmem_alloc(tmem_slot, 64);
    tmem_relinquish();
  }
  fence_proxy_async_smem();
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tmem_o = tmem_base + 32;   // S^T: columns [0,16) and [16,32) (even / odd tile); O^T: [32,48)
  pdl_wait();  // the set-up above is CTA-local; queries, cache pages and lengths are global memory

  // item -> (b, h, split) and its token range, identical in every role
  auto item_range = [&](int item, int& b, int& h, int& split, int& t0, int& t1) {
    split = item % p.nsplit;
    int bh = item / p.nsplit;
    h = bh % p.hkv;
    b = bh / p.hkv;
    const int len = p.seq_lens[b];
    const int tb = p.prefix_pages ? min(p.prefix_pages[b] * PDT_PAGE, len) : 0;
    int chunk = (len - tb + p.nsplit - 1) / p.nsplit;
    chunk = (chunk + PDT_PAGE - 1) / PDT_PAGE * PDT_PAGE;
    t0 = tb + split * chunk;
    t1 = min(len, t0 + chunk);
    if (t1 < t0) t1 = t0;
  };
  auto item_tiles = [&](int item) -> int {
    int b, h, split, t0, t1;
    item_range(item, b, h, split, t0, t1);
    return (t1 - t0 + PDT_PAGE - 1) / PDT_PAGE;
  };

  if (warp == 0) {
    // ------------------------------------------------ TMA producer
    if (lane == 0) {
      uint32_t kv_it = 0, item_it = 0;
      // work items with an empty token range are skipped by every role (item_it counts the others)
      for (int item = blockIdx.x; item < n_items && !*abort_flag; item += gridDim.x) {
        int b, h, split, t0, t1;
        item_range(item, b, h, split, t0, t1);
        const int ntiles = (t1 - t0 + PDT_PAGE - 1) / PDT_PAGE;
        if (ntiles == 0) continue;
        const uint32_t qs = item_it & 1;
        if (!mbar_wait(&qempty[qs], ((item_it >> 1) & 1) ^ 1)) { atomicCAS(p.status, ST_OK, ST_TIMEOUT_EMPTY); *abort_flag = 1; break; }
        mbar_arrive_expect_tx(&qfull[qs], PDT_Q_BYTES);
        const int qrow = b * p.hq + h * G;
        tma_load_2d(q_sh + qs * PDT_Q_BYTES, &tm_q, &qfull[qs], 0, qrow);
        tma_load_2d(q_sh + qs * PDT_Q_BYTES + PDT_N * 128, &tm_q, &qfull[qs], 64, qrow);
        const int* bt = p.block_table + (long long)b * p.max_pages + t0 / PDT_PAGE;
        for (int j = 0; j < ntiles; ++j, ++kv_it) {
          const uint32_t st = kv_it % PDT_STAGES, ph = (kv_it / PDT_STAGES) & 1;
          if (!mbar_wait(&kvempty[st], ph ^ 1)) { atomicCAS(p.status, ST_OK, ST_TIMEOUT_EMPTY); *abort_flag = 1; break; }
          const int page = bt[j];
          const int krow = ((page * 2 + 0) * p.hkv + h) * PDT_PAGE;
          const int vrow = ((page * 2 + 1) * p.hkv + h) * PDT_PAGE;
          uint8_t* ks = smem + st * PDT_STAGE_BYTES;
          uint8_t* vs = ks + PDT_SLAB_BYTES;
          mbar_arrive_expect_tx(&kfull[st], PDT_SLAB_BYTES);
          tma_load_2d(ks, &tm_cache, &kfull[st], 0, krow);
          tma_load_2d(ks + PDT_PAGE * 128, &tm_cache, &kfull[st], 64, krow);
          mbar_arrive_expect_tx(&vfull[st], PDT_SLAB_BYTES);
          tma_load_2d(vs, &tm_cache, &vfull[st], 0, vrow);
          tma_load_2d(vs + PDT_D * 128, &tm_cache, &vfull[st], 64, vrow);
        }
        ++item_it;
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------ MMA issuer
    // S^T of tile t+1 (also the first tile of the next work item) is issued before the softmax warps have finished
    // tile t: S, P and the query tile are double-buffered, so the K.Q^T product never waits for the softmax.
    if (lane == 0) {
      constexpr uint32_t idesc = umma_idesc_bf16_f32(128, PDT_N);
      uint32_t kv_it = 0, item_it = 0;
      const uint32_t q_base = smem_u32(q_sh), p_base = smem_u32(p_sh);
      // issue S^T for global tile index `t` (ring stage / S buffer from t) with the query tile of item `it`
      auto mma1 = [&](uint32_t t, uint32_t it) -> bool {
        const uint32_t st = t % PDT_STAGES, ph = (t / PDT_STAGES) & 1;
        if (!mbar_wait(&kfull[st], ph)) return false;
        tc_fence_after_sync();
        const uint32_t ks = smem_u32(smem + st * PDT_STAGE_BYTES), qa = q_base + (it & 1) * PDT_Q_BYTES;
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          const uint32_t half = k >> 2, off = (k & 3) * 32;
          umma_bf16_ss(tmem_base + (t & 1) * 16, umma_desc_kmajor_sw128(ks + half * (PDT_PAGE * 128) + off),
                       umma_desc_kmajor_sw128(qa + half * (PDT_N * 128) + off), idesc, k > 0 ? 1u : 0u);
        }
        tc_commit(&s_ready[t & 1]);
        return true;
      };
      auto mma2 = [&](uint32_t t, bool first) {  // O^T += V^T . P^T
        const uint32_t st = t % PDT_STAGES;
        const uint32_t vs = smem_u32(smem + st * PDT_STAGE_BYTES + PDT_SLAB_BYTES), pa = p_base + (t & 1) * PDT_P_BYTES;
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          const uint32_t half = k >> 2, off = (k & 3) * 32;
          umma_bf16_ss(tmem_o, umma_desc_kmajor_sw128(vs + half * (PDT_D * 128) + off),
                       umma_desc_kmajor_sw128(pa + half * (PDT_N * 128) + off), idesc, (first && k == 0) ? 0u : 1u);
        }
      };
      bool ok = true, s_issued = false;
      for (int item = blockIdx.x; item < n_items && ok && !*abort_flag; item += gridDim.x) {
        const int ntiles = item_tiles(item);
        if (ntiles == 0) continue;
        const uint32_t qs = item_it & 1;
        if (!s_issued) {
          if (!mbar_wait(&qfull[qs], (item_it >> 1) & 1)) { atomicCAS(p.status, ST_OK, ST_TIMEOUT_FULL); *abort_flag = 1; break; }
          tc_fence_after_sync();
          if (!mma1(kv_it, item_it)) { atomicCAS(p.status, ST_OK, ST_TIMEOUT_FULL); *abort_flag = 1; break; }
        }
        s_issued = false;
        for (int j = 0; j < ntiles; ++j, ++kv_it) {
          const uint32_t st = kv_it % PDT_STAGES, ph = (kv_it / PDT_STAGES) & 1;
          // look ahead: S^T of the next tile, possibly the first tile of the next non-empty work item
          if (j + 1 < ntiles) {
            if (!mma1(kv_it + 1, item_it)) { atomicCAS(p.status, ST_OK, ST_TIMEOUT_FULL); *abort_flag = 1; ok = false; break; }
          } else {
            int nxt = item + gridDim.x;
            while (nxt < n_items && item_tiles(nxt) == 0) nxt += gridDim.x;
            if (nxt < n_items) {
              if (!mbar_wait(&qfull[(item_it + 1) & 1], ((item_it + 1) >> 1) & 1)) { atomicCAS(p.status, ST_OK, ST_TIMEOUT_FULL); *abort_flag = 1; ok = false; break; }
              tc_fence_after_sync();
              if (!mma1(kv_it + 1, item_it + 1)) { atomicCAS(p.status, ST_OK, ST_TIMEOUT_FULL); *abort_flag = 1; ok = false; break; }
              s_issued = true;
            }
          }
          if (!mbar_wait(&p_ready[kv_it & 1], (kv_it >> 1) & 1)) { atomicCAS(p.status, ST_OK, ST_TIMEOUT_TMEM_EMPTY); *abort_flag = 1; ok = false; break; }
          if (!mbar_wait(&vfull[st], ph)) { atomicCAS(p.status, ST_OK, ST_TIMEOUT_FULL); *abort_flag = 1; ok = false; break; }
          tc_fence_after_sync();
          mma2(kv_it, j == 0);
          tc_commit(&kvempty[st]);
          if (j + 1 == ntiles) {
            tc_commit(&qempty[qs]);
            tc_commit(o_ready);
          }
        }
        ++item_it;
      }
    }
  } else {
    // ------------------------------------------------ softmax / epilogue (warps 2..5)
    const int quad = warp & 3;
    const int row = quad * 32 + lane;            // TMEM lane of this thread
    const uint32_t lane_addr = (uint32_t)(quad * 32) << 16;
    uint32_t item_it = 0, tile_it = 0;
    bool ok = true;
    for (int item = blockIdx.x; item < n_items && ok && !*abort_flag; item += gridDim.x) {
      int b, h, split, t0, t1;
      item_range(item, b, h, split, t0, t1);
      const int ntiles = (t1 - t0 + PDT_PAGE - 1) / PDT_PAGE;
      if (ntiles == 0) {
        // empty split: an empty partial result (only reachable in the scratch modes), no barrier is touched
        for (int g = 0; g < G; ++g) {
          const long long head = (long long)b * p.hq + h * G + g;
          if (p.nsplit == 1 && !p.prefix_pages) {      // a sequence of length 0: define the output as zero
            p.out[head * PDT_D + row] = __float2bfloat16(0.f);
            continue;
          }
          const int ns = p.prefix_pages ? p.ns_total : p.nsplit;
          const int si = p.prefix_pages ? p.max_shared + split : split;
          float* sp = p.scratch + (head * ns + si) * (PDT_D + 2);
          sp[row] = 0.f;
          if (row == 0) { sp[PDT_D] = -INFINITY; sp[PDT_D + 1] = 0.f; }
        }
        continue;
      }
      float m_run[8], l_run[8];
#pragma unroll
      for (int g = 0; g < 8; ++g) { m_run[g] = -INFINITY; l_run[g] = 0.f; }
      for (int j = 0; j < ntiles; ++j, ++tile_it) {
        const uint32_t tb = tile_it & 1;
        if (!mbar_wait(&s_ready[tb], (tile_it >> 1) & 1)) { atomicCAS(p.status, ST_OK, ST_TIMEOUT_TMEM_FULL); *abort_flag = 1; ok = false; break; }
        tc_fence_after_sync();
        uint32_t sr[16];
        tmem_ld_32x32b_x16(tmem_base + tb * 16 + lane_addr, sr);
        tmem_ld_wait();
        const bool valid = (t0 + j * PDT_PAGE + row) < t1;
        float s[8], wmax[8];
#pragma unroll
        for (int g = 0; g < 8; ++g) {
          s[g] = valid ? __uint_as_float(sr[g]) * p.scale_log2 : -INFINITY;
          float v = s[g];
#pragma unroll
          for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
          wmax[g] = v;
        }
        if (lane == 0) {
#pragma unroll
          for (int g = 0; g < 8; ++g) red[quad * 8 + g] = wmax[g];
        }
        softmax_bar();
        float corr[8], pv[8], wsum[8];
#pragma unroll
        for (int g = 0; g < 8; ++g) {
          float tmax = fmaxf(fmaxf(red[g], red[8 + g]), fmaxf(red[16 + g], red[24 + g]));
          float nm = fmaxf(m_run[g], tmax);
          corr[g] = (nm == -INFINITY) ? 1.f : exp2f(m_run[g] - nm);
          pv[g] = (valid && nm != -INFINITY) ? exp2f(s[g] - nm) : 0.f;
          m_run[g] = nm;
          float v = pv[g];
#pragma unroll
          for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
          wsum[g] = v;
        }
        if (lane == 0) {
#pragma unroll
          for (int g = 0; g < 8; ++g) red[32 + quad * 8 + g] = wsum[g];
        }
        // The P tile written two tiles ago and the running output are in use until the PV product of the previous
        // tile has finished (kvempty of its ring stage).
        if (tile_it > 0) {
          const uint32_t pt = tile_it - 1;
          if (!mbar_wait(&kvempty[pt % PDT_STAGES], (pt / PDT_STAGES) & 1)) { atomicCAS(p.status, ST_OK, ST_TIMEOUT_TMEM_FULL); *abort_flag = 1; ok = false; }
          tc_fence_after_sync();
        }
        // P[head g][token row] -> shared memory, K-major rows of 64 tokens (128 bytes), 128-byte swizzle
        {
          const int half = row >> 6, tk = row & 63;
          const int chunk = tk >> 3, within = (tk & 7) * 2;
          uint8_t* base = p_sh + tb * PDT_P_BYTES + half * (PDT_N * 128);
#pragma unroll
          for (int g = 0; g < 8; ++g) {
            if (g < G) {
              const int sw = chunk ^ (g & 7);
              *reinterpret_cast<__nv_bfloat16*>(base + g * 128 + sw * 16 + within) = __float2bfloat16(pv[g]);
            }
          }
        }
        // rescale the running output (a head-dim row per thread, one column per head)
        if (j > 0) {
          uint32_t orr[16];
          tmem_ld_32x32b_x16(tmem_o + lane_addr, orr);
          tmem_ld_wait();
#pragma unroll
          for (int g = 0; g < 8; ++g) orr[g] = __float_as_uint(__uint_as_float(orr[g]) * corr[g]);
          tmem_st_32x32b_x16(tmem_o + lane_addr, orr);
          tmem_st_wait();
        }
        softmax_bar();
#pragma unroll
        for (int g = 0; g < 8; ++g)
          l_run[g] = l_run[g] * corr[g] + (red[32 + g] + red[40 + g] + red[48 + g] + red[56 + g]);
        fence_proxy_async_smem();
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive(&p_ready[tb]);
        if (!ok) break;
      }
      if (!ok) break;
      // ---- item epilogue
      if (!mbar_wait(o_ready, item_it & 1)) { atomicCAS(p.status, ST_OK, ST_TIMEOUT_TMEM_FULL); *abort_flag = 1; break; }
      tc_fence_after_sync();
      float o[8];
      {
        uint32_t orr[16];
        tmem_ld_32x32b_x16(tmem_o + lane_addr, orr);
        tmem_ld_wait();
#pragma unroll
        for (int g = 0; g < 8; ++g) o[g] = __uint_as_float(orr[g]);
      }
      tc_fence_before_sync();
#pragma unroll
      for (int g = 0; g < 8; ++g) {
        if (g < G) {
          const long long head = (long long)b * p.hq + h * G + g;
          if (p.nsplit == 1 && !p.prefix_pages) {
            p.out[head * PDT_D + row] = __float2bfloat16(l_run[g] > 0.f ? o[g] / l_run[g] : 0.f);
          } else {
            const int ns = p.prefix_pages ? p.ns_total : p.nsplit;
            const int si = p.prefix_pages ? p.max_shared + split : split;
            float* sp = p.scratch + (head * ns + si) * (PDT_D + 2);
            sp[row] = o[g];
            if (row == 0) { sp[PDT_D] = m_run[g]; sp[PDT_D + 1] = l_run[g]; }
          }
        }
      }
      softmax_bar();  // `red` and TMEM reads are done before the next item starts overwriting
      ++item_it;
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (*abort_flag && threadIdx.x == 0) {
    for (int i = 0; i < 100; ++i) __nanosleep(1000);  // let issued copies land before shared memory is released
  }
  __syncthreads();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, 64);
  }
}

// Merge of the partial results of one (sequence, head). Without prefix_pages: splits [0, nsplit). With it: the
// prefix pages [0, prefix_pages[b]) and the suffix splits [max_shared, max_shared + nsplit) out of ns slots.
__global__ void pdt_merge_kernel(const float* __restrict__ scratch, __nv_bfloat16* __restrict__ out, int nsplit,
                                 const int* __restrict__ prefix_pages, int max_shared, int hq) {
  pdl_launch_dependents();
  pdl_wait();
  const long long head = blockIdx.x;
  const int c = threadIdx.x;
  const int ns = prefix_pages ? max_shared + nsplit : nsplit;
  const int npre = prefix_pages ? min(prefix_pages[head / hq], max_shared) : 0;
  const float* sp = scratch + head * ns * (PDT_D + 2);
  float M = -INFINITY;
  for (int s = 0; s < ns; ++s) {
    if (prefix_pages && s >= npre && s < max_shared) continue;
    M = fmaxf(M, sp[s * (PDT_D + 2) + PDT_D]);
  }
  float L = 0.f, A = 0.f;
  for (int s = 0; s < ns; ++s) {
    if (prefix_pages && s >= npre && s < max_shared) continue;
    const float ms = sp[s * (PDT_D + 2) + PDT_D];
    const float cw = (ms == -INFINITY) ? 0.f : exp2f(ms - M);
    L += sp[s * (PDT_D + 2) + PDT_D + 1] * cw;
    A += sp[s * (PDT_D + 2) + c] * cw;
  }
  out[head * PDT_D + c] = __float2bfloat16(L > 0.f ? A / L : 0.f);
}

// ---------------------------------------------------------------------------------------------------------------
// Shared-prefix pass. The n samples of a prompt group share the prompt's full pages; instead of every sequence
// streaming those pages again, one CTA per (shared page, kv head, group) loads the page once and attends ALL
// query rows of the group that use this kv head: rows (sample j, head g) = n * G <= 128 rows of one MMA.
//     S[rows, 128 tokens] = Q K^T,  P = exp2(S c - rowmax),  O[rows, d] = P V        (V^T slab = K-major B operand)
// Every row's (o, m, l) goes to split slot `page` of that (sequence, head); the merge kernel combines them with
// the per-sequence suffix. The group's sequences occupy consecutive slots [grp * n, grp * n + n).
// ---------------------------------------------------------------------------------------------------------------
// RMAX = 64 keeps only 64 query / probability rows in shared memory (two CTAs per SM); the M = 128 MMAs then read
// rows 64..127 from whatever follows, and those accumulator rows are never used.
template <int RMAX> constexpr int ppf_smem() { return 2 * PDT_SLAB_BYTES + 2 * (RMAX * 256) + 256 + 1024; }

struct PpfParams {
  const int* block_table;
  const int* prefix_pages;
  float* scratch;
  int B, hq, hkv, max_pages, n, ns_total;
  float scale_log2;
  uint32_t* status;
};

template <int RMAX>
__global__ void __launch_bounds__(PDT_THREADS, RMAX == 64 ? 2 : 1)
paged_prefix_tc_kernel(const __grid_constant__ CUtensorMap tm_cache, const __grid_constant__ CUtensorMap tm_q3,
                       PpfParams p) {
  constexpr int QP_BYTES = RMAX * 256;         // two halves of RMAX rows x 128 bytes
  constexpr int QP_HALF = RMAX * 128;
  const int pg = blockIdx.x, hk = blockIdx.y, s0 = blockIdx.z * p.n;
  if (s0 >= p.B) return;
  // the group's shared page count / page list come from its first member that still has a prefix
  int shared = 0, owner = s0;
  for (int j = 0; j < p.n && s0 + j < p.B; ++j) {
    const int v = p.prefix_pages[s0 + j];
    if (v > shared) { shared = v; owner = s0 + j; }
  }
  if (pg >= shared) return;
  const int page = p.block_table[(long long)owner * p.max_pages + pg];
  const int G = p.hq / p.hkv;
  const int rows_used = p.n * G;

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  // order: Q, P, K, V^T so that the over-reads of the 64-row variant stay inside the allocation
  uint8_t* q_sh = smem;
  uint8_t* p_sh = smem + QP_BYTES;
  uint8_t* k_sh = smem + 2 * QP_BYTES;
  uint8_t* v_sh = k_sh + PDT_SLAB_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(v_sh + PDT_SLAB_BYTES);
  uint64_t* qk_full = bars;
  uint64_t* v_full = bars + 1;
  uint64_t* s_ready = bars + 2;
  uint64_t* p_ready = bars + 3;
  uint64_t* o_ready = bars + 4;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 5);
  volatile uint32_t* abort_flag = tmem_slot + 1;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    mbar_init(qk_full, 1);
    mbar_init(v_full, 1);
    mbar_init(s_ready, 1);
    mbar_init(p_ready, 4);
    mbar_init(o_ready, 1);
    *abort_flag = 0;
    mbar_fence_init();
  }
  // rows of the query tile that the TMA box does not cover must not hold NaN bit patterns
  for (int i = threadIdx.x; i < QP_BYTES / 16; i += blockDim.x) reinterpret_cast<uint4*>(q_sh)[i] = make_uint4(0, 0, 0, 0);
  if (warp == 1) {
    tmem_alloc(tmem_slot, 256);
    tmem_relinquish();
  }
  fence_proxy_async_smem();
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tmem_s = tmem_base, tmem_o = tmem_base + 128;

  if (warp == 0) {
    if (lane == 0) {
      const uint32_t q_bytes = 2u * (uint32_t)rows_used * 128u;
      mbar_arrive_expect_tx(qk_full, q_bytes + PDT_SLAB_BYTES);
      tma_load_3d(q_sh, &tm_q3, qk_full, 0, hk * G, s0);
      tma_load_3d(q_sh + QP_HALF, &tm_q3, qk_full, 64, hk * G, s0);
      const int krow = ((page * 2 + 0) * p.hkv + hk) * PDT_PAGE;
      const int vrow = ((page * 2 + 1) * p.hkv + hk) * PDT_PAGE;
      tma_load_2d(k_sh, &tm_cache, qk_full, 0, krow);
      tma_load_2d(k_sh + PDT_SLAB_BYTES / 2, &tm_cache, qk_full, 64, krow);
      mbar_arrive_expect_tx(v_full, PDT_SLAB_BYTES);
      tma_load_2d(v_sh, &tm_cache, v_full, 0, vrow);
      tma_load_2d(v_sh + PDT_SLAB_BYTES / 2, &tm_cache, v_full, 64, vrow);
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc = umma_idesc_bf16_f32(128, 128);
      const uint32_t q_a = smem_u32(q_sh), k_a = smem_u32(k_sh), v_a = smem_u32(v_sh), p_a = smem_u32(p_sh);
      do {
        if (!mbar_wait(qk_full, 0)) { atomicCAS(p.status, ST_OK, ST_TIMEOUT_FULL); *abort_flag = 1; break; }
        tc_fence_after_sync();
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          const uint32_t off = (k >> 2) * (PDT_SLAB_BYTES / 2) + (k & 3) * 32;
          const uint32_t qoff = (k >> 2) * QP_HALF + (k & 3) * 32;
          umma_bf16_ss(tmem_s, umma_desc_kmajor_sw128(q_a + qoff), umma_desc_kmajor_sw128(k_a + off), idesc, k > 0 ? 1u : 0u);
        }
        tc_commit(s_ready);
        if (!mbar_wait(p_ready, 0) || !mbar_wait(v_full, 0)) { atomicCAS(p.status, ST_OK, ST_TIMEOUT_FULL); *abort_flag = 1; break; }
        tc_fence_after_sync();
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          const uint32_t off = (k >> 2) * (PDT_SLAB_BYTES / 2) + (k & 3) * 32;
          const uint32_t poff = (k >> 2) * QP_HALF + (k & 3) * 32;
          umma_bf16_ss(tmem_o, umma_desc_kmajor_sw128(p_a + poff), umma_desc_kmajor_sw128(v_a + off), idesc, k > 0 ? 1u : 0u);
        }
        tc_commit(o_ready);
      } while (false);
    }
  } else {
    const int quad = warp & 3;
    const int row = quad * 32 + lane;
    const uint32_t lane_addr = (uint32_t)(quad * 32) << 16;
    bool ok = mbar_wait(s_ready, 0);
    if (!ok) { atomicCAS(p.status, ST_OK, ST_TIMEOUT_TMEM_FULL); *abort_flag = 1; }
    ok = __all_sync(0xffffffffu, ok);
    float m = -INFINITY, l = 0.f;
    if (ok) {
      tc_fence_after_sync();
#pragma unroll 1
      for (int c = 0; c < PDT_PAGE; c += 32) {
        uint32_t r[32];
        tmem_ld_32x32b_x32(tmem_s + lane_addr + c, r);
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 32; ++i) m = fmaxf(m, __uint_as_float(r[i]));
      }
      m *= p.scale_log2;
#pragma unroll 1
      for (int c = 0; c < PDT_PAGE; c += 32) {
        uint32_t r[32];
        tmem_ld_32x32b_x32(tmem_s + lane_addr + c, r);
        tmem_ld_wait();
        float e[32];
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          e[i] = exp2f(fmaf(__uint_as_float(r[i]), p.scale_log2, -m));
          l += e[i];
        }
        uint8_t* dst = p_sh + (c >> 6) * QP_HALF + row * 128;
        const int chunk0 = (c & 63) >> 3;
        if (row < RMAX) {
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
      }
      fence_proxy_async_smem();
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(p_ready);
      if (!mbar_wait(o_ready, 0)) { atomicCAS(p.status, ST_OK, ST_TIMEOUT_TMEM_FULL); *abort_flag = 1; ok = false; }
      ok = __all_sync(0xffffffffu, ok);
    }
    if (ok) {
      tc_fence_after_sync();
      const int j = row / G, g = row % G;
      const bool live = row < rows_used && s0 + j < p.B;
      float* sp = p.scratch + (((long long)(s0 + j) * p.hq + hk * G + g) * p.ns_total + pg) * (PDT_D + 2);
#pragma unroll 1
      for (int c = 0; c < PDT_D; c += 32) {
        uint32_t r[32];
        tmem_ld_32x32b_x32(tmem_o + lane_addr + c, r);
        tmem_ld_wait();
        if (live) {
#pragma unroll
          for (int i = 0; i < 32; i += 2) *reinterpret_cast<float2*>(sp + c + i) = make_float2(__uint_as_float(r[i]), __uint_as_float(r[i + 1]));
        }
      }
      if (live) { sp[PDT_D] = m; sp[PDT_D + 1] = l; }
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
    tmem_dealloc(tmem_base, 256);
  }
}

// V is stored transposed: slab (page, 1, h) = [d, token]
__global__ void kv_append_vt_kernel(const __nv_bfloat16* __restrict__ k, const __nv_bfloat16* __restrict__ v,
                                    __nv_bfloat16* __restrict__ cache, const int* __restrict__ slot_mapping, int T,
                                    int hkv, long long k_stride, long long v_stride) {
  const int vec_per_tok = hkv * PDT_D / 8;
  long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= (long long)T * vec_per_tok) return;
  const int t = (int)(idx / vec_per_tok);
  const int e = (int)(idx % vec_per_tok) * 8;
  const int slot = slot_mapping[t];
  if (slot < 0) return;
  const int page = slot / PDT_PAGE, off = slot % PDT_PAGE;
  const int h = e / PDT_D, c = e % PDT_D;
  const long long slab = (long long)PDT_PAGE * PDT_D;
  __nv_bfloat16* kd = cache + ((long long)(page * 2 + 0) * hkv + h) * slab + (long long)off * PDT_D + c;
  *reinterpret_cast<uint4*>(kd) = *reinterpret_cast<const uint4*>(k + t * k_stride + e);
  __nv_bfloat16* vd = cache + ((long long)(page * 2 + 1) * hkv + h) * slab + (long long)c * PDT_PAGE + off;
  uint4 vv = *reinterpret_cast<const uint4*>(v + t * v_stride + e);
  const __nv_bfloat16* ve = reinterpret_cast<const __nv_bfloat16*>(&vv);
#pragma unroll
  for (int i = 0; i < 8; ++i) vd[(long long)i * PDT_PAGE] = ve[i];
}

}  // namespace b200

extern "C" {

int b200_kv_append_vt(const void* k, const void* v, void* cache, const int* slot_mapping, int T, int hkv, int d,
                      long long k_stride, long long v_stride, int page_size, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (d != b200::PDT_D || page_size != b200::PDT_PAGE) return B200_ERR_ARG;
  long long n = (long long)T * hkv * d / 8;
  b200::kv_append_vt_kernel<<<(unsigned)((n + 255) / 256), 256, 0, stream>>>(
      (const __nv_bfloat16*)k, (const __nv_bfloat16*)v, (__nv_bfloat16*)cache, slot_mapping, T, hkv, k_stride, v_stride);
  return cudaGetLastError() == cudaSuccess ? 0 : B200_ERR_LAUNCH;
}

int b200_paged_decode_tc(const void* q, const void* cache, long long num_pages, const int* block_table,
                         const int* seq_lens, void* out, float* scratch, int B, int hq, int hkv, int d, int page_size,
                         int max_pages, int nsplit, float scale, uint32_t* status, int num_sms, cudaStream_t stream) {
  return b200_paged_decode_prefix_tc(q, cache, num_pages, block_table, seq_lens, out, scratch, B, hq, hkv, d, page_size,
                                     max_pages, nsplit, scale, nullptr, 0, 0, status, num_sms, stream);
}

// prefix_pages (int32 [B], nullable): number of leading pages of each sequence that are shared by the `group`
// consecutive sequences of its group (0 = none). max_shared bounds it. scratch: B * hq * (max_shared + nsplit) * (d + 2).
int b200_paged_decode_prefix_tc(const void* q, const void* cache, long long num_pages, const int* block_table,
                                const int* seq_lens, void* out, float* scratch, int B, int hq, int hkv, int d,
                                int page_size, int max_pages, int nsplit, float scale, const int* prefix_pages,
                                int group, int max_shared, uint32_t* status, int num_sms, cudaStream_t stream) {
  using namespace b200;
  if (B <= 0) return 0;
  if (d != PDT_D || page_size != PDT_PAGE || hkv <= 0 || hq % hkv || hq / hkv > 8 || nsplit <= 0 ||
      ((nsplit > 1 || prefix_pages) && !scratch))
    return B200_ERR_ARG;
  const int G = hq / hkv;
  if (prefix_pages && (group <= 0 || group * G > 128 || max_shared <= 0)) return B200_ERR_ARG;
  CUtensorMap tm_cache, tm_q;
  if (make_tmap_2d(&tm_cache, cache, (uint64_t)num_pages * 2 * hkv * PDT_PAGE, PDT_D, PDT_D, PDT_PAGE, 64, 2))
    return B200_ERR_TENSORMAP;
  if (make_tmap_2d(&tm_q, q, (uint64_t)B * hq, PDT_D, PDT_D, PDT_N, 64, 2)) return B200_ERR_TENSORMAP;
  static bool attr_set = false;
  if (!attr_set) {
    if (cudaFuncSetAttribute(paged_decode_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, PDT_SMEM) !=
            cudaSuccess ||
        cudaFuncSetAttribute(paged_prefix_tc_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             ppf_smem<64>()) != cudaSuccess ||
        cudaFuncSetAttribute(paged_prefix_tc_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             ppf_smem<128>()) != cudaSuccess)
      return B200_ERR_LAUNCH;
    attr_set = true;
  }
  const int ns_total = prefix_pages ? max_shared + nsplit : nsplit;
  if (prefix_pages) {
    CUtensorMap tm_q3;
    if (make_tmap_3d(&tm_q3, q, B, hq, PDT_D, PDT_D, (uint64_t)hq * PDT_D, G, 64, 2, group)) return B200_ERR_TENSORMAP;
    PpfParams pp{block_table, prefix_pages, scratch, B, hq, hkv, max_pages, group, ns_total, scale * PDT_LOG2E, status};
    dim3 grid(max_shared, hkv, (B + group - 1) / group);
    if (group * G <= 64)
      paged_prefix_tc_kernel<64><<<grid, PDT_THREADS, ppf_smem<64>(), stream>>>(tm_cache, tm_q3, pp);
    else
      paged_prefix_tc_kernel<128><<<grid, PDT_THREADS, ppf_smem<128>(), stream>>>(tm_cache, tm_q3, pp);
  }
  PdtParams p{block_table, seq_lens, (__nv_bfloat16*)out, scratch, B, hq, hkv, max_pages, nsplit, scale * PDT_LOG2E,
              status, prefix_pages, max_shared, ns_total};
  const int items = B * hkv * nsplit;
  const int grid = items < num_sms ? items : num_sms;
  if (launch_pdl(paged_decode_tc_kernel, dim3(grid), dim3(PDT_THREADS), PDT_SMEM, stream, tm_cache, tm_q, p) != cudaSuccess)
    return B200_ERR_LAUNCH;
  if (nsplit > 1 || prefix_pages)
    if (launch_pdl(pdt_merge_kernel, dim3(B * hq), dim3(PDT_D), 0, stream, scratch, (__nv_bfloat16*)out, nsplit, prefix_pages,
                   max_shared, hq) != cudaSuccess)
      return B200_ERR_LAUNCH;
  return cudaGetLastError() == cudaSuccess ? 0 : B200_ERR_LAUNCH;
}

}  // extern "C"
