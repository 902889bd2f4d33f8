// Dense bf16 GEMM main loop for CTA pairs (tcgen05 cta_group::2) on sm_100a.
//
//   D[M, N] = A[M, K] * B[N, K]^T      (fp32 accumulate; operands K-major or MN-major)
//
// Two CTAs of a cluster work on one 256 x BN output tile. Each CTA streams ITS half of the operands (128 rows
// of A, BN/2 rows of B) into its own shared-memory ring with plain TMA loads (no cluster multicast), the leader
// CTA issues one tcgen05.mma (M = 256) per 16 contraction elements that reads both CTAs' shared memory, and
// each CTA keeps the fp32 accumulator of its own 128 rows in its own TMEM (two accumulators, so the epilogue
// of tile i overlaps the main loop of tile i + 1). Compared with one CTA per 128 x BN tile this halves the
// shared-memory traffic for B, which is what bounds the single-CTA kernel.
//
// Epilogue: the four epilogue warps of each CTA read their TMEM lane quadrant with tcgen05.ld, convert, write
// 32-row x 128-byte slabs into swizzled staging buffers and hand them to TMA stores (or TMA reduce-adds when
// the result is accumulated into C). TMA clips rows and columns outside C, so no edge code exists.
//
// Barriers (per CTA unless stated): full[s] (leader's is the one in use; loads of both CTAs complete on it),
// empty[s] (the leader's tcgen05.commit arrives on both CTAs'), tfull[a] (same), tempty[a] (leader's; the 8
// epilogue warps of the pair arrive on it). Every wait is bounded; on a timeout the kernel records a status
// code, lets the copies in flight land, frees its TMEM and returns.
#pragma once
#include "gemm_core.cuh"

namespace b200 {

constexpr int G2_BM_CTA = 128;  // accumulator rows per CTA
constexpr int G2_BM = 256;      // rows of the pair's tile
constexpr int G2_BK = 64;
constexpr int G2_THREADS = 192;

enum { G2_EPI_STORE = 0, G2_EPI_SWIGLU = 1 };

template <int BN, int STAGES>
struct Gemm2Smem {
  static constexpr int A_BYTES = G2_BM_CTA * G2_BK * 2;
  static constexpr int B_BYTES = (BN / 2) * G2_BK * 2;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int STAGING_BYTES = 4 * 2 * 4096;  // 4 epilogue warps x 2 slabs of 32 rows x 128 bytes
  static constexpr int BAR_BYTES = 256;
  static constexpr int TOTAL = STAGES * STAGE_BYTES + STAGING_BYTES + BAR_BYTES + 1024;
};

struct Gemm2Params {
  const void* bias;  // [N] added to every row (nullable); bf16 when bias_bf16 else fp32
  int bias_bf16;
  int out_fp32;      // element type of C (the C tensor map must agree)
  int accumulate;    // C += result (TMA reduce-add)
  int up_row0;       // G2_EPI_SWIGLU: first row of the "up" half inside B (= intermediate size)
  int group_m;       // raster: tiles of this many 256-row blocks share their B columns in time
};

// tile index -> (m_blk, n_blk): groups of `G` row blocks sweep all column blocks before the next group starts, so
// the tiles in flight at any time reuse a bounded set of A and B panels out of L2.
__device__ __forceinline__ void g2_tile_coords(int i, int num_m, int num_n, int G, int& m_blk, int& n_blk) {
  const int group_size = G * num_n;
  const int group = i / group_size;
  const int first_m = group * G;
  const int gsz = min(num_m - first_m, G);
  const int r = i - group * group_size;
  m_blk = first_m + r % gsz;
  n_blk = r / gsz;
}

template <int BN, int STAGES, bool A_MN, bool B_MN, int EPI>
__device__ __forceinline__ void gemm2_mainloop(const CUtensorMap* tmA, const CUtensorMap* tmB, const CUtensorMap* tmC,
                                               int M, int N, int K, const Gemm2Params& ep, uint32_t* status) {
  using SM = Gemm2Smem<BN, STAGES>;
  static_assert(BN == 128 || BN == 256, "BN");
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* staging = smem + STAGES * SM::STAGE_BYTES;
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(staging + SM::STAGING_BYTES);
  uint64_t* empty_bar = full_bar + STAGES;
  uint64_t* tfull_bar = empty_bar + STAGES;  // [2]
  uint64_t* tempty_bar = tfull_bar + 2;      // [2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty_bar + 2);
  volatile uint32_t* abort_flag = tmem_slot + 1;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t cta_rank = cluster_ctarank();  // 0: leader of the pair
  const bool leader = cta_rank == 0;
  constexpr uint32_t TMEM_COLS = 2 * BN;  // 256 or 512: a power of two

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&tfull_bar[a], 1);
      mbar_init(&tempty_bar[a], 8);  // 4 epilogue warps of each CTA of the pair
    }
    *abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(tmA);
    tma_prefetch_desc(tmB);
    tma_prefetch_desc(tmC);
  }
  if (warp == 1) {
    tmem_alloc_pair(tmem_slot, TMEM_COLS);
    tmem_relinquish_pair();
  }
  tc_fence_before_sync();
  __syncthreads();
  cluster_sync_all();  // both CTAs' barriers exist before anything arrives on them from the other side
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  const int num_m = (M + G2_BM - 1) / G2_BM;
  constexpr int OUT_BN = (EPI == G2_EPI_SWIGLU) ? BN / 2 : BN;  // columns of C per tile
  const int n_cols = (EPI == G2_EPI_SWIGLU) ? N / 2 : N;        // columns of C
  const int num_n = (n_cols + OUT_BN - 1) / OUT_BN;
  const int total = num_m * num_n;
  const int num_kb = (K + G2_BK - 1) / G2_BK;
  const int cluster_id = blockIdx.x >> 1;
  const int num_clusters = gridDim.x >> 1;
  const int G = ep.group_m > 0 ? ep.group_m : 8;

  if (warp == 0) {
    // ------------------------------ TMA producer (both CTAs) ------------------------------
    if (lane == 0) {
      uint32_t stage = 0, phase = 0;
      bool ok = true;
      for (int i = cluster_id; i < total && ok && !*abort_flag; i += num_clusters) {
        int m_blk, n_blk;
        g2_tile_coords(i, num_m, num_n, G, m_blk, n_blk);
        const int a_row0 = m_blk * G2_BM + (int)cta_rank * G2_BM_CTA;
        // rows of B that this CTA feeds: its half of the tile's columns; with the SwiGLU epilogue the leader
        // feeds the gate rows and the other CTA the matching up rows, so a thread sees both in its TMEM lane
        int b_row0;
        if constexpr (EPI == G2_EPI_SWIGLU) b_row0 = n_blk * (BN / 2) + (cta_rank ? ep.up_row0 : 0);
        else b_row0 = n_blk * BN + (int)cta_rank * (BN / 2);
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(&empty_bar[stage], phase ^ 1)) {
            atomicCAS(status, ST_OK, ST_TIMEOUT_EMPTY);
            *abort_flag = 1;
            ok = false;
            break;
          }
          uint8_t* sa = smem + stage * SM::STAGE_BYTES;
          uint8_t* sb = sa + SM::A_BYTES;
          const int k = kb * G2_BK;
          if (leader) mbar_arrive_expect_tx(&full_bar[stage], 2 * SM::STAGE_BYTES);
          const uint32_t bar = mapa_shared(smem_u32(&full_bar[stage]), 0);
          if constexpr (!A_MN) {
            tma_load_2d_pair(sa, tmA, bar, k, a_row0);
          } else {
#pragma unroll
            for (int j = 0; j < G2_BM_CTA / 64; ++j) tma_load_2d_pair(sa + j * 8192, tmA, bar, a_row0 + j * 64, k);
          }
          if constexpr (!B_MN) {
            tma_load_2d_pair(sb, tmB, bar, k, b_row0);
          } else {
#pragma unroll
            for (int j = 0; j < (BN / 2) / 64; ++j) tma_load_2d_pair(sb + j * 8192, tmB, bar, b_row0 + j * 64, k);
          }
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
      }
      // tail: the leader's commits keep arriving on this CTA's empty barriers until its last MMA retired; the CTA
      // must not exit (and release its shared memory) before they have landed
      if (ok && !*abort_flag) {
        for (int s = 0; s < STAGES; ++s) {
          if (!mbar_wait(&empty_bar[stage], phase ^ 1)) {
            atomicCAS(status, ST_OK, ST_TIMEOUT_EMPTY);
            *abort_flag = 1;
            break;
          }
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------ MMA issuer (leader CTA only) --------------------------
    if (leader && lane == 0) {
      constexpr uint32_t idesc =
          umma_idesc_bf16_f32(G2_BM, BN) | (A_MN ? (1u << 15) : 0u) | (B_MN ? (1u << 16) : 0u);
      uint32_t stage = 0, phase = 0;
      uint32_t acc = 0, acc_phase = 0;
      bool ok = true;
      for (int i = cluster_id; i < total && ok && !*abort_flag; i += num_clusters) {
        if (!mbar_wait(&tempty_bar[acc], acc_phase ^ 1)) {
          atomicCAS(status, ST_OK, ST_TIMEOUT_TMEM_EMPTY);
          *abort_flag = 1;
          break;
        }
        tc_fence_after_sync();
        const uint32_t tmem_d = tmem_base + acc * BN;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(&full_bar[stage], phase)) {
            atomicCAS(status, ST_OK, ST_TIMEOUT_FULL);
            *abort_flag = 1;
            ok = false;
            break;
          }
          tc_fence_after_sync();
          const uint32_t sa = smem_u32(smem + stage * SM::STAGE_BYTES);
          const uint32_t sb = sa + SM::A_BYTES;
#pragma unroll
          for (int k = 0; k < G2_BK / 16; ++k) {
            uint64_t ad = A_MN ? umma_desc_mnmajor_sw128(sa + k * 2048, 8192) : umma_desc_kmajor_sw128(sa + k * 32);
            uint64_t bd = B_MN ? umma_desc_mnmajor_sw128(sb + k * 2048, 8192) : umma_desc_kmajor_sw128(sb + k * 32);
            umma_bf16_ss_pair(tmem_d, ad, bd, idesc, (kb > 0 || k > 0) ? 1u : 0u);
          }
          tc_commit_pair(&empty_bar[stage], 3);  // frees this stage in both CTAs once the MMAs retire
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
        if (!ok) break;
        tc_commit_pair(&tfull_bar[acc], 3);  // accumulator complete, in both CTAs
        if (++acc == 2) { acc = 0; acc_phase ^= 1; }
      }
    }
  } else {
    // ------------------------------ epilogue (warps 2..5 of both CTAs) --------------------
    const int quad = warp & 3;  // TMEM lane quadrant this warp may access
    uint8_t* slab0 = staging + quad * 8192;
    const uint32_t tempty_leader0 = mapa_shared(smem_u32(&tempty_bar[0]), 0);
    const uint32_t tempty_leader1 = mapa_shared(smem_u32(&tempty_bar[1]), 0);
    uint32_t acc = 0, acc_phase = 0;
    uint32_t slab_idx = 0;
    const uint32_t sw = (uint32_t)(lane & 7);  // 128-byte swizzle: 16-byte chunk j of row r sits at chunk j ^ (r & 7)
    for (int i = cluster_id; i < total && !*abort_flag; i += num_clusters) {
      int m_blk, n_blk;
      g2_tile_coords(i, num_m, num_n, G, m_blk, n_blk);
      if (!mbar_wait(&tfull_bar[acc], acc_phase)) {
        atomicCAS(status, ST_OK, ST_TIMEOUT_TMEM_FULL);
        *abort_flag = 1;
        break;
      }
      tc_fence_after_sync();
      const uint32_t taddr = tmem_base + acc * BN + ((uint32_t)(quad * 32) << 16);
      const int row0 = m_blk * G2_BM + (int)cta_rank * G2_BM_CTA + quad * 32;  // first row of this warp's slabs
      const int col_base = n_blk * OUT_BN;
      // a slab = 32 rows x 128 bytes of C: 64 bf16 or 32 fp32 columns
      const int slab_cols = ep.out_fp32 ? 32 : 64;
#pragma unroll 1
      for (int c = 0; c < OUT_BN; c += slab_cols) {
        uint8_t* slab = slab0 + (slab_idx & 1) * 4096;
        // the store issued two slabs ago has finished reading this buffer
        if (lane == 0) tma_store_wait_read<1>();
        __syncwarp();
        uint8_t* my_row = slab + lane * 128;
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          if (ep.out_fp32 && h == 1) break;
          const int cc = c + h * 32;  // 32 accumulator columns [cc, cc + 32)
          uint32_t r[32];
          tmem_ld_32x32b_x32(taddr + cc, r);
          float v[32];
          if constexpr (EPI == G2_EPI_SWIGLU) {
            uint32_t u[32];
            tmem_ld_32x32b_x32(taddr + BN / 2 + cc, u);
            tmem_ld_wait();
#pragma unroll
            for (int j = 0; j < 32; ++j) {
              const float g = __uint_as_float(r[j]);
              v[j] = g / (1.f + __expf(-g)) * __uint_as_float(u[j]);
            }
          } else {
            tmem_ld_wait();
#pragma unroll
            for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(r[j]);
            if (ep.bias != nullptr) {
              const int gc = col_base + cc;
#pragma unroll
              for (int j = 0; j < 32; ++j) {
                if (gc + j < n_cols)
                  v[j] += ep.bias_bf16 ? __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(ep.bias)[gc + j])
                                       : reinterpret_cast<const float*>(ep.bias)[gc + j];
              }
            }
          }
          if (ep.out_fp32) {
#pragma unroll
            for (int j = 0; j < 8; ++j) {  // 8 chunks of 4 floats
              float4 o = make_float4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
              *reinterpret_cast<float4*>(my_row + ((((uint32_t)j) ^ sw) << 4)) = o;
            }
          } else {
#pragma unroll
            for (int j = 0; j < 4; ++j) {  // 4 chunks of 8 bf16; this half starts at chunk 4 * h
              uint4 o;
              o.x = pack_bf16x2(v[8 * j], v[8 * j + 1]);
              o.y = pack_bf16x2(v[8 * j + 2], v[8 * j + 3]);
              o.z = pack_bf16x2(v[8 * j + 4], v[8 * j + 5]);
              o.w = pack_bf16x2(v[8 * j + 6], v[8 * j + 7]);
              *reinterpret_cast<uint4*>(my_row + ((((uint32_t)(4 * h + j)) ^ sw) << 4)) = o;
            }
          }
        }
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) {
          const int gc = col_base + c;
          if (gc < n_cols && row0 < M) {
            if (ep.accumulate) tma_reduce_add_2d(tmC, slab, gc, row0);
            else tma_store_2d(tmC, slab, gc, row0);
          }
          tma_store_commit();
        }
        ++slab_idx;
      }
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(acc ? tempty_leader1 : tempty_leader0);
      if (++acc == 2) { acc = 0; acc_phase ^= 1; }
    }
    if (lane == 0) tma_store_wait<0>();
  }

  // ------------------------------ teardown ------------------------------------
  tc_fence_before_sync();
  __syncthreads();
  if (*abort_flag && threadIdx.x == 0) {
    // let copies that were already issued land before the CTA's shared memory is released
    for (int i = 0; i < 100; ++i) __nanosleep(1000);
  }
  cluster_sync_all();  // neither CTA frees TMEM or exits while the other may still signal it
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc_pair(tmem_base, TMEM_COLS);
  }
}

// Row-major [rows, cols] tensor of fp32 / bf16 for the epilogue's TMA stores: box = 32 rows x 128 bytes, 128-byte swizzle.
inline int make_tmap_out(CUtensorMap* out, const void* ptr, uint64_t rows, uint64_t cols, uint64_t ld, int out_fp32) {
  PFN_encodeTiled enc = get_encode_tiled();
  if (!enc) { last_tmap_error() = 1 << 24; return -1; }
  const int eb = out_fp32 ? 4 : 2;
  if ((reinterpret_cast<uintptr_t>(ptr) & 15) || ((ld * eb) & 15)) {
    last_tmap_error() = (2 << 24) | 0x10000;
    return -2;
  }
  cuuint64_t gdim[2] = {cols, rows};
  cuuint64_t gstr[1] = {ld * (uint64_t)eb};
  cuuint32_t box[2] = {(cuuint32_t)(128 / eb), 32};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = encode_with_context([&] {
    return enc(out, out_fp32 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2,
               const_cast<void*>(ptr), gdim, gstr, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
               CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  });
  if (r != CUDA_SUCCESS) last_tmap_error() = (3 << 24) | 0x10000 | (int)r;
  return r == CUDA_SUCCESS ? 0 : -3;
}

}  // namespace b200
