// Persistent, warp-specialised tcgen05 GEMM main loop for sm_100a.
//
//   D[M, N] = A[M, K] * B[N, K]^T      (both operands K-major, bf16, fp32 accumulate)
//
// One CTA per SM walks a list of 128 x BN output tiles. Warp 0 streams A/B tiles
// into a STAGES-deep shared-memory ring with TMA (128-byte swizzle), warp 1 issues
// tcgen05.mma (M=128, N=BN, K=16) from a single elected thread into one of two
// TMEM accumulators, and warps 2..5 drain the other accumulator with tcgen05.ld
// and hand 32-column row fragments to an Epilogue functor. The epilogue of tile i
// overlaps the main loop of tile i+1.
//
// The Epilogue and the tile Schedule are template parameters so that fused
// kernels (online-softmax log-prob, gather-from-peer prologues, ...) reuse the
// same pipeline. All mbarrier waits are bounded; on a timeout the kernel records
// a status code, frees its TMEM and returns.
#pragma once
#include <type_traits>

#include "sm100.cuh"

namespace b200 {

constexpr int GEMM_BM = 128;
constexpr int GEMM_BK = 64;  // 64 bf16 = 128 bytes = one swizzle row
constexpr int GEMM_THREADS = 192;

template <int BN, int STAGES>
struct GemmSmem {
  static constexpr int A_BYTES = GEMM_BM * GEMM_BK * 2;
  static constexpr int B_BYTES = BN * GEMM_BK * 2;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int BAR_BYTES = 256;
  // +1024 so the ring can be aligned to 1024 bytes inside dynamic shared memory
  static constexpr int TOTAL = STAGES * STAGE_BYTES + BAR_BYTES + 1024;
  // Epilogues that stage their output in shared memory (TMA stores) get EPI_BYTES more, 1024-byte aligned, after
  // the barriers: launch with TOTAL_WITH_EPI and read the pointer that the custom tile() call receives.
  static constexpr int EPI_OFFSET = STAGES * STAGE_BYTES + 1024;
  static constexpr int EPI_BYTES = 4 * 2 * 4096;  // 4 epilogue warps x 2 slabs of 32 rows x 128 bytes
  static constexpr int TOTAL_WITH_EPI = EPI_OFFSET + EPI_BYTES + 1024;
};

// One output tile as seen by every role of the pipeline.
struct TileInfo {
  int m_blk, n_blk;  // tile indices handed to the epilogue
  int a_mn0;         // first row of the A operand (coordinate along A's M dimension)
  int b_mn0;         // first row of the B operand (coordinate along B's N dimension)
  int k0;            // first contraction index
  int num_kb;        // number of 64-wide contraction blocks
  int batch;         // third tensor-map coordinate (expert / batch index) when a map is 3-D
  int b_mn1;         // Traits::B_TWO_BOXES: first row of the second half of the B tile (rows b_mn0.. and b_mn1..)
};

// Operand layouts. K-major: the contraction index is contiguous in memory (x[M,K] row-major, W[N,K]
// row-major). MN-major: the M (or N) index is contiguous, i.e. the operand is stored transposed
// ([K, M] row-major); this is what dgrad (B = W[N,K] contracted over N) and wgrad (both operands contracted
// over the token dimension) need, so no transposed copies are ever made.
// SIDE_WARPS > 0: the CTA is launched with GEMM_THREADS + 32 * SIDE_WARPS threads and warps 6.. run
// Epi::side() concurrently with the pipeline (used by the fused GEMM + cross-GPU reduction kernel).
// PRODUCER_HOOK: the TMA producer calls sched.before_tile_load(tile, ep, status) before the first load of a tile
// and gives up (abort) when it returns false (used to wait for operand rows that another GPU is still sending).
// B_TWO_BOXES (K-major 2-D B only): the B tile is fetched as two boxes of BN / 2 rows starting at rows t.b_mn0 and
// t.b_mn1 (gate and up rows of a fused gate/up weight, so that one accumulator row holds both).
template <bool A_MN_ = false, bool B_MN_ = false, bool A_3D_ = false, bool B_3D_ = false, int SIDE_WARPS_ = 0,
          bool PRODUCER_HOOK_ = false, bool B_TWO_BOXES_ = false>
struct GemmTraits {
  static constexpr bool A_MN = A_MN_, B_MN = B_MN_, A_3D = A_3D_, B_3D = B_3D_;
  static constexpr int SIDE_WARPS = SIDE_WARPS_;
  static constexpr bool PRODUCER_HOOK = PRODUCER_HOOK_;
  static constexpr bool B_TWO_BOXES = B_TWO_BOXES_;
};

// An epilogue that declares `static constexpr bool CUSTOM_TILE = true` reads its accumulator itself:
//   __device__ void tile(const Params&, const TileInfo&, int row, uint32_t taddr /* this warp's lanes, column 0 */,
//                        uint8_t* epi_smem /* GemmSmem::EPI_BYTES, when launched with TOTAL_WITH_EPI */);
template <class E, class = void>
struct epi_custom_tile : std::false_type {};
template <class E>
struct epi_custom_tile<E, std::void_t<decltype(E::CUSTOM_TILE)>> : std::true_type {};

// Default schedule: grouped raster over (m, n) tiles, strided over the grid.
struct RasterSchedule {
  int num_m, num_n, total, num_kb;
  template <class P>
  __device__ __forceinline__ void init(int M, int N, int K, int BN, const P&) {
    num_m = (M + GEMM_BM - 1) / GEMM_BM;
    num_n = (N + BN - 1) / BN;
    total = num_m * num_n;
    num_kb = (K + GEMM_BK - 1) / GEMM_BK;
    bn = BN;
  }
  int bn;
  __device__ __forceinline__ bool get(int it, TileInfo& t) const {
    int i = blockIdx.x + it * gridDim.x;
    if (i >= total) return false;
    constexpr int G = 8;
    int group_size = G * num_n;
    int group = i / group_size;
    int first_m = group * G;
    int gsz = min(num_m - first_m, G);
    int r = i - group * group_size;
    t.m_blk = first_m + r % gsz;
    t.n_blk = r / gsz;
    t.a_mn0 = t.m_blk * GEMM_BM;
    t.b_mn0 = t.n_blk * bn;
    t.k0 = 0;
    t.num_kb = num_kb;
    t.batch = 0;
    return true;
  }
};

// Epilogue concept:
//   struct Epi { struct Params {...};
//     __device__ void tile_begin(const Params&, const TileInfo&, int row /*0..127*/);
//     __device__ void chunk(const Params&, const TileInfo&, int row, int col0 /*within tile*/, const float (&v)[32]);
//     __device__ void tile_end(const Params&, const TileInfo&, int row);
//     __device__ void finish(const Params&);   // after the last tile
//   };

template <int BN, int STAGES, class Epi, class Sched, class Traits = GemmTraits<>>
__device__ __forceinline__ void gemm_mainloop(const CUtensorMap* tmA, const CUtensorMap* tmB, int M, int N, int K,
                                              const typename Epi::Params& ep, uint32_t* status) {
  using SM = GemmSmem<BN, STAGES>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + STAGES * SM::STAGE_BYTES);
  uint64_t* empty_bar = full_bar + STAGES;
  uint64_t* tfull_bar = empty_bar + STAGES;   // [2]
  uint64_t* tempty_bar = tfull_bar + 2;       // [2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty_bar + 2);
  volatile uint32_t* abort_flag = tmem_slot + 1;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  constexpr uint32_t TMEM_COLS = (2 * BN <= 32) ? 32 : (2 * BN <= 64) ? 64 : (2 * BN <= 128) ? 128 : (2 * BN <= 256) ? 256 : 512;

  pdl_launch_dependents();
  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&tfull_bar[a], 1);
      mbar_init(&tempty_bar[a], 4);  // one arrive per epilogue warp
    }
    *abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(tmA);
    tma_prefetch_desc(tmB);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  pdl_wait();  // everything above touched only this CTA's own state; global memory comes next

  Sched sched;
  sched.init(M, N, K, BN, ep);

  if (warp == 0) {
    // ------------------------------ TMA producer ------------------------------
    if (lane == 0) {
      uint32_t stage = 0, phase = 0;
      TileInfo t;
      for (int it = 0; sched.get(it, t) && !*abort_flag; ++it) {
        if constexpr (Traits::PRODUCER_HOOK) {
          if (!sched.before_tile_load(t, ep, status)) {
            *abort_flag = 1;
            break;
          }
        }
        for (int kb = 0; kb < t.num_kb; ++kb) {
          if (!mbar_wait(&empty_bar[stage], phase ^ 1)) {
            atomicCAS(status, ST_OK, ST_TIMEOUT_EMPTY);
            *abort_flag = 1;
            break;
          }
          uint8_t* sa = smem + stage * SM::STAGE_BYTES;
          uint8_t* sb = sa + SM::A_BYTES;
          const int k = t.k0 + kb * GEMM_BK;
          mbar_arrive_expect_tx(&full_bar[stage], SM::STAGE_BYTES);
          if constexpr (!Traits::A_MN) {
            if constexpr (Traits::A_3D) tma_load_3d(sa, tmA, &full_bar[stage], k, t.a_mn0, t.batch);
            else tma_load_2d(sa, tmA, &full_bar[stage], k, t.a_mn0);
          } else {
#pragma unroll
            for (int i = 0; i < GEMM_BM / 64; ++i) {
              if constexpr (Traits::A_3D) tma_load_3d(sa + i * 8192, tmA, &full_bar[stage], t.a_mn0 + i * 64, k, t.batch);
              else tma_load_2d(sa + i * 8192, tmA, &full_bar[stage], t.a_mn0 + i * 64, k);
            }
          }
          if constexpr (Traits::B_TWO_BOXES) {
            tma_load_2d(sb, tmB, &full_bar[stage], k, t.b_mn0);
            tma_load_2d(sb + SM::B_BYTES / 2, tmB, &full_bar[stage], k, t.b_mn1);
          } else if constexpr (!Traits::B_MN) {
            if constexpr (Traits::B_3D) tma_load_3d(sb, tmB, &full_bar[stage], k, t.b_mn0, t.batch);
            else tma_load_2d(sb, tmB, &full_bar[stage], k, t.b_mn0);
          } else {
#pragma unroll
            for (int i = 0; i < BN / 64; ++i) {
              if constexpr (Traits::B_3D) tma_load_3d(sb + i * 8192, tmB, &full_bar[stage], t.b_mn0 + i * 64, k, t.batch);
              else tma_load_2d(sb + i * 8192, tmB, &full_bar[stage], t.b_mn0 + i * 64, k);
            }
          }
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------ MMA issuer --------------------------------
    if (lane == 0) {
      constexpr uint32_t idesc = umma_idesc_bf16_f32(GEMM_BM, BN) | (Traits::A_MN ? (1u << 15) : 0u) |
                                 (Traits::B_MN ? (1u << 16) : 0u);
      uint32_t stage = 0, phase = 0;
      uint32_t acc = 0, acc_phase = 0;
      TileInfo t;
      for (int it = 0; sched.get(it, t) && !*abort_flag; ++it) {
        if (!mbar_wait(&tempty_bar[acc], acc_phase ^ 1)) {
          atomicCAS(status, ST_OK, ST_TIMEOUT_TMEM_EMPTY);
          *abort_flag = 1;
          break;
        }
        tc_fence_after_sync();
        const uint32_t tmem_d = tmem_base + acc * BN;
        bool ok = true;
        for (int kb = 0; kb < t.num_kb; ++kb) {
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
          for (int k = 0; k < GEMM_BK / 16; ++k) {
            // K-major: 16 contraction elements = 32 bytes inside the 128-byte swizzle row.
            // MN-major: 16 contraction rows of 128 bytes = 2048 bytes.
            uint64_t ad = Traits::A_MN ? umma_desc_mnmajor_sw128(sa + k * 2048, 8192) : umma_desc_kmajor_sw128(sa + k * 32);
            uint64_t bd = Traits::B_MN ? umma_desc_mnmajor_sw128(sb + k * 2048, 8192) : umma_desc_kmajor_sw128(sb + k * 32);
            umma_bf16_ss(tmem_d, ad, bd, idesc, (kb > 0 || k > 0) ? 1u : 0u);
          }
          tc_commit(&empty_bar[stage]);  // frees this smem stage once the MMAs retire
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
        if (!ok) break;
        if (t.num_kb == 0) {
          // nothing to contract: the epilogue of this tile reads zeros it must not rely on; signal anyway
        }
        tc_commit(&tfull_bar[acc]);  // accumulator complete
        if (++acc == 2) { acc = 0; acc_phase ^= 1; }
      }
    }
  } else if (warp < 6) {
    // ------------------------------ epilogue (warps 2..5) ---------------------
    const int quad = warp & 3;  // TMEM lane quadrant this warp may access
    const int row = quad * 32 + lane;
    Epi epi;
    uint32_t acc = 0, acc_phase = 0;
    TileInfo t;
    for (int it = 0; sched.get(it, t) && !*abort_flag; ++it) {
      if (!mbar_wait(&tfull_bar[acc], acc_phase)) {
        atomicCAS(status, ST_OK, ST_TIMEOUT_TMEM_FULL);
        *abort_flag = 1;
        break;
      }
      tc_fence_after_sync();
      const uint32_t taddr = tmem_base + acc * BN + ((uint32_t)(quad * 32) << 16);
      if constexpr (epi_custom_tile<Epi>::value) {
        epi.tile(ep, t, row, taddr, smem + SM::EPI_OFFSET);
      } else {
        epi.tile_begin(ep, t, row);
#pragma unroll 1
        for (int c = 0; c < BN; c += 32) {
          uint32_t r[32];
          tmem_ld_32x32b_x32(taddr + c, r);
          tmem_ld_wait();
          float v[32];
#pragma unroll
          for (int i = 0; i < 32; ++i) v[i] = (t.num_kb > 0) ? __uint_as_float(r[i]) : 0.f;
          epi.chunk(ep, t, row, c, v);
        }
        epi.tile_end(ep, t, row);
      }
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tempty_bar[acc]);
      if (++acc == 2) { acc = 0; acc_phase ^= 1; }
    }
    epi.finish(ep);
  } else {
    // ------------------------------ side warps (6..) --------------------------
    if constexpr (Traits::SIDE_WARPS > 0) {
      Epi epi;
      epi.side(ep, sched, warp - 6, lane, status);
    }
  }

  // ------------------------------ teardown ------------------------------------
  tc_fence_before_sync();
  __syncthreads();
  if (*abort_flag && threadIdx.x == 0) {
    // let copies that were already issued land before the CTA's shared memory is released
    for (int i = 0; i < 100; ++i) __nanosleep(1000);
  }
  __syncthreads();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

// ---------------------------------------------------------------------------
// Host side: tensor-map encoding through the driver entry point (no -lcuda).
// ---------------------------------------------------------------------------
typedef CUresult (*PFN_encodeTiled)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                    const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                    CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// Diagnostics of the last failed tensor-map encode of this process: (reason << 24) | CUresult, where reason is
// 1 = no driver entry point, 2 = pointer or stride not 16-byte aligned, 3 = the driver refused the map.
inline int& last_tmap_error() {
  static int e = 0;
  return e;
}

// The driver refuses to encode a map on a host thread that has no current context yet (CUDA_ERROR_INVALID_CONTEXT;
// seen on autograd worker threads whose first CUDA call is this one): a runtime call binds the primary context.
template <class F>
inline CUresult encode_with_context(F&& call) {
  CUresult r = call();
  if (r == CUDA_ERROR_INVALID_CONTEXT || r == CUDA_ERROR_NOT_INITIALIZED) {
    (void)cudaFree(nullptr);
    r = call();
  }
  return r;
}

inline PFN_encodeTiled get_encode_tiled() {
  static PFN_encodeTiled fn = nullptr;
  if (!fn) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess)
      return nullptr;
    fn = reinterpret_cast<PFN_encodeTiled>(p);
  }
  return fn;
}

// Generic tiled map over a row-major tensor [d2][rows][cols] (d2 = 1 for 2-D): box = box_rows x box_cols with the
// 128-byte swizzle (box_cols * elem_bytes == 128). ld = elements between rows, ld2 = elements between slices.
inline int make_tmap_3d(CUtensorMap* out, const void* ptr, uint64_t d2, uint64_t rows, uint64_t cols, uint64_t ld,
                        uint64_t ld2, uint32_t box_rows, uint32_t box_cols, int elem_bytes, uint32_t box_d2 = 1) {
  PFN_encodeTiled enc = get_encode_tiled();
  if (!enc) { last_tmap_error() = 1 << 24; return -1; }
  if ((reinterpret_cast<uintptr_t>(ptr) & 15) || ((ld * elem_bytes) & 15) || ((ld2 * elem_bytes) & 15)) {
    last_tmap_error() = 2 << 24;
    return -2;
  }
  cuuint64_t gdim[3] = {cols, rows, d2};
  cuuint64_t gstr[2] = {ld * (uint64_t)elem_bytes, ld2 * (uint64_t)elem_bytes};
  cuuint32_t box[3] = {box_cols, box_rows, box_d2};
  cuuint32_t estr[3] = {1, 1, 1};
  CUtensorMapDataType dt = elem_bytes == 2 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_UINT8;
  CUresult r = encode_with_context([&] {
    return enc(out, dt, 3, const_cast<void*>(ptr), gdim, gstr, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
               CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  });
  if (r != CUDA_SUCCESS) last_tmap_error() = (3 << 24) | (int)r;
  return r == CUDA_SUCCESS ? 0 : -3;
}

// Row-major [rows, cols] matrix of 2-byte (or 1-byte) elements with leading dimension ld (elements);
// box = box_rows x box_cols, 128-byte swizzle (box_cols * elem_bytes must be 128).
inline int make_tmap_2d(CUtensorMap* out, const void* ptr, uint64_t rows, uint64_t cols, uint64_t ld,
                        uint32_t box_rows, uint32_t box_cols, int elem_bytes) {
  PFN_encodeTiled enc = get_encode_tiled();
  if (!enc) { last_tmap_error() = 1 << 24; return -1; }
  if ((reinterpret_cast<uintptr_t>(ptr) & 15) || ((ld * elem_bytes) & 15)) {
    last_tmap_error() = 2 << 24;
    return -2;
  }
  cuuint64_t gdim[2] = {cols, rows};
  cuuint64_t gstr[1] = {ld * (uint64_t)elem_bytes};
  cuuint32_t box[2] = {box_cols, box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUtensorMapDataType dt = elem_bytes == 2 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_UINT8;
  CUresult r = encode_with_context([&] {
    return enc(out, dt, 2, const_cast<void*>(ptr), gdim, gstr, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
               CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  });
  if (r != CUDA_SUCCESS) last_tmap_error() = (3 << 24) | (int)r;
  return r == CUDA_SUCCESS ? 0 : -3;
}

}  // namespace b200
