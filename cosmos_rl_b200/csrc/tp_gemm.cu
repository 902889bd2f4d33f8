// Row-parallel linear layer fused with its tensor-parallel reduction, in ONE kernel over NVLink peer memory:
//
//     out = sum over TP ranks r of  A_r[M, K_r] * W_r[N, K_r]^T            (all-reduce,    mode 0)
//     out[rows owned by this rank] = the same sum                          (reduce-scatter, mode 1)
//
// Each rank runs the persistent tcgen05 pipeline on its K-slice. The epilogue warps convert an accumulator
// tile to bf16, transpose it through shared memory so that every store instruction writes whole 256-byte row
// segments, and PUSH it with plain peer stores into slot[src rank] of the staging area of every rank that
// needs the tile, then bump that rank's per-tile arrival counter (red.release.sys). Four additional warps of
// the same CTA run concurrently with the pipeline: they wait (bounded) for a tile's counter to reach
// 4 epilogue warps x tp ranks, sum the tp slots from LOCAL memory in fp32 and write the bf16 result. The
// NVLink transfer of tile i therefore overlaps the MMAs of tile i+1, and no separate collective is launched.
// Replaces o_proj / down_proj + NCCL all-reduce (or reduce-scatter under sequence parallelism) of the
// reference's TP plan (cosmos_rl/policy/model/gpt/parallelize.py:233-340) and of its rollout engine.
//
// Staging and counters are double-buffered by the parity of a call counter kept in device memory (so a CUDA
// graph can replay the launch): a peer can run at most one call ahead of this rank, because finishing call
// k+1 needs this rank's pushes of call k+1, which are issued after this rank's call k has ended.
#include "gemm_core.cuh"
#include "api.h"

namespace b200 {

constexpr int TP_MAX = 8;
constexpr int TP_SIDE_WARPS = 4;
constexpr int TP_THREADS = GEMM_THREADS + 32 * TP_SIDE_WARPS;
constexpr int TP_ROW_BYTES = 256;                            // 128 bf16 columns; 16-byte pieces XOR-swizzled by row
constexpr int TP_XPOSE_BYTES = 128 * TP_ROW_BYTES;           // one 32-row slab per epilogue warp

struct TpParams {
    __nv_bfloat16* stage[TP_MAX];   // staging base of every rank (own included), peer-mapped
    uint32_t* flags[TP_MAX];        // arrival counters of every rank: [2][max_tiles]
    uint32_t* seq;                  // local call counter
    __nv_bfloat16* out;
    const __nv_bfloat16* residual;  // optional, added to the reduced result
    long long ldo, ldr;
    long long slot_elems;           // elements per (set, source rank) slot
    unsigned long long wait_ns;     // limit of one wait for a tile's partials
    int M, N, tp, rank, mode, max_tiles, rows_per_rank, num_n;
};

// BN = 256 (4 stages) is the wide tile for large M; BN = 128 (5 stages) gives more tiles for small M.
template <int BN, int STAGES>
struct TpEpilogue {
  using Params = TpParams;
  int set = -1;

  static __device__ __forceinline__ uint8_t* xpose_base() {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    return smem + STAGES * GemmSmem<BN, STAGES>::STAGE_BYTES + GemmSmem<BN, STAGES>::BAR_BYTES;
  }
  static __device__ __forceinline__ int owner_of(const Params& p, int m_blk) {
    return (m_blk * GEMM_BM) / p.rows_per_rank;
  }

  __device__ __forceinline__ void tile_begin(const Params& p, const TileInfo&, int) {
    if (set < 0) set = (int)(*reinterpret_cast<volatile uint32_t*>(p.seq) & 1u);
  }

  // 32 fp32 columns of this thread's row -> bf16 in the transposition slab; a full 128-column half is pushed
  __device__ __forceinline__ void chunk(const Params& p, const TileInfo& t, int row, int col0, const float (&v)[32]) {
    uint8_t* dst = xpose_base() + (size_t)row * TP_ROW_BYTES;
    const int piece0 = (col0 & 127) >> 3;
#pragma unroll
    for (int g = 0; g < 4; ++g) {
      uint4 o;
      o.x = pack_bf16x2(v[8 * g + 0], v[8 * g + 1]);
      o.y = pack_bf16x2(v[8 * g + 2], v[8 * g + 3]);
      o.z = pack_bf16x2(v[8 * g + 4], v[8 * g + 5]);
      o.w = pack_bf16x2(v[8 * g + 6], v[8 * g + 7]);
      *reinterpret_cast<uint4*>(dst + (((piece0 + g) ^ (row & 15)) << 4)) = o;
    }
    if ((col0 & 127) == 96) push_half(p, t, row, col0 >> 7);
  }

  __device__ __forceinline__ void push_half(const Params& p, const TileInfo& t, int row, int half) {
    const int lane = threadIdx.x & 31;
    const int slab0 = row - lane;                 // first tile row of this warp's 32-row slab
    __syncwarp();
    const int first = p.mode == 0 ? 0 : owner_of(p, t.m_blk);
    const int last = p.mode == 0 ? p.tp : first + 1;
    const long long row_base = p.mode == 0 ? 0 : (long long)first * p.rows_per_rank;
    const int piece = lane & 15;
    const int col = t.n_blk * BN + half * 128 + piece * 8;
#pragma unroll 4
    for (int rr = 0; rr < 32; rr += 2) {
      const int rt = slab0 + rr + (lane >> 4);
      const long long grow = (long long)t.m_blk * GEMM_BM + rt;
      if (grow < p.M && col < p.N) {
        const uint4 val = *reinterpret_cast<const uint4*>(xpose_base() + (size_t)rt * TP_ROW_BYTES +
                                                          ((piece ^ (rt & 15)) << 4));
        const long long off = ((long long)set * p.tp + p.rank) * p.slot_elems + (grow - row_base) * p.N + col;
        for (int d = first; d < last; ++d) *reinterpret_cast<uint4*>(p.stage[d] + off) = val;
      }
    }
    __syncwarp();                                 // slab is free for the next half
  }

  __device__ __forceinline__ void tile_end(const Params& p, const TileInfo& t, int) {
    const int lane = threadIdx.x & 31;
    const int first = p.mode == 0 ? 0 : owner_of(p, t.m_blk);
    const int last = p.mode == 0 ? p.tp : first + 1;
    __threadfence_system();
    __syncwarp();
    if (lane == 0) {
      const int tile = t.m_blk * p.num_n + t.n_blk;
      for (int d = first; d < last; ++d) {
        uint32_t* f = p.flags[d] + (size_t)set * p.max_tiles + tile;
        asm volatile("red.release.sys.global.add.u32 [%0], 1;" ::"l"(f) : "memory");
      }
    }
  }

  __device__ __forceinline__ void finish(const Params&) {}

  // reducer warps: run beside the pipeline, one tile at a time in the pipeline's own tile order
  template <class Sched>
  __device__ __forceinline__ void side(const Params& p, const Sched& sched, int w, int lane, uint32_t* status) {
    __shared__ volatile int side_ok;
    const int st = (int)(*reinterpret_cast<volatile uint32_t*>(p.seq) & 1u);
    const uint32_t target = 4u * (uint32_t)p.tp;
    // after an earlier failure (recorded in the status word) do not sit out the full limit again
    const unsigned long long limit =
        (*reinterpret_cast<volatile uint32_t*>(status) != ST_OK) ? 1000000ull : p.wait_ns;
    const long long row_base = p.mode == 0 ? 0 : (long long)p.rank * p.rows_per_rank;
    const int piece = lane & 15;
    TileInfo t;
    for (int it = 0; sched.get(it, t); ++it) {
      if (p.mode == 1 && owner_of(p, t.m_blk) != p.rank) continue;
      uint32_t* flag = p.flags[p.rank] + (size_t)st * p.max_tiles + t.m_blk * p.num_n + t.n_blk;
      if (w == 0 && lane == 0) {
        const unsigned long long t0 = globaltimer_ns();
        int ok = 1;
        while (true) {
          uint32_t v;
          asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(flag) : "memory");
          if (v >= target) break;
          if (globaltimer_ns() - t0 > limit) {
            atomicCAS(status, ST_OK, ST_TIMEOUT_PEER_FLAG);
            ok = 0;
            break;
          }
          __nanosleep(100);
        }
        side_ok = ok;
      }
      asm volatile("bar.sync 1, %0;" ::"n"(32 * TP_SIDE_WARPS) : "memory");
      if (!side_ok) break;
#pragma unroll 1
      for (int it2 = 0; it2 < 16 * (BN / 128); ++it2) {
        const int rr = (it2 & 15) * 2;
        const int col = t.n_blk * BN + (it2 >> 4) * 128 + piece * 8;
        const long long grow = (long long)t.m_blk * GEMM_BM + w * 32 + rr + (lane >> 4);
        if (grow >= p.M || col >= p.N) continue;
        float acc[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[j] = 0.f;
        const __nv_bfloat16* src = p.stage[p.rank] + (long long)st * p.tp * p.slot_elems + (grow - row_base) * p.N + col;
        for (int s = 0; s < p.tp; ++s) {
          const uint4 v = __ldcg(reinterpret_cast<const uint4*>(src + (long long)s * p.slot_elems));
          const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const float2 f = __bfloat1622float2(h[j]);
            acc[2 * j] += f.x;
            acc[2 * j + 1] += f.y;
          }
        }
        const long long orow = grow - row_base;
        if (p.residual != nullptr) {
          const uint4 v = *reinterpret_cast<const uint4*>(p.residual + orow * p.ldr + col);
          const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const float2 f = __bfloat1622float2(h[j]);
            acc[2 * j] += f.x;
            acc[2 * j + 1] += f.y;
          }
        }
        uint4 o;
        o.x = pack_bf16x2(acc[0], acc[1]);
        o.y = pack_bf16x2(acc[2], acc[3]);
        o.z = pack_bf16x2(acc[4], acc[5]);
        o.w = pack_bf16x2(acc[6], acc[7]);
        *reinterpret_cast<uint4*>(p.out + orow * p.ldo + col) = o;
      }
      asm volatile("bar.sync 1, %0;" ::"n"(32 * TP_SIDE_WARPS) : "memory");
      // consumed: re-arm the counter for the next use of this set (two calls from now)
      if (w == 0 && lane == 0) *reinterpret_cast<volatile uint32_t*>(flag) = 0u;
    }
  }
};

template <int BN, int STAGES>
__global__ void __launch_bounds__(TP_THREADS, 1)
tp_gemm_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, int M, int N, int K,
               TpParams ep, uint32_t* exit_count, uint32_t* status) {
  gemm_mainloop<BN, STAGES, TpEpilogue<BN, STAGES>, RasterSchedule,
                GemmTraits<false, false, false, false, TP_SIDE_WARPS>>(&tmA, &tmB, M, N, K, ep, status);
  // every role of every CTA has read the call counter by now; the last CTA to leave advances it
  if (threadIdx.x == 0) {
    __threadfence();
    if (atomicAdd(exit_count, 1u) == gridDim.x - 1) {
      *reinterpret_cast<volatile uint32_t*>(exit_count) = 0u;
      __threadfence();
      atomicAdd(ep.seq, 1u);
    }
  }
}

template <int BN, int STAGES>
static int launch_tp(const void* A, const void* W, int M, int N, int K, long long lda, long long ldw, TpParams ep,
                     uint32_t* ctrl, uint32_t* status, int num_sms, cudaStream_t stream) {
  CUtensorMap tmA, tmB;
  if (make_tmap_2d(&tmA, A, M, K, lda, GEMM_BM, GEMM_BK, 2)) return B200_ERR_TENSORMAP;
  if (make_tmap_2d(&tmB, W, N, K, ldw, BN, GEMM_BK, 2)) return B200_ERR_TENSORMAP;
  constexpr int SMEM = GemmSmem<BN, STAGES>::TOTAL + TP_XPOSE_BYTES;
  static_assert(SMEM <= 232448, "shared memory budget");
  auto kern = tp_gemm_kernel<BN, STAGES>;
  static bool attr_set = false;
  if (!attr_set) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM) != cudaSuccess)
      return B200_ERR_LAUNCH;
    attr_set = true;
  }
  const int num_m = (M + GEMM_BM - 1) / GEMM_BM;
  ep.num_n = (N + BN - 1) / BN;
  const int tiles = num_m * ep.num_n;
  if (tiles > ep.max_tiles) return B200_ERR_ARG;
  const int grid = tiles < num_sms ? tiles : num_sms;
  kern<<<grid, TP_THREADS, SMEM, stream>>>(tmA, tmB, M, N, K, ep, ctrl + 1, status);
  return cudaGetLastError() == cudaSuccess ? 0 : B200_ERR_LAUNCH;
}

}  // namespace b200

// stage_ptrs / flag_ptrs: host arrays of `tp` device pointers (index = TP rank; entry `rank` is this rank's own
// memory, the others are peer mappings). ctrl points at two local uint32 {call counter, exit counter}.
// mode 0: all-reduce, out is [M, N]. mode 1: reduce-scatter over rows, out is [M / tp, N] and M / tp must be a
// multiple of 128. residual (optional) has out's shape. slot_elems is the capacity of one staging slot.
extern "C" int b200_tp_gemm(const void* A, const void* W, void* out, const void* residual, int M, int N, int K,
                            long long lda, long long ldw, long long ldo, long long ldr, void* const* stage_ptrs,
                            void* const* flag_ptrs, uint32_t* ctrl, int tp, int rank, int mode, long long slot_elems,
                            int max_tiles, unsigned long long wait_ns, uint32_t* status, int num_sms,
                            cudaStream_t stream) {
  using namespace b200;
  if (M <= 0 || N <= 0 || K <= 0 || tp < 1 || tp > TP_MAX || rank < 0 || rank >= tp) return B200_ERR_ARG;
  if ((lda & 7) || (ldw & 7) || (N & 7) || (ldo & 7) || (ldr & 7)) return B200_ERR_ARG;
  int rows_per_rank = M;
  if (mode == 1) {
    if (M % tp) return B200_ERR_ARG;
    rows_per_rank = M / tp;
    if (rows_per_rank % GEMM_BM) return B200_ERR_ARG;
  }
  if ((long long)rows_per_rank * N > slot_elems || (slot_elems & 7)) return B200_ERR_ARG;
  TpParams ep{};
  for (int r = 0; r < tp; ++r) {
    ep.stage[r] = reinterpret_cast<__nv_bfloat16*>(stage_ptrs[r]);
    ep.flags[r] = reinterpret_cast<uint32_t*>(flag_ptrs[r]);
  }
  ep.seq = ctrl;
  ep.out = reinterpret_cast<__nv_bfloat16*>(out);
  ep.residual = reinterpret_cast<const __nv_bfloat16*>(residual);
  ep.ldo = ldo;
  ep.ldr = ldr;
  ep.slot_elems = slot_elems;
  ep.wait_ns = wait_ns ? wait_ns : WAIT_LIMIT_NS;
  ep.M = M; ep.N = N; ep.tp = tp; ep.rank = rank; ep.mode = mode; ep.max_tiles = max_tiles;
  ep.rows_per_rank = rows_per_rank;
  // wide tiles once there are enough of them to fill the machine; narrow tiles otherwise
  const long long wide_tiles = (long long)((M + GEMM_BM - 1) / GEMM_BM) * ((N + 255) / 256);
  if (wide_tiles >= num_sms)
    return launch_tp<256, 4>(A, W, M, N, K, lda, ldw, ep, ctrl, status, num_sms, stream);
  return launch_tp<128, 5>(A, W, M, N, K, lda, ldw, ep, ctrl, status, num_sms, stream);
}
