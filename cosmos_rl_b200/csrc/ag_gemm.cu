// Sequence-parallel column-parallel linear layer: tensor-parallel all-gather of the activation rows fused into the
// GEMM that consumes them, in ONE kernel over NVLink peer memory:
//
//     y[M, N_local] = gather_r(x_r)[M, K] * W[N_local, K]^T,        x_r [M / tp, K] = the rows rank r owns
//
// Four side warps of every CTA PUSH this rank's rows, 128-row block by 128-row block, into the gathered-activation
// buffer of every rank (plain 16-byte peer stores, a warp writes 512 contiguous bytes of one row) and bump the
// destination's arrival counter of that row block (red.release.sys). The TMA producer of the tcgen05 pipeline
// waits (bounded) for a row block's counter before it loads A tiles of that block from LOCAL memory; tiles are
// visited starting with the rank's own rows, then the next rank's, so the math starts at once and the transfers
// of later blocks hide behind it. Replaces all-gather + nn.Linear of the reference's sequence-parallel TP plan
// (cosmos_rl/policy/model/gpt/parallelize.py:233-340, async-TP :329-334).
//
// The gathered buffer and the counters are double-buffered by the parity of a call counter in device memory (a peer
// can run at most one call ahead: finishing call k+1 needs this rank's rows of call k+1); the last CTA to leave
// re-arms the counters of the set it used and advances the call counter.
#include "gemm_core.cuh"
#include "api.h"

namespace b200 {

constexpr int AG_MAX = 8;
constexpr int AG_SIDE_WARPS = 4;
constexpr int AG_THREADS = GEMM_THREADS + 32 * AG_SIDE_WARPS;
constexpr int AG_SLAB = 1024;    // columns (elements) per push unit: 128 rows x 2 KB

struct AgParams {
  __nv_bfloat16* gathered[AG_MAX];   // gathered-activation buffer of every rank: [2 sets][rows_cap * K]
  uint32_t* flags[AG_MAX];           // arrival counters of every rank: [2 sets][max_blocks]
  uint32_t* seq;                     // local call counter
  const __nv_bfloat16* x;            // this rank's rows [rows_per_rank, K]
  long long ldx, set_elems;
  unsigned long long wait_ns;
  void* C;
  long long ldc;
  int M, N, K, tp, rank, rows_per_rank, blocks_per_rank, max_blocks, n_slabs;
};

struct AgEpilogue {
  using Params = AgParams;
  __device__ __forceinline__ void tile_begin(const Params&, const TileInfo&, int) {}
  __device__ __forceinline__ void tile_end(const Params&, const TileInfo&, int) {}
  __device__ __forceinline__ void finish(const Params&) {}
  __device__ __forceinline__ void chunk(const Params& p, const TileInfo& t, int row, int col0, const float (&v)[32]) {
    const long long r = (long long)t.m_blk * GEMM_BM + row;
    const int c = t.n_blk * 256 + col0;
    if (r >= p.M || c >= p.N) return;
    __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(p.C) + r * p.ldc + c;
    if (c + 32 <= p.N) {
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

  // side warps: push this rank's rows to every rank, one (row block, column slab) unit at a time
  template <class Sched>
  __device__ __forceinline__ void side(const Params& p, const Sched&, int w, int lane, uint32_t*) {
    const int set = (int)(*reinterpret_cast<volatile uint32_t*>(p.seq) & 1u);
    const int units = p.blocks_per_rank * p.n_slabs;
    for (int u = blockIdx.x; u < units; u += gridDim.x) {
      const int lb = u / p.n_slabs, slab = u % p.n_slabs;       // local row block, column slab
      const int c_lo = slab * AG_SLAB, c_hi = min(p.K, c_lo + AG_SLAB);
      const int vec_per_row = (c_hi - c_lo) >> 3;
      const int r_lo = lb * GEMM_BM + w * 32, r_hi = min(p.rows_per_rank, r_lo + 32);
      // destinations in ring order starting with this rank, so the local copy (needed first) lands first
      for (int dd = 0; dd < p.tp; ++dd) {
        const int d = (p.rank + dd) % p.tp;
        __nv_bfloat16* base = p.gathered[d] + (long long)set * p.set_elems +
                              ((long long)p.rank * p.rows_per_rank) * p.K;
        for (int r = r_lo; r < r_hi; ++r) {
          const uint4* src = reinterpret_cast<const uint4*>(p.x + (long long)r * p.ldx + c_lo);
          uint4* dst = reinterpret_cast<uint4*>(base + (long long)r * p.K + c_lo);
#pragma unroll 4
          for (int v = lane; v < vec_per_row; v += 32) dst[v] = src[v];
        }
        __threadfence_system();
        fence_proxy_async_all();
        __syncwarp();
        if (lane == 0) {
          uint32_t* f = p.flags[d] + (size_t)set * p.max_blocks + p.rank * p.blocks_per_rank + lb;
          asm volatile("red.release.sys.global.add.u32 [%0], 1;" ::"l"(f) : "memory");
        }
      }
    }
  }
};

// Tiles in an order that starts with the row blocks this rank owns (their data is local), then the next rank's ...
struct AgSchedule {
  int num_m, num_n, total, num_kb, rot;
  const AgParams* prm;
  __device__ __forceinline__ void init(int M, int N, int K, int BN, const AgParams& p) {
    num_m = (M + GEMM_BM - 1) / GEMM_BM;
    num_n = (N + BN - 1) / BN;
    total = num_m * num_n;
    num_kb = (K + GEMM_BK - 1) / GEMM_BK;
    rot = p.rank * p.blocks_per_rank;
    prm = &p;
  }
  __device__ __forceinline__ bool get(int it, TileInfo& t) const {
    const int i = blockIdx.x + it * gridDim.x;
    if (i >= total) return false;
    constexpr int G = 8;
    const int group_size = G * num_n;
    const int group = i / group_size, first_m = group * G;
    const int gsz = min(num_m - first_m, G);
    const int r = i - group * group_size;
    t.m_blk = (first_m + r % gsz + rot) % num_m;
    t.n_blk = r / gsz;
    t.a_mn0 = t.m_blk * GEMM_BM;
    t.b_mn0 = t.n_blk * 256;
    t.k0 = 0;
    t.num_kb = num_kb;
    t.batch = 0;
    return true;
  }
  // wait until every slab of the row block has arrived from its owner (4 side warps per slab)
  __device__ __forceinline__ bool before_tile_load(const TileInfo& t, const AgParams& p, uint32_t* status) const {
    const int set = (int)(*reinterpret_cast<volatile uint32_t*>(p.seq) & 1u);
    const uint32_t* f = p.flags[p.rank] + (size_t)set * p.max_blocks + t.m_blk;
    const uint32_t target = 4u * (uint32_t)p.n_slabs;
    const unsigned long long limit = (*reinterpret_cast<volatile uint32_t*>(status) != ST_OK) ? 1000000ull : p.wait_ns;
    const unsigned long long t0 = globaltimer_ns();
    while (true) {
      uint32_t v;
      asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(f) : "memory");
      if (v >= target) break;
      if (globaltimer_ns() - t0 > limit) {
        atomicCAS(status, ST_OK, ST_TIMEOUT_PEER_FLAG);
        return false;
      }
      __nanosleep(100);
    }
    fence_proxy_async_all();     // the rows were written through the generic proxy; TMA reads them next
    return true;
  }
};

__global__ void __launch_bounds__(AG_THREADS, 1)
ag_gemm_kernel(const __grid_constant__ CUtensorMap tmA0, const __grid_constant__ CUtensorMap tmA1,
               const __grid_constant__ CUtensorMap tmB, AgParams ep, uint32_t* exit_count, uint32_t* status) {
  const uint32_t set = *reinterpret_cast<volatile uint32_t*>(ep.seq) & 1u;
  gemm_mainloop<256, 4, AgEpilogue, AgSchedule, GemmTraits<false, false, false, false, AG_SIDE_WARPS, true>>(
      set ? &tmA1 : &tmA0, &tmB, ep.M, ep.N, ep.K, ep, status);
  // every role of every CTA has read the call counter by now; the last CTA re-arms this set and advances it
  if (threadIdx.x == 0) {
    __threadfence();
    if (atomicAdd(exit_count, 1u) == gridDim.x - 1) {
      uint32_t* f = ep.flags[ep.rank] + (size_t)set * ep.max_blocks;
      for (int i = 0; i < ep.max_blocks; ++i) reinterpret_cast<volatile uint32_t*>(f)[i] = 0u;
      *reinterpret_cast<volatile uint32_t*>(exit_count) = 0u;
      __threadfence();
      atomicAdd(ep.seq, 1u);
    }
  }
}

}  // namespace b200

// x: this rank's rows [M / tp, K] (row stride ldx); W [N, K]; out [M, N] bf16 (row stride ldc).
// gathered_ptrs / flag_ptrs: host arrays of tp device pointers (entry `rank` = own memory, others peer mappings).
// set_elems: elements of one gathered set (>= M * K). ctrl: two local uint32 {call counter, exit counter}.
extern "C" int b200_ag_gemm(const void* x, const void* W, void* out, int M, int N, int K, long long ldx, long long ldw,
                            long long ldc, void* const* gathered_ptrs, void* const* flag_ptrs, uint32_t* ctrl, int tp,
                            int rank, long long set_elems, int max_blocks, unsigned long long wait_ns,
                            uint32_t* status, int num_sms, cudaStream_t stream) {
  using namespace b200;
  if (M <= 0 || N <= 0 || K <= 0 || tp < 1 || tp > AG_MAX || rank < 0 || rank >= tp) return B200_ERR_ARG;
  if ((ldx & 7) || (ldw & 7) || (ldc & 7) || (K & 7) || (M % tp)) return B200_ERR_ARG;
  const int rows_per_rank = M / tp;
  if (rows_per_rank % GEMM_BM) return B200_ERR_ARG;
  const int num_m = M / GEMM_BM;
  if (num_m > max_blocks || (long long)M * K > set_elems) return B200_ERR_ARG;
  AgParams ep{};
  for (int r = 0; r < tp; ++r) {
    ep.gathered[r] = reinterpret_cast<__nv_bfloat16*>(gathered_ptrs[r]);
    ep.flags[r] = reinterpret_cast<uint32_t*>(flag_ptrs[r]);
  }
  ep.seq = ctrl;
  ep.x = reinterpret_cast<const __nv_bfloat16*>(x);
  ep.ldx = ldx;
  ep.set_elems = set_elems;
  ep.wait_ns = wait_ns ? wait_ns : WAIT_LIMIT_NS;
  ep.C = out;
  ep.ldc = ldc;
  ep.M = M; ep.N = N; ep.K = K; ep.tp = tp; ep.rank = rank;
  ep.rows_per_rank = rows_per_rank;
  ep.blocks_per_rank = rows_per_rank / GEMM_BM;
  ep.max_blocks = max_blocks;
  ep.n_slabs = (K + AG_SLAB - 1) / AG_SLAB;
  CUtensorMap tmA0, tmA1, tmB;
  const __nv_bfloat16* g = ep.gathered[rank];
  if (make_tmap_2d(&tmA0, g, M, K, K, GEMM_BM, GEMM_BK, 2)) return B200_ERR_TENSORMAP;
  if (make_tmap_2d(&tmA1, g + set_elems, M, K, K, GEMM_BM, GEMM_BK, 2)) return B200_ERR_TENSORMAP;
  if (make_tmap_2d(&tmB, W, N, K, ldw, 256, GEMM_BK, 2)) return B200_ERR_TENSORMAP;
  constexpr int SMEM = GemmSmem<256, 4>::TOTAL;
  static bool attr_set = false;
  if (!attr_set) {
    if (cudaFuncSetAttribute(ag_gemm_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM) != cudaSuccess)
      return B200_ERR_LAUNCH;
    attr_set = true;
  }
  // every CTA must be resident (the producers wait for rows pushed by the side warps of other CTAs)
  const int tiles = num_m * ((N + 255) / 256);
  const int grid = tiles < num_sms ? tiles : num_sms;
  ag_gemm_kernel<<<grid, AG_THREADS, SMEM, stream>>>(tmA0, tmA1, tmB, ep, ctrl + 1, status);
  return cudaGetLastError() == cudaSuccess ? 0 : B200_ERR_LAUNCH;
}
