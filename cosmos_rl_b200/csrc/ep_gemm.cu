// Expert-parallel MoE forward: token DISPATCH fused into the first grouped expert GEMM, and the COMBINE exchange,
// over NVLink peer memory (inference / rollout path; training uses the separate exchange + grouped GEMMs).
//
//   1. ep_layout_kernel: from the all-gathered per-(rank, expert) token counts every rank derives, on the device,
//      where its rows land in each owner's receive buffer (expert-sorted, every expert block padded to 128 rows), the
//      tile -> expert map of its own buffer and how many valid rows each 128-row block will receive.
//   2. ep_dispatch_gemm_kernel: ONE kernel. Four side warps per CTA push this rank's token rows (sorted by expert)
//      into the owners' receive buffers with 16-byte peer stores and bump the arrival counter of the 128-row block
//      they land in (red.release.sys). The tcgen05 grouped-GEMM pipeline of the same kernel computes
//      Y[block] = X_recv[block] . W_gate_up[expert]^T; its TMA producer waits (bounded) until a block's counter has
//      reached the block's valid-row count before loading it, so expert blocks are multiplied as they arrive.
//   3. ep_combine_push_kernel: rows of the down-projection output go back to the rank that sent the token, into
//      the slot of that (token, k) copy, followed by an arrival count the source waits for.
// Replaces DeepEP dispatch/combine + grouped_gemm of the reference (cosmos_rl/policy/kernel/megatron_moe/fused_a2a.py:84-230,
// token_dispatcher.py:808-1201, moe/moe.py:420-443).
#include "gemm_core.cuh"
#include "api.h"

namespace b200 {

constexpr int EPG_MAX = 8;
constexpr int EPG_SIDE_WARPS = 4;
constexpr int EPG_THREADS = GEMM_THREADS + 32 * EPG_SIDE_WARPS;

// ------------------------------------------------------------------------------------------------ layout
// counts[s * E + e]: rows rank s sends to global expert e. One block of 256 threads.
__global__ void ep_layout_kernel(const int* __restrict__ counts, int ep, int E, int rank, int max_tiles,
                                 int* __restrict__ send_off,      // [E + 1] prefix of this rank's counts
                                 int* __restrict__ dst_base,      // [E] first row of this rank's rows in the owner's buffer
                                 int* __restrict__ ret_base,      // [ep * E] first row in rank s's return buffer of its expert-e copies
                                 int* __restrict__ block_start,   // [El + 1] padded start row of each local expert block
                                 int* __restrict__ tile_expert,   // [max_tiles]
                                 int* __restrict__ block_target,  // [max_tiles] valid rows of each 128-row tile
                                 int* __restrict__ n_tiles) {     // [1]
  const int El = E / ep;
  if (threadIdx.x == 0) {
    int acc = 0;
    for (int e = 0; e < E; ++e) { send_off[e] = acc; acc += counts[rank * E + e]; }
    send_off[E] = acc;
    // return buffers: rank s receives its copies back in its own send order
    for (int s = 0; s < ep; ++s) {
      int a = 0;
      for (int e = 0; e < E; ++e) { ret_base[s * E + e] = a; a += counts[s * E + e]; }
    }
    // every owner's expert-sorted, 128-padded layout
    for (int d = 0; d < ep; ++d) {
      int start = 0;
      for (int j = 0; j < El; ++j) {
        const int e = d * El + j;
        int rows = 0, before_me = 0;
        for (int s = 0; s < ep; ++s) {
          if (s < rank) before_me += counts[s * E + e];
          rows += counts[s * E + e];
        }
        dst_base[e] = start + before_me;
        if (d == rank) {
          block_start[j] = start;
          const int nt = (rows + GEMM_BM - 1) / GEMM_BM;
          for (int t = 0; t < nt; ++t) {
            const int ti = start / GEMM_BM + t;
            if (ti < max_tiles) {
              tile_expert[ti] = j;
              block_target[ti] = min(GEMM_BM, rows - t * GEMM_BM);
            }
          }
        }
        start += (rows + GEMM_BM - 1) / GEMM_BM * GEMM_BM;
      }
      if (d == rank) {
        block_start[El] = start;
        n_tiles[0] = min(start / GEMM_BM, max_tiles);
      }
    }
  }
}

// ------------------------------------------------------------------------------------------------ fused kernel
struct EpgParams {
  const __nv_bfloat16* x;        // [n_rows, H] this rank's token copies sorted by global expert
  long long ldx;
  const int* send_off;           // [E + 1]
  const int* dst_base;           // [E]
  __nv_bfloat16* recv[EPG_MAX];  // receive buffer (set in use) of every rank
  uint32_t* flags[EPG_MAX];      // per-128-row-block arrival counters (set in use) of every rank
  const int* tile_expert;
  const int* block_target;
  const int* n_tiles;
  void* C;
  long long ldc;
  unsigned long long wait_ns;
  int E, El, ep, rank, H, N, rows_limit;
};

struct EpgEpilogue {
  using Params = EpgParams;
  __device__ __forceinline__ void tile_begin(const Params&, const TileInfo&, int) {}
  __device__ __forceinline__ void tile_end(const Params&, const TileInfo&, int) {}
  __device__ __forceinline__ void finish(const Params&) {}
  __device__ __forceinline__ void chunk(const Params& p, const TileInfo& t, int row, int col0, const float (&v)[32]) {
    const long long r = (long long)t.m_blk * GEMM_BM + row;
    const int c = t.n_blk * 256 + col0;
    if (r >= p.rows_limit || c >= p.N) return;
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

  // side warps: a warp pushes batches of EPG_BATCH token rows, then one system fence, then the arrival counts.
  // Rows are visited starting with those owed to the NEXT rank (they have the longest way), this rank's own last.
  template <class Sched>
  __device__ __forceinline__ void side(const Params& p, const Sched&, int w, int lane, uint32_t*) {
    constexpr int EPG_BATCH = 4;
    const int n_rows = p.send_off[p.E];
    const int vec = p.H >> 3;
    const int rot = p.send_off[((p.rank + 1) % p.ep) * p.El];
    const int n_warps = gridDim.x * EPG_SIDE_WARPS, me = blockIdx.x * EPG_SIDE_WARPS + w;
    for (int base = me * EPG_BATCH; base < n_rows; base += n_warps * EPG_BATCH) {
      uint32_t* fl[EPG_BATCH];
#pragma unroll
      for (int q = 0; q < EPG_BATCH; ++q) {
        fl[q] = nullptr;
        const int i = base + q;
        if (i >= n_rows) continue;
        int r = i + rot;
        if (r >= n_rows) r -= n_rows;
        int lo = 0, hi = p.E - 1;                     // last expert whose first row <= r
        while (lo < hi) {
          const int mid = (lo + hi + 1) >> 1;
          if (p.send_off[mid] <= r) lo = mid; else hi = mid - 1;
        }
        const int e = lo, d = e / p.El;
        const long long drow = (long long)p.dst_base[e] + (r - p.send_off[e]);
        const uint4* src = reinterpret_cast<const uint4*>(p.x + (long long)r * p.ldx);
        uint4* dst = reinterpret_cast<uint4*>(p.recv[d] + drow * p.H);
        for (int v = lane; v < vec; v += 32) dst[v] = src[v];
        fl[q] = p.flags[d] + drow / GEMM_BM;
      }
      __threadfence_system();
      fence_proxy_async_all();
      __syncwarp();
      if (lane == 0) {
#pragma unroll
        for (int q = 0; q < EPG_BATCH; ++q)
          if (fl[q]) asm volatile("red.release.sys.global.add.u32 [%0], 1;" ::"l"(fl[q]) : "memory");
      }
    }
  }
};

struct EpgSchedule {
  int num_n, total, num_kb;
  const int* tile_expert;
  __device__ __forceinline__ void init(int, int N, int K, int BN, const EpgParams& p) {
    num_n = (N + BN - 1) / BN;
    total = p.n_tiles[0] * num_n;
    num_kb = (K + GEMM_BK - 1) / GEMM_BK;
    tile_expert = p.tile_expert;
  }
  __device__ __forceinline__ bool get(int it, TileInfo& t) const {
    const int i = blockIdx.x + it * gridDim.x;
    if (i >= total) return false;
    t.m_blk = i / num_n;
    t.n_blk = i - t.m_blk * num_n;
    t.a_mn0 = t.m_blk * GEMM_BM;
    t.b_mn0 = t.n_blk * 256;
    t.k0 = 0;
    t.num_kb = num_kb;
    t.batch = tile_expert[t.m_blk];
    return true;
  }
  __device__ __forceinline__ bool before_tile_load(const TileInfo& t, const EpgParams& p, uint32_t* status) const {
    const uint32_t* f = p.flags[p.rank] + t.m_blk;
    const uint32_t target = (uint32_t)p.block_target[t.m_blk];
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
    fence_proxy_async_all();
    return true;
  }
};

__global__ void __launch_bounds__(EPG_THREADS, 1)
ep_dispatch_gemm_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, int M, int N,
                        int K, EpgParams ep, uint32_t* status) {
  gemm_mainloop<256, 4, EpgEpilogue, EpgSchedule, GemmTraits<false, false, false, true, EPG_SIDE_WARPS, true>>(
      &tmA, &tmB, M, N, K, ep, status);
}

// ------------------------------------------------------------------------------------------------ combine
struct EpcParams {
  const __nv_bfloat16* y;        // [Mp, H] expert-sorted rows of this rank (output of the down projection)
  const int* counts;             // [ep * E]
  const int* block_start;        // [El + 1]
  const int* ret_base;           // [ep * E]
  __nv_bfloat16* ret[EPG_MAX];   // return buffer (set in use) of every rank: [its n_rows, H]
  uint32_t* flags[EPG_MAX];      // one arrival counter per rank (set in use)
  int E, El, ep, rank, H;
};

__global__ void __launch_bounds__(256)
ep_combine_push_kernel(EpcParams p) {
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  const int n_warps = (gridDim.x * blockDim.x) >> 5;
  const int vec = p.H >> 3;
  unsigned cnt[EPG_MAX];
#pragma unroll
  for (int d = 0; d < EPG_MAX; ++d) cnt[d] = 0;
  // (local expert j, source s) segments; rows of a segment are contiguous in y
  for (int j = 0; j < p.El; ++j) {
    const int e = p.rank * p.El + j;
    int seg = p.block_start[j];
    for (int s = 0; s < p.ep; ++s) {
      const int c = p.counts[s * p.E + e];
      for (int i = warp; i < c; i += n_warps) {
        const uint4* src = reinterpret_cast<const uint4*>(p.y + (long long)(seg + i) * p.H);
        uint4* dst = reinterpret_cast<uint4*>(p.ret[s] + ((long long)p.ret_base[s * p.E + e] + i) * p.H);
        for (int v = lane; v < vec; v += 32) dst[v] = src[v];
#pragma unroll
        for (int q = 0; q < EPG_MAX; ++q) cnt[q] += (q == s) ? 1u : 0u;
      }
      seg += c;
    }
  }
  __threadfence_system();
  __syncwarp();
  if (lane == 0) {
#pragma unroll
    for (int d = 0; d < EPG_MAX; ++d)
      if (d < p.ep && cnt[d])
        asm volatile("red.release.sys.global.add.u32 [%0], %1;" ::"l"(p.flags[d]), "r"(cnt[d]) : "memory");
  }
}

}  // namespace b200

extern "C" {

int b200_ep_layout(const int* counts, int ep, int E, int rank, int max_tiles, int* send_off, int* dst_base,
                   int* ret_base, int* block_start, int* tile_expert, int* block_target, int* n_tiles,
                   cudaStream_t stream) {
  if (ep < 1 || ep > b200::EPG_MAX || E % ep) return B200_ERR_ARG;
  b200::ep_layout_kernel<<<1, 32, 0, stream>>>(counts, ep, E, rank, max_tiles, send_off, dst_base, ret_base,
                                               block_start, tile_expert, block_target, n_tiles);
  return cudaGetLastError() == cudaSuccess ? 0 : B200_ERR_LAUNCH;
}

// x [n_rows, H] sorted by expert; W [El, N, H]; Y [max_rows, N]; recv_ptrs / flag_ptrs: host arrays [ep] (set in use).
int b200_ep_dispatch_gemm(const void* x, long long ldx, const void* W, void* Y, long long ldy, int max_rows, int N,
                          int H, int E, int ep, int rank, const int* send_off, const int* dst_base,
                          void* const* recv_ptrs, void* const* flag_ptrs, const int* tile_expert,
                          const int* block_target, const int* n_tiles, unsigned long long wait_ns, uint32_t* status,
                          int num_sms, cudaStream_t stream) {
  using namespace b200;
  if (ep < 1 || ep > EPG_MAX || E % ep || (H & 7) || (ldx & 7) || (ldy & 7) || (max_rows % GEMM_BM)) return B200_ERR_ARG;
  EpgParams p{};
  p.x = reinterpret_cast<const __nv_bfloat16*>(x);
  p.ldx = ldx;
  p.send_off = send_off;
  p.dst_base = dst_base;
  for (int d = 0; d < ep; ++d) {
    p.recv[d] = reinterpret_cast<__nv_bfloat16*>(recv_ptrs[d]);
    p.flags[d] = reinterpret_cast<uint32_t*>(flag_ptrs[d]);
  }
  p.tile_expert = tile_expert;
  p.block_target = block_target;
  p.n_tiles = n_tiles;
  p.C = Y;
  p.ldc = ldy;
  p.wait_ns = wait_ns ? wait_ns : WAIT_LIMIT_NS;
  p.E = E; p.El = E / ep; p.ep = ep; p.rank = rank; p.H = H; p.N = N; p.rows_limit = max_rows;
  CUtensorMap tmA, tmB;
  if (make_tmap_2d(&tmA, p.recv[rank], max_rows, H, H, GEMM_BM, GEMM_BK, 2)) return B200_ERR_TENSORMAP;
  if (make_tmap_3d(&tmB, W, E / ep, N, H, H, (uint64_t)N * H, 256, GEMM_BK, 2)) return B200_ERR_TENSORMAP;
  constexpr int SMEM = GemmSmem<256, 4>::TOTAL;
  static bool attr_set = false;
  if (!attr_set) {
    if (cudaFuncSetAttribute(ep_dispatch_gemm_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM) != cudaSuccess)
      return B200_ERR_LAUNCH;
    attr_set = true;
  }
  // every CTA resident: producers wait for rows that the side warps of other CTAs (and other GPUs) push
  ep_dispatch_gemm_kernel<<<num_sms, EPG_THREADS, SMEM, stream>>>(tmA, tmB, max_rows, N, H, p, status);
  return cudaGetLastError() == cudaSuccess ? 0 : B200_ERR_LAUNCH;
}

int b200_ep_combine_push(const void* y, int H, int E, int ep, int rank, const int* counts, const int* block_start,
                         const int* ret_base, void* const* ret_ptrs, void* const* flag_ptrs, cudaStream_t stream) {
  using namespace b200;
  if (ep < 1 || ep > EPG_MAX || E % ep || (H & 7)) return B200_ERR_ARG;
  EpcParams p{};
  p.y = reinterpret_cast<const __nv_bfloat16*>(y);
  p.counts = counts;
  p.block_start = block_start;
  p.ret_base = ret_base;
  for (int d = 0; d < ep; ++d) {
    p.ret[d] = reinterpret_cast<__nv_bfloat16*>(ret_ptrs[d]);
    p.flags[d] = reinterpret_cast<uint32_t*>(flag_ptrs[d]);
  }
  p.E = E; p.El = E / ep; p.ep = ep; p.rank = rank; p.H = H;
  ep_combine_push_kernel<<<148 * 2, 256, 0, stream>>>(p);
  return cudaGetLastError() == cudaSuccess ? 0 : B200_ERR_LAUNCH;
}

}  // extern "C"
