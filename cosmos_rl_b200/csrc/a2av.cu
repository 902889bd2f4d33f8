// All-to-all-v of token rows over NVLink peer memory: the expert-parallel dispatch / combine exchange without a
// library collective. Every rank pushes the rows it owes each peer (rows are sorted by destination rank) straight
// into that peer's receive buffer at the row offset both sides derive from the exchanged split sizes, with plain
// 16-byte peer stores (one warp per row: a warp writes the row's contiguous bytes), then adds the number of rows
// it delivered to the peer's arrival counter (red.release.sys). The receiver's stream waits for the counter with
// the bounded flag-wait kernel of peer.cu before the expert GEMMs start.
// Replaces torch.distributed.all_to_all_single with split sizes and the reference's symmetric-memory on-device
// all-to-all-v / DeepEP dispatch (cosmos_rl/policy/kernel/megatron_moe/fused_a2a.py:84-230,
// cosmos_rl/policy/kernel/moe/indices.py, token_dispatcher.py:808-1201).
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "api.h"

namespace {

constexpr int A2A_MAX = 8;

struct A2avParams {
  const uint4* src;          // [rows, vec_per_row] rows sorted by destination rank
  long long src_ld;          // uint4 per source row
  int vec_per_row;           // row bytes / 16
  int ep;
  int send_off[A2A_MAX + 1]; // row prefix by destination
  uint4* dst[A2A_MAX];       // receive buffer of each destination (peer mapped), already offset to the set in use
  long long dst_row[A2A_MAX];// first row this rank writes in that buffer
  long long dst_ld;          // uint4 per destination row
  uint32_t* flags[A2A_MAX];  // arrival counter of each destination (set in use)
};

__global__ void __launch_bounds__(256)
a2av_push_kernel(A2avParams p) {
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  const int n_warps = (gridDim.x * blockDim.x) >> 5;
  const int rows = p.send_off[p.ep];
  unsigned cnt[A2A_MAX];
#pragma unroll
  for (int d = 0; d < A2A_MAX; ++d) cnt[d] = 0;
  for (int r = warp; r < rows; r += n_warps) {
    int d = 0;
#pragma unroll
    for (int q = 1; q < A2A_MAX; ++q)
      if (q < p.ep && r >= p.send_off[q]) d = q;
    const uint4* s = p.src + (long long)r * p.src_ld;
    uint4* t = p.dst[d] + (p.dst_row[d] + (r - p.send_off[d])) * p.dst_ld;
    for (int v = lane; v < p.vec_per_row; v += 32) t[v] = s[v];
#pragma unroll
    for (int q = 0; q < A2A_MAX; ++q) cnt[q] += (q == d) ? 1u : 0u;
  }
  __threadfence_system();
  __syncwarp();
  if (lane == 0) {
#pragma unroll
    for (int d = 0; d < A2A_MAX; ++d)
      if (d < p.ep && cnt[d])
        asm volatile("red.release.sys.global.add.u32 [%0], %1;" ::"l"(p.flags[d]), "r"(cnt[d]) : "memory");
  }
}

}  // namespace

// src: [rows, row_bytes] (row stride src_ld_bytes), rows sorted by destination; send_off: host array [ep + 1] (row
// prefix by destination rank); dst_ptrs / flag_ptrs: host arrays [ep] of device pointers (receive buffer base and
// arrival counter of every rank for the buffer set in use; entry `rank` = own memory); dst_row: host array [ep]:
// first row this rank writes in each destination. row_bytes, strides: multiples of 16.
extern "C" int b200_a2av_push(const void* src, long long src_ld_bytes, int row_bytes, int ep, const int* send_off,
                              void* const* dst_ptrs, const long long* dst_row, long long dst_ld_bytes,
                              void* const* flag_ptrs, cudaStream_t stream) {
  if (ep < 1 || ep > A2A_MAX || (row_bytes & 15) || (src_ld_bytes & 15) || (dst_ld_bytes & 15)) return B200_ERR_ARG;
  A2avParams p{};
  p.src = reinterpret_cast<const uint4*>(src);
  p.src_ld = src_ld_bytes / 16;
  p.vec_per_row = row_bytes / 16;
  p.ep = ep;
  p.dst_ld = dst_ld_bytes / 16;
  for (int d = 0; d <= ep; ++d) p.send_off[d] = send_off[d];
  for (int d = 0; d < ep; ++d) {
    p.dst[d] = reinterpret_cast<uint4*>(dst_ptrs[d]);
    p.dst_row[d] = dst_row[d];
    p.flags[d] = reinterpret_cast<uint32_t*>(flag_ptrs[d]);
  }
  const int rows = send_off[ep];
  if (rows <= 0) return 0;
  long long want = ((long long)rows * 32 + 255) / 256;
  int grid = (int)(want < 148 * 8 ? want : 148 * 8);
  a2av_push_kernel<<<grid, 256, 0, stream>>>(p);
  return cudaGetLastError() == cudaSuccess ? 0 : B200_ERR_LAUNCH;
}
