// Policy -> rollout weight synchronisation as ONE pull kernel over NVLink peer memory, fused with the
// bf16 -> fp8 (e4m3, one fp32 scale per 128 x 128 block) quantisation of the rollout engine's weights.
//
// The reference moves every parameter slice with its own ncclSend/ncclRecv pair in fp32, copies it into
// place, and then re-quantises in a second pass (cosmos_rl/policy/worker/rl_worker.py:419-571,
// cosmos_rl/rollout/worker/rollout_control.py:674-1027, vllm_rollout.py:989-999). Here the resharding
// planner emits a flat table of rectangle-copy descriptors (source pointer in a peer GPU's memory that
// was mapped into this process, destination in the engine's own layout); CTAs walk 128 x 128 tiles of
// those rectangles, read them with plain 16-byte loads through NVLink, reduce the tile's amax in
// shared memory, and write either bf16 or e4m3 + scale. No TMA and no multicast touch peer memory.
#include <cuda_bf16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "api.h"

namespace {

constexpr int RS_THREADS = 256;
constexpr int RS_TILE = 128;
constexpr float E4M3_MAX = 448.f;

__device__ __forceinline__ uint4 ld_stream(const void* p) {
  uint4 v;
  asm volatile("ld.global.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}

__device__ __forceinline__ float amax8(const uint4& u) {
  const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&u);
  float a = 0.f;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    float2 f = __bfloat1622float2(p[i]);
    a = fmaxf(a, fmaxf(fabsf(f.x), fabsf(f.y)));
  }
  return a;
}

__device__ __forceinline__ uint2 quant8(const uint4& u, float inv_scale) {
  const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&u);
  uint16_t o[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    float2 f = __bfloat1622float2(p[i]);
    f.x *= inv_scale;
    f.y *= inv_scale;
    o[i] = (uint16_t)__nv_cvt_float2_to_fp8x2(f, __NV_SATFINITE, __NV_E4M3);
  }
  uint2 r;
  r.x = (uint32_t)o[0] | ((uint32_t)o[1] << 16);
  r.y = (uint32_t)o[2] | ((uint32_t)o[3] << 16);
  return r;
}

// One CTA per 128x128 tile. 256 threads: thread t handles row (t / 16) + 16*i, 8 columns at (t % 16) * 8.
__device__ __forceinline__ void process_tile(const __nv_bfloat16* src, long long src_ld, void* dst, long long dst_ld,
                                             float* scale_out, int rows, int cols, int quant, float* sh) {
  const int cvec = (threadIdx.x & 15) * 8;
  const int r0 = threadIdx.x >> 4;
  uint4 buf[8];
  float amax = 0.f;
  const bool vec_ok = ((src_ld & 7) == 0) && ((reinterpret_cast<uintptr_t>(src) & 15) == 0);
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int r = r0 + 16 * i;
    buf[i] = make_uint4(0, 0, 0, 0);
    if (r < rows && cvec < cols) {
      const __nv_bfloat16* p = src + (long long)r * src_ld + cvec;
      if (vec_ok && cvec + 8 <= cols) {
        buf[i] = ld_stream(p);
      } else {
        __nv_bfloat16 tmp[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) tmp[j] = (cvec + j < cols) ? p[j] : __float2bfloat16(0.f);
        buf[i] = *reinterpret_cast<uint4*>(tmp);
      }
      if (quant) amax = fmaxf(amax, amax8(buf[i]));
    }
  }
  float inv_scale = 1.f;
  if (quant) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    __syncthreads();
    if ((threadIdx.x & 31) == 0) sh[threadIdx.x >> 5] = amax;
    __syncthreads();
    float a = 0.f;
#pragma unroll
    for (int w = 0; w < RS_THREADS / 32; ++w) a = fmaxf(a, sh[w]);
    const float scale = fmaxf(a, 1e-12f) / E4M3_MAX;
    inv_scale = 1.f / scale;
    if (threadIdx.x == 0 && scale_out) *scale_out = scale;
  }
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int r = r0 + 16 * i;
    if (r < rows && cvec < cols) {
      if (quant) {
        uint8_t* p = reinterpret_cast<uint8_t*>(dst) + (long long)r * dst_ld + cvec;
        uint2 qv = quant8(buf[i], inv_scale);
        if (cvec + 8 <= cols && ((reinterpret_cast<uintptr_t>(p) & 7) == 0)) {
          *reinterpret_cast<uint2*>(p) = qv;
        } else {
          const uint8_t* b = reinterpret_cast<const uint8_t*>(&qv);
          for (int j = 0; j < 8 && cvec + j < cols; ++j) p[j] = b[j];
        }
      } else {
        __nv_bfloat16* p = reinterpret_cast<__nv_bfloat16*>(dst) + (long long)r * dst_ld + cvec;
        if (cvec + 8 <= cols && ((reinterpret_cast<uintptr_t>(p) & 15) == 0)) {
          *reinterpret_cast<uint4*>(p) = buf[i];
        } else {
          const __nv_bfloat16* b = reinterpret_cast<const __nv_bfloat16*>(&buf[i]);
          for (int j = 0; j < 8 && cvec + j < cols; ++j) p[j] = b[j];
        }
      }
    }
  }
}

__global__ void __launch_bounds__(RS_THREADS)
reshard_pull_kernel(const B200CopyDesc* __restrict__ descs, const int* __restrict__ tile_prefix, int n_desc,
                    int total_tiles, uint32_t* status) {
  __shared__ float sh[RS_THREADS / 32];
  for (int tile = blockIdx.x; tile < total_tiles; tile += gridDim.x) {
    // binary search: last descriptor whose first tile <= tile
    int lo = 0, hi = n_desc - 1;
    while (lo < hi) {
      int mid = (lo + hi + 1) >> 1;
      if (tile_prefix[mid] <= tile) lo = mid; else hi = mid - 1;
    }
    const B200CopyDesc d = descs[lo];
    const int local = tile - tile_prefix[lo];
    const int tiles_c = (d.cols + RS_TILE - 1) / RS_TILE;
    const int tr = local / tiles_c, tc = local % tiles_c;
    const int rows = min(RS_TILE, d.rows - tr * RS_TILE);
    const int cols = min(RS_TILE, d.cols - tc * RS_TILE);
    const __nv_bfloat16* src =
        reinterpret_cast<const __nv_bfloat16*>(d.src) + (long long)tr * RS_TILE * d.src_ld + tc * RS_TILE;
    void* dst;
    float* sc = nullptr;
    if (d.quant) {
      dst = reinterpret_cast<uint8_t*>(d.dst) + (long long)tr * RS_TILE * d.dst_ld + tc * RS_TILE;
      sc = d.dst_scale ? d.dst_scale + (long long)tr * d.ld_scale + tc : nullptr;
    } else {
      dst = reinterpret_cast<__nv_bfloat16*>(d.dst) + (long long)tr * RS_TILE * d.dst_ld + tc * RS_TILE;
    }
    process_tile(src, d.src_ld, dst, d.dst_ld, sc, rows, cols, d.quant, sh);
    __syncthreads();
  }
  (void)status;
}

// 1 x 128 activation quantisation: one warp per (row, 128-column block)
__global__ void quant_act_kernel(const __nv_bfloat16* __restrict__ src, long long ld_src, uint8_t* __restrict__ dst,
                                 long long ld_dst, float* __restrict__ scales, int R, int C) {
  const int nblk = (C + 127) / 128;
  long long w = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (w >= (long long)R * nblk) return;
  const int r = (int)(w / nblk), bc = (int)(w % nblk);
  const int c = bc * 128 + lane * 4;
  float f[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
  for (int j = 0; j < 4; ++j)
    if (c + j < C) f[j] = __bfloat162float(src[(long long)r * ld_src + c + j]);
  float a = fmaxf(fmaxf(fabsf(f[0]), fabsf(f[1])), fmaxf(fabsf(f[2]), fabsf(f[3])));
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) a = fmaxf(a, __shfl_xor_sync(0xffffffffu, a, o));
  const float scale = fmaxf(a, 1e-12f) / E4M3_MAX;
  const float inv = 1.f / scale;
  if (lane == 0) scales[(long long)r * nblk + bc] = scale;
#pragma unroll
  for (int j = 0; j < 4; ++j)
    if (c + j < C)
      dst[(long long)r * ld_dst + c + j] = (uint8_t)__nv_cvt_float_to_fp8(f[j] * inv, __NV_SATFINITE, __NV_E4M3);
}

__global__ void __launch_bounds__(RS_THREADS)
quant_weight_kernel(const __nv_bfloat16* __restrict__ src, long long ld_src, uint8_t* __restrict__ dst,
                    long long ld_dst, float* __restrict__ scales, int R, int C) {
  __shared__ float sh[RS_THREADS / 32];
  const int tiles_c = (C + RS_TILE - 1) / RS_TILE;
  const int tr = blockIdx.x / tiles_c, tc = blockIdx.x % tiles_c;
  const int rows = min(RS_TILE, R - tr * RS_TILE), cols = min(RS_TILE, C - tc * RS_TILE);
  process_tile(src + (long long)tr * RS_TILE * ld_src + tc * RS_TILE, ld_src,
               dst + (long long)tr * RS_TILE * ld_dst + tc * RS_TILE, ld_dst, scales + (long long)tr * tiles_c + tc,
               rows, cols, 1, sh);
}

}  // namespace

extern "C" {

int b200_reshard_pull(const B200CopyDesc* descs_dev, const int* tile_prefix_dev, int n_desc, int total_tiles,
                      uint32_t* status, cudaStream_t stream) {
  if (n_desc <= 0 || total_tiles <= 0) return 0;
  int grid = total_tiles < 148 * 8 ? total_tiles : 148 * 8;
  reshard_pull_kernel<<<grid, RS_THREADS, 0, stream>>>(descs_dev, tile_prefix_dev, n_desc, total_tiles, status);
  return cudaGetLastError() == cudaSuccess ? 0 : B200_ERR_LAUNCH;
}

int b200_quant_fp8_block(const void* src, long long ld_src, void* dst, long long ld_dst, float* scales, int R, int C,
                         int block_rows, cudaStream_t stream) {
  if (R <= 0 || C <= 0) return 0;
  if (block_rows == 128) {
    int tiles = ((R + RS_TILE - 1) / RS_TILE) * ((C + RS_TILE - 1) / RS_TILE);
    quant_weight_kernel<<<tiles, RS_THREADS, 0, stream>>>((const __nv_bfloat16*)src, ld_src, (uint8_t*)dst, ld_dst,
                                                          scales, R, C);
  } else if (block_rows == 1) {
    long long warps = (long long)R * ((C + 127) / 128);
    quant_act_kernel<<<(unsigned)((warps * 32 + 255) / 256), 256, 0, stream>>>((const __nv_bfloat16*)src, ld_src,
                                                                              (uint8_t*)dst, ld_dst, scales, R, C);
  } else {
    return B200_ERR_ARG;
  }
  return cudaGetLastError() == cudaSuccess ? 0 : B200_ERR_LAUNCH;
}

}  // extern "C"
