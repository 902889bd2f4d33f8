// Microscaling fp4 (OCP MX: 32 elements share one power-of-two E8M0 scale, elements are E2M1) quantisation of bf16
// weights, the scale-factor layout block-scaled tensor-core MMA consumes, and the inverse (for numerics tests and for
// serving through bf16 GEMMs). Pure streaming kernels (2.53 bytes moved per element), grid-stride over 148 SMs.
//
// Scale-factor layouts:
//   swizzle = 0: row-major [R, C/32].
//   swizzle = 1: 128-row x 4-block tiles, 512 B each, tile (rt, ct) at ((rt * ceil(C/128)) + ct) * 512; inside a tile
//                the scale of (row r, block c) sits at (r % 32) * 16 + (r / 32) * 4 + c. This is the interleaving the
//                tcgen05 block-scaled MMA reads scale factors in (one 32-lane x 16-byte TMEM column group per tile).
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "api.h"

namespace {

__device__ __forceinline__ long long sf_index(int r, int cb, int n_cb, int swizzle) {
  if (!swizzle) return (long long)r * n_cb + cb;
  const int tiles_c = (n_cb + 3) / 4;
  const long long tile = (long long)(r / 128) * tiles_c + cb / 4;
  const int rr = r % 128;
  return tile * 512 + (rr % 32) * 16 + (rr / 32) * 4 + (cb % 4);
}

// Work item = 8 consecutive elements (one 16-byte load, one 4-byte store); the 4 lanes of a 32-element block share
// the block maximum with two shuffles. Consecutive lanes take consecutive items, so every warp instruction reads 512
// and writes 128 contiguous bytes.
__global__ void __launch_bounds__(256) quant_mxfp4_kernel(const __nv_bfloat16* __restrict__ x, long long ldx,
                                                           uint8_t* __restrict__ q, uint8_t* __restrict__ sf, int R,
                                                           int C, int swizzle) {
  const uint32_t n_cb = (uint32_t)C / 32;
  const uint32_t per_row = n_cb * 4;                          // items of 8 elements per row
  const uint32_t lane = threadIdx.x & 31;
  // blocks stride over rows, threads over the items of a row: no division anywhere. The inner loop condition is
  // warp-uniform (first lane's item), so every lane reaches the full-mask shuffles below.
  for (uint32_t r = blockIdx.x; r < (uint32_t)R; r += gridDim.x)
  for (uint32_t it0 = threadIdx.x - lane; it0 < per_row; it0 += blockDim.x) {
    const uint32_t it = it0 + lane;
    const bool valid = it < per_row;
    const uint32_t cb = it >> 2, part = it & 3;
    const long long i = (long long)r * per_row + it;
    uint4 v = make_uint4(0, 0, 0, 0);
    if (valid) v = __ldg(reinterpret_cast<const uint4*>(x + (long long)r * ldx + cb * 32 + part * 8));
    const uint32_t w4[4] = {v.x, v.y, v.z, v.w};
    // block maximum of |x| on packed bf16 pairs (sign bits cleared), then across the 4 lanes of the block
    const uint32_t a4[4] = {w4[0] & 0x7fff7fffu, w4[1] & 0x7fff7fffu, w4[2] & 0x7fff7fffu, w4[3] & 0x7fff7fffu};
    const __nv_bfloat162* ab = reinterpret_cast<const __nv_bfloat162*>(a4);
    const __nv_bfloat162 m2 = __hmax2(__hmax2(ab[0], ab[1]), __hmax2(ab[2], ab[3]));
    uint32_t mb = *reinterpret_cast<const uint32_t*>(&m2);
    uint32_t amax_bits = max(mb & 0xffffu, mb >> 16);             // non-negative bf16 bit patterns order like integers
    amax_bits = max(amax_bits, __shfl_xor_sync(0xffffffffu, amax_bits, 1));
    amax_bits = max(amax_bits, __shfl_xor_sync(0xffffffffu, amax_bits, 2));
    // shared exponent: floor(log2(amax)) - 2 (the largest E2M1 magnitude is 6 = 1.5 * 2^2); zero / denormal blocks
    // take the smallest scale. bf16 keeps the fp32 exponent field in bits 7..14.
    int ex = (amax_bits >> 7) ? (int)(amax_bits >> 7) - 127 - 2 : -127;
    ex = max(-127, min(127, ex));
    const float inv = __uint_as_float((uint32_t)(127 - ex) << 23);   // 2^-ex: exponent field 2..254 for finite input
    // eight scaled values -> four e2m1x2 bytes with the sm_100a conversion instruction (round to nearest even,
    // saturating at 6); the first source operand lands in the high nibble. bf16 -> fp32 is a 16-bit shift.
    uint32_t w;
    asm("{\n"
        ".reg .b8 b0, b1, b2, b3;\n"
        "cvt.rn.satfinite.e2m1x2.f32 b0, %2, %1;\n"
        "cvt.rn.satfinite.e2m1x2.f32 b1, %4, %3;\n"
        "cvt.rn.satfinite.e2m1x2.f32 b2, %6, %5;\n"
        "cvt.rn.satfinite.e2m1x2.f32 b3, %8, %7;\n"
        "mov.b32 %0, {b0, b1, b2, b3};\n"
        "}"
        : "=r"(w)
        : "f"(__uint_as_float(w4[0] << 16) * inv), "f"(__uint_as_float(w4[0] & 0xffff0000u) * inv),
          "f"(__uint_as_float(w4[1] << 16) * inv), "f"(__uint_as_float(w4[1] & 0xffff0000u) * inv),
          "f"(__uint_as_float(w4[2] << 16) * inv), "f"(__uint_as_float(w4[2] & 0xffff0000u) * inv),
          "f"(__uint_as_float(w4[3] << 16) * inv), "f"(__uint_as_float(w4[3] & 0xffff0000u) * inv));
    if (valid) {
      reinterpret_cast<uint32_t*>(q)[i] = w;                // packed output is dense: item i = word i
      if (part == 0) sf[sf_index((int)r, (int)cb, (int)n_cb, swizzle)] = (uint8_t)(ex + 127);
    }
  }
}

__global__ void __launch_bounds__(256) dequant_mxfp4_kernel(const uint8_t* __restrict__ q,
                                                             const uint8_t* __restrict__ sf,
                                                             __nv_bfloat16* __restrict__ out, long long ldo, int R,
                                                             int C, int swizzle) {
  const int n_cb = C / 32;
  const long long total = (long long)R * n_cb * 4;
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += stride) {
    const uint32_t blk = (uint32_t)(i >> 2);
    const int part = (int)(i & 3);
    const uint32_t r = blk / (uint32_t)n_cb, cb = blk - r * (uint32_t)n_cb;
    const uint32_t w = __ldg(reinterpret_cast<const uint32_t*>(q) + i);
    const int eb = sf[sf_index((int)r, (int)cb, n_cb, swizzle)];
    const float scale = eb == 0 ? 5.877471754e-39f : __uint_as_float((uint32_t)eb << 23);   // 2^(eb - 127)
    // four e2m1x2 bytes -> four f16x2 pairs with the sm_100a conversion instruction (low nibble first), then scale
    uint32_t h[4];
    asm("{\n"
        ".reg .b8 b0, b1, b2, b3;\n"
        "mov.b32 {b0, b1, b2, b3}, %4;\n"
        "cvt.rn.f16x2.e2m1x2 %0, b0;\n"
        "cvt.rn.f16x2.e2m1x2 %1, b1;\n"
        "cvt.rn.f16x2.e2m1x2 %2, b2;\n"
        "cvt.rn.f16x2.e2m1x2 %3, b3;\n"
        "}"
        : "=r"(h[0]), "=r"(h[1]), "=r"(h[2]), "=r"(h[3])
        : "r"(w));
    __align__(16) __nv_bfloat162 o[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const float2 v2 = __half22float2(*reinterpret_cast<const __half2*>(&h[k]));
      o[k] = __floats2bfloat162_rn(v2.x * scale, v2.y * scale);
    }
    *reinterpret_cast<uint4*>(out + (long long)r * ldo + cb * 32 + part * 8) = *reinterpret_cast<const uint4*>(o);
  }
}

}  // namespace

extern "C" {

// x bf16 [R, C] (row stride ldx elements, C % 32 == 0, rows 16-byte aligned) -> q packed E2M1 [R, C / 2] (low nibble =
// even element), sf E8M0 bytes (layout by `swizzle`; the swizzled buffer holds ceil(R/128) * ceil(C/128) * 512 bytes).
int b200_quant_mxfp4(const void* x, long long ldx, void* q, void* sf, int R, int C, int swizzle, cudaStream_t stream) {
  if (R <= 0 || C <= 0) return 0;
  if (C % 32 != 0 || ldx % 8 != 0 || (long long)R * (C / 32) >= (1ll << 29)) return B200_ERR_ARG;
  const int grid = R < 148 * 16 ? R : 148 * 16;            // blocks stride over rows
  quant_mxfp4_kernel<<<grid, 256, 0, stream>>>((const __nv_bfloat16*)x, ldx, (uint8_t*)q, (uint8_t*)sf, R, C, swizzle);
  return cudaGetLastError() == cudaSuccess ? 0 : B200_ERR_LAUNCH;
}

int b200_dequant_mxfp4(const void* q, const void* sf, void* out, long long ldo, int R, int C, int swizzle,
                       cudaStream_t stream) {
  if (R <= 0 || C <= 0) return 0;
  if (C % 32 != 0 || ldo % 8 != 0 || (long long)R * (C / 32) >= (1ll << 31)) return B200_ERR_ARG;
  const long long total = (long long)R * (C / 32) * 4;
  const int grid = (int)((total + 255) / 256 < 148 * 16 ? (total + 255) / 256 : 148 * 16);
  dequant_mxfp4_kernel<<<grid, 256, 0, stream>>>((const uint8_t*)q, (const uint8_t*)sf, (__nv_bfloat16*)out, ldo, R, C,
                                                 swizzle);
  return cudaGetLastError() == cudaSuccess ? 0 : B200_ERR_LAUNCH;
}

}  // extern "C"
