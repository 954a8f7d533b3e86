// Device helpers of the MXFP8 quantisers, shared with the GEMM epilogues that quantise their own output.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp8.h>
#include <stdint.h>

#include "ptx.cuh"

namespace b200moe {

__device__ __forceinline__ uint32_t e8m0_from_amax(float amax) {
  const uint32_t e = (__float_as_uint(amax) >> 23) & 0xffu;   // biased exponent = floor(log2) + 127
  return e > 8u ? (e - 8u > 254u ? 254u : e - 8u) : 0u;        // zero / denormal amax -> smallest scale
}
__device__ __forceinline__ float inv_scale_from_e8m0(uint32_t sb) {
  return __uint_as_float((254u - sb) << 23);                   // 2^(127 - sb), sb <= 247 here
}
__device__ __forceinline__ uint32_t cvt4_e4m3(float a, float b, float c, float d) {
  const uint32_t lo = __nv_cvt_float2_to_fp8x2(make_float2(a, b), __NV_SATFINITE, __NV_E4M3);
  const uint32_t hi = __nv_cvt_float2_to_fp8x2(make_float2(c, d), __NV_SATFINITE, __NV_E4M3);
  return lo | (hi << 16);
}
__device__ __forceinline__ long long sf_offset(long long row, long long kblock, long long k_chunks) {
  return ((row >> 7) * k_chunks + (kblock >> 2)) * 512 + (row & 31) * 16 + ((row & 127) >> 5) * 4 + (kblock & 3);
}

// running |max| of packed bf16 pairs (exact: bf16 comparisons; a NaN operand is ignored like fmaxf does)
__device__ __forceinline__ uint32_t absmax_bf16x2(uint32_t acc, uint32_t v) {
  const __nv_bfloat162 r = __hmax2(*reinterpret_cast<__nv_bfloat162*>(&acc), __habs2(*reinterpret_cast<__nv_bfloat162*>(&v)));
  return *reinterpret_cast<const uint32_t*>(&r);
}
__device__ __forceinline__ float bf16_lo(uint32_t u) { return __uint_as_float(u << 16); }
__device__ __forceinline__ float bf16_hi(uint32_t u) { return __uint_as_float(u & 0xffff0000u); }

// 32 consecutive bf16 values of one row (16 packed registers) -> 32 e4m3 bytes at `q32` and the scale
// byte of (row, kblock); identical to what quant_rows_kernel writes for the same values.
__device__ __forceinline__ void mx_quant_store32(const uint32_t* pk, uint8_t* q32, uint8_t* sf, long long row,
                                                 long long kblock, long long k_chunks) {
  uint32_t m = 0u;
#pragma unroll
  for (int i = 0; i < 16; ++i) m = absmax_bf16x2(m, pk[i]);
  const uint32_t sb = e8m0_from_amax(fmaxf(bf16_lo(m), bf16_hi(m)));
  const float inv = inv_scale_from_e8m0(sb);
  uint4 o[2];
  uint32_t* ow = reinterpret_cast<uint32_t*>(o);
#pragma unroll
  for (int j = 0; j < 8; ++j)
    ow[j] = cvt4_e4m3(bf16_lo(pk[2 * j]) * inv, bf16_hi(pk[2 * j]) * inv, bf16_lo(pk[2 * j + 1]) * inv,
                      bf16_hi(pk[2 * j + 1]) * inv);
  reinterpret_cast<uint4*>(q32)[0] = o[0];
  reinterpret_cast<uint4*>(q32)[1] = o[1];
  sf[sf_offset(row, kblock, k_chunks)] = static_cast<uint8_t>(sb);
}

}  // namespace b200moe
