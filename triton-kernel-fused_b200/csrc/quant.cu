// MXFP8 quantisation: bf16 -> e4m3 elements with one E8M0 (power-of-two) scale per block of 32
// elements along the reduction dimension K of the GEMM that will consume the tensor.
//
//   scale exponent = floor(log2(amax)) - 8   (8 = largest exponent of e4m3, 448 = 1.75 * 2^8)
//   stored byte    = exponent + 127, clamped to [0, 254]
//   element        = round-to-nearest-even, saturating, of x * 2^-exponent
//
// Scales are written in the layout tcgen05 block-scaled MMAs consume from tensor memory: the scales
// of a (128 rows x 128 k) block form one 512-byte atom, byte offset inside the atom =
// (row % 32) * 16 + ((row % 128) / 32) * 4 + (k / 32) % 4; atoms are ordered row-block major,
// k-chunk minor.
#include <cuda_bf16.h>
#include <cuda_fp8.h>

#include "common.cuh"
#include "mxfp8_quant.cuh"

namespace b200moe {

// One thread quantises one block of 32 consecutive elements of a row.
// interleave_I > 0: the source is a stack of (2I, C) gate|up matrices; destination rows are
// re-ordered per 64 so that each group of 128 output rows holds gate rows j..j+63 then up rows
// j..j+63 (the SwiGLU GEMM then sees gate and up of the same columns in one 128-wide tile).
__global__ void __launch_bounds__(256)
quant_rows_kernel(const __nv_bfloat16* __restrict__ x, long long R, long long C, long long interleave_I,
                  uint8_t* __restrict__ q, uint8_t* __restrict__ sf) {
  const long long blocks_per_row = C >> 5;
  const long long k_chunks = (C + 127) >> 7;
  const long long total = R * blocks_per_row;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long r = i / blocks_per_row;
    const long long b = i - r * blocks_per_row;
    const uint4* src = reinterpret_cast<const uint4*>(x + r * C + b * 32);
    uint4 v[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) v[j] = __ldg(src + j);
    float f[32];
    float amax = 0.0f;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const uint32_t w[4] = {v[j].x, v[j].y, v[j].z, v[j].w};
#pragma unroll
      for (int h = 0; h < 4; ++h) {
        const float2 t = unpack_bf16x2(w[h]);
        f[j * 8 + 2 * h] = t.x;
        f[j * 8 + 2 * h + 1] = t.y;
        amax = fmaxf(amax, fmaxf(fabsf(t.x), fabsf(t.y)));
      }
    }
    const uint32_t sb = e8m0_from_amax(amax);
    const float inv = inv_scale_from_e8m0(sb);
    long long dr = r;
    if (interleave_I > 0) {
      const long long e = r / (2 * interleave_I);
      const long long rr = r - e * 2 * interleave_I;
      const long long up = rr >= interleave_I ? 1 : 0;
      const long long j = rr - up * interleave_I;
      dr = e * 2 * interleave_I + (j >> 6) * 128 + up * 64 + (j & 63);
    }
    uint4 o[2];
    uint32_t* ow = reinterpret_cast<uint32_t*>(o);
#pragma unroll
    for (int j = 0; j < 8; ++j)
      ow[j] = cvt4_e4m3(f[4 * j] * inv, f[4 * j + 1] * inv, f[4 * j + 2] * inv, f[4 * j + 3] * inv);
    uint4* dst = reinterpret_cast<uint4*>(q + dr * C + b * 32);
    dst[0] = o[0];
    dst[1] = o[1];
    sf[sf_offset(dr, b, k_chunks)] = static_cast<uint8_t>(sb);
  }
}

// Transposing quantiser: x (G, R, C) bf16 -> q (G, C, R) e4m3 with blocks of 32 along R (the rows of
// x become the reduction dimension).  One warp owns 32 rows x 64 columns; lane l owns columns
// 2l, 2l+1 and writes 32 bytes (one block) for each of them.  R must be a multiple of 32.
__global__ void __launch_bounds__(256)
quant_transpose_kernel(const __nv_bfloat16* __restrict__ x, long long G, long long R, long long C,
                       uint8_t* __restrict__ q, uint8_t* __restrict__ sf) {
  const int lane = threadIdx.x & 31;
  const long long warps_per_grid = (static_cast<long long>(gridDim.x) * blockDim.x) >> 5;
  const long long cblocks = (C + 63) >> 6;
  const long long rblocks = R >> 5;
  const long long k_chunks = (R + 127) >> 7;
  const long long total = G * rblocks * cblocks;
  for (long long wi = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5; wi < total;
       wi += warps_per_grid) {
    const long long g = wi / (rblocks * cblocks);
    const long long rem = wi - g * rblocks * cblocks;
    const long long rb = rem / cblocks;
    const long long cb = rem - rb * cblocks;
    const long long c = cb * 64 + 2 * lane;
    if (c >= C) continue;
    const __nv_bfloat16* src = x + (g * R + rb * 32) * C + c;
    float a[32], b[32];
    float amax_a = 0.0f, amax_b = 0.0f;
#pragma unroll
    for (int i = 0; i < 32; ++i) {
      const float2 t = unpack_bf16x2(__ldg(reinterpret_cast<const uint32_t*>(src + i * C)));
      a[i] = t.x;
      b[i] = t.y;
      amax_a = fmaxf(amax_a, fabsf(t.x));
      amax_b = fmaxf(amax_b, fabsf(t.y));
    }
    const uint32_t sa = e8m0_from_amax(amax_a), sbb = e8m0_from_amax(amax_b);
    const float ia = inv_scale_from_e8m0(sa), ib = inv_scale_from_e8m0(sbb);
    uint4 oa[2], ob[2];
    uint32_t* wa = reinterpret_cast<uint32_t*>(oa);
    uint32_t* wb = reinterpret_cast<uint32_t*>(ob);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      wa[j] = cvt4_e4m3(a[4 * j] * ia, a[4 * j + 1] * ia, a[4 * j + 2] * ia, a[4 * j + 3] * ia);
      wb[j] = cvt4_e4m3(b[4 * j] * ib, b[4 * j + 1] * ib, b[4 * j + 2] * ib, b[4 * j + 3] * ib);
    }
    const long long orow = g * C + c;   // output row (a column of x)
    uint4* da = reinterpret_cast<uint4*>(q + orow * R + rb * 32);
    da[0] = oa[0];
    da[1] = oa[1];
    sf[sf_offset(orow, rb, k_chunks)] = static_cast<uint8_t>(sa);
    if (c + 1 < C) {
      uint4* db = reinterpret_cast<uint4*>(q + (orow + 1) * R + rb * 32);
      db[0] = ob[0];
      db[1] = ob[1];
      sf[sf_offset(orow + 1, rb, k_chunks)] = static_cast<uint8_t>(sbb);
    }
  }
}

// Gather fused with the row quantiser: x_s[r] = x[row_slot[r] / k] (bf16 copy kept for the backward)
// and its e4m3 codes + scales; pad rows become zeros with scale byte 0.  One thread per 32-element block.
__global__ void __launch_bounds__(256)
gather_quant_kernel(const __nv_bfloat16* __restrict__ x, const int* __restrict__ row_slot,
                    const int* __restrict__ total_rows, int k, long long C, __nv_bfloat16* __restrict__ x_s,
                    uint8_t* __restrict__ q, uint8_t* __restrict__ sf) {
  const long long blocks_per_row = C >> 5;
  const long long k_chunks = (C + 127) >> 7;
  const long long total = static_cast<long long>(*total_rows) * blocks_per_row;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long r = i / blocks_per_row;
    const long long b = i - r * blocks_per_row;
    const int slot = row_slot[r];
    uint4 v[4];
    if (slot >= 0) {
      const uint4* src = reinterpret_cast<const uint4*>(x + static_cast<long long>(slot / k) * C + b * 32);
#pragma unroll
      for (int j = 0; j < 4; ++j) v[j] = __ldg(src + j);
    } else {
#pragma unroll
      for (int j = 0; j < 4; ++j) v[j] = make_uint4(0u, 0u, 0u, 0u);
    }
    uint4* dst = reinterpret_cast<uint4*>(x_s + r * C + b * 32);
#pragma unroll
    for (int j = 0; j < 4; ++j) dst[j] = v[j];
    mx_quant_store32(reinterpret_cast<const uint32_t*>(v), q + r * C + b * 32, sf, r, b, k_chunks);
  }
}

}  // namespace b200moe

using namespace b200moe;

extern "C" {

size_t b200moe_mxfp8_sf_bytes(int64_t rows, int64_t K) {
  if (rows <= 0 || K <= 0) return 0;
  return static_cast<size_t>(((rows + 127) / 128) * ((K + 127) / 128) * 512);
}

int b200moe_mxfp8_quant_rows(const void* x, int64_t R, int64_t C, int64_t interleave_I, void* q, void* sf,
                             b200moe_stream_t stream) {
  B200_CHECK_ARG(x && q && sf, B200MOE_E_NULL, "mxfp8_quant_rows: null pointer");
  B200_CHECK_ARG(R >= 0 && C > 0 && C % 32 == 0, B200MOE_E_BAD_SHAPE,
                 "mxfp8_quant_rows: C = %lld must be a positive multiple of 32", (long long)C);
  B200_CHECK_ARG(interleave_I == 0 || (interleave_I % 64 == 0 && R % (2 * interleave_I) == 0), B200MOE_E_BAD_SHAPE,
                 "mxfp8_quant_rows: interleave needs I %% 64 == 0 and R a multiple of 2I (I = %lld, R = %lld)",
                 (long long)interleave_I, (long long)R);
  B200_CHECK_ARG(aligned16(x) && aligned16(q), B200MOE_E_ALIGN, "mxfp8_quant_rows: pointers must be 16-byte aligned");
  if (R == 0) return 0;
  const long long total = R * (C / 32);
  long long grid = (total + 255) / 256;
  const long long cap = static_cast<long long>(num_sms()) * 32;
  if (grid > cap) grid = cap;
  quant_rows_kernel<<<static_cast<int>(grid), 256, 0, (cudaStream_t)stream>>>(
      reinterpret_cast<const __nv_bfloat16*>(x), R, C, interleave_I, reinterpret_cast<uint8_t*>(q),
      reinterpret_cast<uint8_t*>(sf));
  B200_CUDA(cudaGetLastError());
  return 0;
}

int b200moe_mxfp8_gather_quant(const void* x, const int32_t* row_slot, const int32_t* total_rows, int k, int64_t H,
                               int64_t rows_cap, void* x_s, void* q, void* sf, b200moe_stream_t stream) {
  B200_CHECK_ARG(x && row_slot && total_rows && x_s && q && sf, B200MOE_E_NULL, "mxfp8_gather_quant: null pointer");
  B200_CHECK_ARG(H > 0 && H % 32 == 0 && k >= 1, B200MOE_E_BAD_SHAPE, "mxfp8_gather_quant: H = %lld must be a multiple of 32",
                 (long long)H);
  B200_CHECK_ARG(aligned16(x) && aligned16(x_s) && aligned16(q), B200MOE_E_ALIGN, "mxfp8_gather_quant: pointers must be aligned");
  if (rows_cap <= 0) return 0;
  const long long total = rows_cap * (H / 32);
  long long grid = (total + 255) / 256;
  const long long cap = static_cast<long long>(num_sms()) * 32;
  if (grid > cap) grid = cap;
  gather_quant_kernel<<<static_cast<int>(grid), 256, 0, (cudaStream_t)stream>>>(
      reinterpret_cast<const __nv_bfloat16*>(x), row_slot, total_rows, k, H, reinterpret_cast<__nv_bfloat16*>(x_s),
      reinterpret_cast<uint8_t*>(q), reinterpret_cast<uint8_t*>(sf));
  B200_CUDA(cudaGetLastError());
  return 0;
}

int b200moe_mxfp8_quant_transpose(const void* x, int64_t G, int64_t R, int64_t C, void* q, void* sf,
                                  b200moe_stream_t stream) {
  B200_CHECK_ARG(x && q && sf, B200MOE_E_NULL, "mxfp8_quant_transpose: null pointer");
  B200_CHECK_ARG(G >= 1 && R > 0 && R % 32 == 0 && C > 0 && C % 2 == 0, B200MOE_E_BAD_SHAPE,
                 "mxfp8_quant_transpose: R = %lld must be a multiple of 32 and C = %lld even", (long long)R, (long long)C);
  B200_CHECK_ARG(R % 16 == 0 && aligned16(q), B200MOE_E_ALIGN, "mxfp8_quant_transpose: output not 16-byte aligned");
  const long long warps = G * (R / 32) * ((C + 63) / 64);
  long long grid = (warps + 7) / 8;
  const long long cap = static_cast<long long>(num_sms()) * 32;
  if (grid > cap) grid = cap;
  quant_transpose_kernel<<<static_cast<int>(grid), 256, 0, (cudaStream_t)stream>>>(
      reinterpret_cast<const __nv_bfloat16*>(x), G, R, C, reinterpret_cast<uint8_t*>(q),
      reinterpret_cast<uint8_t*>(sf));
  B200_CUDA(cudaGetLastError());
  return 0;
}

}  // extern "C"
