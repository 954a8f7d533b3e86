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

// Destination row of source row r when a stack of (2I, C) gate|up matrices is re-ordered per 64 rows.
__device__ __forceinline__ long long interleaved_row(long long r, long long I) {
  const long long e = r / (2 * I);
  const long long rr = r - e * 2 * I;
  const long long up = rr >= I ? 1 : 0;
  const long long j = rr - up * I;
  return e * 2 * I + (j >> 6) * 128 + up * 64 + (j & 63);
}

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
    const long long dr = interleave_I > 0 ? interleaved_row(r, interleave_I) : r;
    mx_quant_store32(reinterpret_cast<const uint32_t*>(v), q + dr * C + b * 32, sf, dr, b, k_chunks);
  }
}

// Transposing quantiser: x (G, R, C) bf16 -> q_t (G, C, R) e4m3 with blocks of 32 along R (the rows of
// x become the reduction dimension).  A CTA owns a 128 x 128 tile; warp w quantises row block w & 3
// (32 rows) of column half w >> 2, lane l owning columns 2l and 2l+1 of that half.  The codes are staged
// in shared memory as [column][128 bytes along R] (16-byte chunks XOR-swizzled against bank conflicts) and
// leave as full 128-byte lines; the four scale bytes of a column leave as one word.  R % 32 == 0.
// ROWS: the same pass also writes the row-wise quantisation of the tile (blocks of 32 along C; rows
// optionally 64-interleaved), re-reading the tile from cache instead of DRAM.  Needs C % 32 == 0.
// GATHER (G = 1): row r of the quantised matrix is x[row_slot[r] / k] (a token row) when r < *total_rows and
// row_slot[r] >= 0, and a zero row otherwise: the gathered matrix itself is never written.
template <bool ROWS, bool GATHER = false>
__global__ void __launch_bounds__(256, 4)
quant_tile_kernel(const __nv_bfloat16* __restrict__ x, long long G, long long R, long long C, long long interleave_I,
                  uint8_t* __restrict__ q_t, uint8_t* __restrict__ sf_t, uint8_t* __restrict__ q_r,
                  uint8_t* __restrict__ sf_r, const int* __restrict__ row_slot = nullptr,
                  const int* __restrict__ total_rows = nullptr, int k = 1) {
  // source row of matrix row r (nullptr = zero row)
  auto src_row = [&](long long g, long long r) -> const __nv_bfloat16* {
    if constexpr (GATHER) {
      if (r >= *total_rows) return nullptr;
      const int slot = row_slot[r];
      return slot < 0 ? nullptr : x + static_cast<long long>(slot / k) * C;
    } else {
      return x + (g * R + r) * C;
    }
  };
  __shared__ __align__(16) uint8_t s_q[128 * 128];
  __shared__ uint32_t s_sf[128];
  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;
  const int rbw = warp & 3, ch = warp >> 2;
  const long long rtiles = (R + 127) >> 7, ctiles = (C + 127) >> 7;
  const long long kc_t = rtiles;             // 128-wide k chunks of the transposed output (K = R)
  const long long kc_r = (C + 127) >> 7;     // ... of the row-wise output (K = C)
  const long long total = G * rtiles * ctiles;
  for (long long tile = blockIdx.x; tile < total; tile += gridDim.x) {
    const long long g = tile / (rtiles * ctiles);
    const long long rem = tile - g * rtiles * ctiles;
    const long long rt = rem / ctiles;
    const long long ct = rem - rt * ctiles;
    if constexpr (ROWS) {   // coalesced first touch of the tile; the strided reads below then hit cache
#pragma unroll
      for (int i = 0; i < 2; ++i) {
        const int it = threadIdx.x + 256 * i;
        const long long r = rt * 128 + (it >> 2);
        const long long cb = ct * 128 + (it & 3) * 32;
        if (r < R && cb < C) {
          const long long gr = g * R + r;
          const __nv_bfloat16* srow = src_row(g, r);
          uint4 v[4];
#pragma unroll
          for (int j = 0; j < 4; ++j)
            v[j] = srow != nullptr ? __ldg(reinterpret_cast<const uint4*>(srow + cb) + j) : make_uint4(0u, 0u, 0u, 0u);
          const long long dr = interleave_I > 0 ? interleaved_row(gr, interleave_I) : gr;
          mx_quant_store32(reinterpret_cast<const uint32_t*>(v), q_r + dr * C + cb, sf_r, dr, cb >> 5, kc_r);
        }
      }
    }
    {
      const long long r0 = rt * 128 + rbw * 32;
      const long long c = ct * 128 + ch * 64 + 2 * lane;
      int my_tok = -1;   // GATHER: lane i looks up the token of row r0 + i once, the warp shares it by shuffle
      if constexpr (GATHER) {
        const long long r = r0 + lane;
        if (r < R && r < *total_rows) {
          const int slot = row_slot[r];
          if (slot >= 0) my_tok = slot / k;
        }
      }
      uint4 oa[2] = {make_uint4(0u, 0u, 0u, 0u), make_uint4(0u, 0u, 0u, 0u)};
      uint4 ob[2] = {make_uint4(0u, 0u, 0u, 0u), make_uint4(0u, 0u, 0u, 0u)};
      uint32_t sa = 0u, sbb = 0u;
      uint32_t v[32];   // row i of the block: column c in the low half, column c + 1 in the high half
      if constexpr (GATHER) {   // every lane takes part in the shuffles, also those past the last column
        const bool in = r0 < R && c < C;
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          const int t = __shfl_sync(0xffffffffu, my_tok, i);
          v[i] = (in && t >= 0) ? __ldg(reinterpret_cast<const uint32_t*>(x + static_cast<long long>(t) * C + c)) : 0u;
        }
      }
      if (r0 < R && c < C) {
        if constexpr (!GATHER) {
          const __nv_bfloat16* src = x + (g * R + r0) * C + c;
#pragma unroll
          for (int i = 0; i < 32; ++i) v[i] = __ldg(reinterpret_cast<const uint32_t*>(src + i * C));
        }
        uint32_t m = 0u;
#pragma unroll
        for (int i = 0; i < 32; ++i) m = absmax_bf16x2(m, v[i]);
        sa = e8m0_from_amax(bf16_lo(m));
        sbb = e8m0_from_amax(bf16_hi(m));
        const float ia = inv_scale_from_e8m0(sa), ib = inv_scale_from_e8m0(sbb);
        uint32_t* wa = reinterpret_cast<uint32_t*>(oa);
        uint32_t* wb = reinterpret_cast<uint32_t*>(ob);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          wa[j] = cvt4_e4m3(bf16_lo(v[4 * j]) * ia, bf16_lo(v[4 * j + 1]) * ia, bf16_lo(v[4 * j + 2]) * ia,
                            bf16_lo(v[4 * j + 3]) * ia);
          wb[j] = cvt4_e4m3(bf16_hi(v[4 * j]) * ib, bf16_hi(v[4 * j + 1]) * ib, bf16_hi(v[4 * j + 2]) * ib,
                            bf16_hi(v[4 * j + 3]) * ib);
        }
      }
      const int cl = ch * 64 + 2 * lane;   // column inside the tile; cl and cl+1 share the swizzle key lane & 7
      const int j0 = rbw * 2;
      uint8_t* ra = s_q + cl * 128;
      *reinterpret_cast<uint4*>(ra + ((j0 ^ (lane & 7)) << 4)) = oa[0];
      *reinterpret_cast<uint4*>(ra + (((j0 + 1) ^ (lane & 7)) << 4)) = oa[1];
      *reinterpret_cast<uint4*>(ra + 128 + ((j0 ^ (lane & 7)) << 4)) = ob[0];
      *reinterpret_cast<uint4*>(ra + 128 + (((j0 + 1) ^ (lane & 7)) << 4)) = ob[1];
      reinterpret_cast<uint8_t*>(s_sf)[cl * 4 + rbw] = static_cast<uint8_t>(sa);
      reinterpret_cast<uint8_t*>(s_sf)[cl * 4 + 4 + rbw] = static_cast<uint8_t>(sbb);
    }
    __syncthreads();
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int idx = threadIdx.x + 256 * i;
      const int cl = idx >> 3, j = idx & 7;
      const long long cg = ct * 128 + cl;
      const long long rr = rt * 128 + j * 16;
      if (cg < C && rr < R)
        *reinterpret_cast<uint4*>(q_t + (g * C + cg) * R + rr) =
            *reinterpret_cast<const uint4*>(s_q + cl * 128 + ((j ^ ((cl >> 1) & 7)) << 4));
    }
    if (threadIdx.x < 128) {
      const long long cg = ct * 128 + threadIdx.x;
      if (cg < C) {
        const long long orow = g * C + cg;   // output row (a column of x)
        uint8_t* dst = sf_t + sf_offset(orow, rt * 4, kc_t);
        if (rt * 128 + 128 <= R) {
          *reinterpret_cast<uint32_t*>(dst) = s_sf[threadIdx.x];
        } else {
          for (int b = 0; rt * 128 + b * 32 < R; ++b) dst[b] = reinterpret_cast<const uint8_t*>(s_sf)[threadIdx.x * 4 + b];
        }
      }
    }
    __syncthreads();   // the staging tile is free again
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

static int launch_quant_tile(const void* x, long long G, long long R, long long C, long long interleave_I, void* q_t,
                             void* sf_t, void* q_r, void* sf_r, cudaStream_t stream) {
  const long long tiles = G * ((R + 127) / 128) * ((C + 127) / 128);
  long long grid = tiles;
  const long long cap = static_cast<long long>(num_sms()) * 8;
  if (grid > cap) grid = cap;
  if (q_r != nullptr)
    quant_tile_kernel<true><<<static_cast<int>(grid), 256, 0, stream>>>(
        reinterpret_cast<const __nv_bfloat16*>(x), G, R, C, interleave_I, reinterpret_cast<uint8_t*>(q_t),
        reinterpret_cast<uint8_t*>(sf_t), reinterpret_cast<uint8_t*>(q_r), reinterpret_cast<uint8_t*>(sf_r));
  else
    quant_tile_kernel<false><<<static_cast<int>(grid), 256, 0, stream>>>(
        reinterpret_cast<const __nv_bfloat16*>(x), G, R, C, 0, reinterpret_cast<uint8_t*>(q_t),
        reinterpret_cast<uint8_t*>(sf_t), nullptr, nullptr);
  B200_CUDA(cudaGetLastError());
  return 0;
}

int b200moe_mxfp8_gather_quant_both(const void* x, const int32_t* row_slot, const int32_t* total_rows, int k, int64_t H,
                                    int64_t rows_cap, void* q_rows, void* sf_rows, void* q_t, void* sf_t,
                                    b200moe_stream_t stream) {
  B200_CHECK_ARG(x && row_slot && total_rows && q_rows && sf_rows && q_t && sf_t, B200MOE_E_NULL,
                 "mxfp8_gather_quant_both: null pointer");
  B200_CHECK_ARG(H > 0 && H % 32 == 0 && k >= 1 && rows_cap >= 0 && rows_cap % 32 == 0, B200MOE_E_BAD_SHAPE,
                 "mxfp8_gather_quant_both: H = %lld and rows_cap = %lld must be multiples of 32", (long long)H,
                 (long long)rows_cap);
  B200_CHECK_ARG(aligned16(x) && aligned16(q_rows) && aligned16(q_t) && (reinterpret_cast<uintptr_t>(sf_t) & 3) == 0,
                 B200MOE_E_ALIGN, "mxfp8_gather_quant_both: pointers must be 16-byte aligned");
  if (rows_cap == 0) return 0;
  const long long tiles = ((rows_cap + 127) / 128) * ((H + 127) / 128);
  long long grid = tiles;
  const long long cap = static_cast<long long>(num_sms()) * 8;
  if (grid > cap) grid = cap;
  quant_tile_kernel<true, true><<<static_cast<int>(grid), 256, 0, (cudaStream_t)stream>>>(
      reinterpret_cast<const __nv_bfloat16*>(x), 1, rows_cap, H, 0, reinterpret_cast<uint8_t*>(q_t),
      reinterpret_cast<uint8_t*>(sf_t), reinterpret_cast<uint8_t*>(q_rows), reinterpret_cast<uint8_t*>(sf_rows), row_slot,
      total_rows, k);
  B200_CUDA(cudaGetLastError());
  return 0;
}

int b200moe_mxfp8_quant_transpose(const void* x, int64_t G, int64_t R, int64_t C, void* q, void* sf,
                                  b200moe_stream_t stream) {
  B200_CHECK_ARG(x && q && sf, B200MOE_E_NULL, "mxfp8_quant_transpose: null pointer");
  B200_CHECK_ARG(G >= 1 && R > 0 && R % 32 == 0 && C > 0 && C % 2 == 0, B200MOE_E_BAD_SHAPE,
                 "mxfp8_quant_transpose: R = %lld must be a multiple of 32 and C = %lld even", (long long)R, (long long)C);
  B200_CHECK_ARG(aligned16(q) && (reinterpret_cast<uintptr_t>(x) & 3) == 0 && (reinterpret_cast<uintptr_t>(sf) & 3) == 0,
                 B200MOE_E_ALIGN, "mxfp8_quant_transpose: pointers not aligned");
  return launch_quant_tile(x, G, R, C, 0, q, sf, nullptr, nullptr, (cudaStream_t)stream);
}

int b200moe_mxfp8_quant_both(const void* x, int64_t G, int64_t R, int64_t C, int64_t interleave_I, void* q_rows,
                             void* sf_rows, void* q_t, void* sf_t, b200moe_stream_t stream) {
  B200_CHECK_ARG(x && q_rows && sf_rows && q_t && sf_t, B200MOE_E_NULL, "mxfp8_quant_both: null pointer");
  B200_CHECK_ARG(G >= 1 && R > 0 && R % 32 == 0 && C > 0 && C % 32 == 0, B200MOE_E_BAD_SHAPE,
                 "mxfp8_quant_both: R = %lld and C = %lld must be positive multiples of 32", (long long)R, (long long)C);
  B200_CHECK_ARG(interleave_I == 0 || (interleave_I % 64 == 0 && R % (2 * interleave_I) == 0), B200MOE_E_BAD_SHAPE,
                 "mxfp8_quant_both: interleave needs I %% 64 == 0 and R a multiple of 2I (I = %lld, R = %lld)",
                 (long long)interleave_I, (long long)R);
  B200_CHECK_ARG(aligned16(x) && aligned16(q_rows) && aligned16(q_t) && (reinterpret_cast<uintptr_t>(sf_t) & 3) == 0,
                 B200MOE_E_ALIGN, "mxfp8_quant_both: pointers must be 16-byte aligned");
  return launch_quant_tile(x, G, R, C, interleave_I, q_t, sf_t, q_rows, sf_rows, (cudaStream_t)stream);
}

}  // extern "C"
