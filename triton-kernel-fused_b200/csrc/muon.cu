// Expert-stack optimizer step (Muon): the element-wise and reduction kernels around the Newton-Schulz GEMMs.
//
// The reference's step (kernels/sm75/muon.py:300-315 `_compute`, :366-434 `step`) is, per stack of E matrices
// (E, r, c): decoupled weight decay, momentum (+ Nesterov), orthogonalisation of the momentum by a Newton-Schulz
// iteration (:62-89 `newton_schulz`: Frobenius normalisation, then X <- a X + (b A + c A A) X with A = X X^T on
// the smaller Gram side), a scale, and the update of the parameters.  The three matrix products per iteration run on
// the grouped tcgen05 GEMMs of gemm.cu over a stack whose row segments are padded to the GEMM's 256-row tiles; the
// kernels here produce that padded (and, for tall matrices, transposed) stack, fold the axpy steps, and apply the
// result.  All of them are HBM-bound streaming kernels: 16-byte accesses, one pass over their operands.
//
// Rounding follows the reference run with a bf16 iteration dtype (its setting for Blackwell,
// kernels/sm120/muon.py): every tensor the reference materialises in bf16 is rounded at the same place here;
// norms are accumulated in fp32 (kernels/sm75/muon.py:78).
#include <cuda_bf16.h>

#include "common.cuh"
#include "ptx.cuh"

namespace b200moe {

__device__ __forceinline__ void unpack8(const uint4& v, float (&f)[8]) {
  const float2 a = unpack_bf16x2(v.x), b = unpack_bf16x2(v.y), c = unpack_bf16x2(v.z), d = unpack_bf16x2(v.w);
  f[0] = a.x; f[1] = a.y; f[2] = b.x; f[3] = b.y; f[4] = c.x; f[5] = c.y; f[6] = d.x; f[7] = d.y;
}
__device__ __forceinline__ uint4 pack8(const float (&f)[8]) {
  uint4 o;
  o.x = pack_bf16x2(f[0], f[1]); o.y = pack_bf16x2(f[2], f[3]);
  o.z = pack_bf16x2(f[4], f[5]); o.w = pack_bf16x2(f[6], f[7]);
  return o;
}
__device__ __forceinline__ float round_bf16(float v) { return __bfloat162float(__float2bfloat16_rn(v)); }

// buf = mu * buf + g;  u = nesterov ? g + mu * buf : buf   (kernels/sm75/muon.py:389-390), 8 elements per thread.
// g is first rounded to bf16 (the reference gathers the gradients into a bf16 staging buffer, :386-388).
template <bool kGradF32>
__global__ void __launch_bounds__(256) muon_momentum_kernel(const void* __restrict__ grad, uint4* __restrict__ mom,
                                                            uint4* __restrict__ u, long long nvec, float mu,
                                                            int nesterov) {
  for (long long i = blockIdx.x * 256LL + threadIdx.x; i < nvec; i += gridDim.x * 256LL) {
    float g[8], m[8], o[8];
    if (kGradF32) {
      const float4 g0 = reinterpret_cast<const float4*>(grad)[2 * i], g1 = reinterpret_cast<const float4*>(grad)[2 * i + 1];
      g[0] = g0.x; g[1] = g0.y; g[2] = g0.z; g[3] = g0.w; g[4] = g1.x; g[5] = g1.y; g[6] = g1.z; g[7] = g1.w;
#pragma unroll
      for (int j = 0; j < 8; ++j) g[j] = round_bf16(g[j]);
    } else {
      unpack8(reinterpret_cast<const uint4*>(grad)[i], g);
    }
    unpack8(mom[i], m);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      m[j] = round_bf16(round_bf16(m[j] * mu) + g[j]);
      o[j] = nesterov ? g[j] + mu * m[j] : m[j];
    }
    mom[i] = pack8(m);
    u[i] = pack8(o);
  }
}

// rowss[row] = sum_j x[row, j]^2 in fp32; one warp per row.
__global__ void __launch_bounds__(256) muon_row_sumsq_kernel(const uint4* __restrict__ x, long long rows, int vec_per_row,
                                                             float* __restrict__ rowss) {
  const int lane = threadIdx.x & 31;
  for (long long row = blockIdx.x * 8LL + (threadIdx.x >> 5); row < rows; row += gridDim.x * 8LL) {
    const uint4* src = x + row * vec_per_row;
    float ss = 0.0f;
    for (int c = lane; c < vec_per_row; c += 32) {
      float f[8];
      unpack8(src[c], f);
#pragma unroll
      for (int j = 0; j < 8; ++j) ss += f[j] * f[j];
    }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, off);
    if (lane == 0) rowss[row] = ss;
  }
}

// out[row, :] = bf16(x[row, :] * (tgt / max(sqrt(rowss[row]), eps))) and the sum of squares of the rounded row:
// the row prescale of the reference's default `aurora` mode (kernels/muon/muon_scaling.py:107-112).
__global__ void __launch_bounds__(256) muon_prescale_rows_kernel(const uint4* __restrict__ x, const float* __restrict__ rowss,
                                                                 long long rows, int vec_per_row, float tgt, float eps,
                                                                 uint4* __restrict__ out, float* __restrict__ rowss_out) {
  const int lane = threadIdx.x & 31;
  for (long long row = blockIdx.x * 8LL + (threadIdx.x >> 5); row < rows; row += gridDim.x * 8LL) {
    const float s = tgt / fmaxf(sqrtf(rowss[row]), eps);
    const uint4* src = x + row * vec_per_row;
    uint4* dst = out + row * vec_per_row;
    float ss = 0.0f;
    for (int c = lane; c < vec_per_row; c += 32) {
      float f[8];
      unpack8(src[c], f);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        f[j] = round_bf16(f[j] * s);
        ss += f[j] * f[j];
      }
      dst[c] = pack8(f);
    }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, off);
    if (lane == 0) rowss_out[row] = ss;
  }
}

// out[row, :] = bf16(x[row, :] * mult[row]) and the sum of squares of the rounded row: the row prescale of the
// reference's `aurora_ema` mode (one combined multiplier per row, kernels/muon/muon_scaling.py:141-142).
__global__ void __launch_bounds__(256) muon_scale_rows_kernel(const uint4* __restrict__ x, const float* __restrict__ mult,
                                                              long long rows, int vec_per_row, uint4* __restrict__ out,
                                                              float* __restrict__ rowss_out) {
  const int lane = threadIdx.x & 31;
  for (long long row = blockIdx.x * 8LL + (threadIdx.x >> 5); row < rows; row += gridDim.x * 8LL) {
    const float s = mult[row];
    const uint4* src = x + row * vec_per_row;
    uint4* dst = out + row * vec_per_row;
    float ss = 0.0f;
    for (int c = lane; c < vec_per_row; c += 32) {
      float f[8];
      unpack8(src[c], f);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        f[j] = round_bf16(f[j] * s);
        ss += f[j] * f[j];
      }
      dst[c] = pack8(f);
    }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, off);
    if (lane == 0) rowss_out[row] = ss;
  }
}

// p[row, :] = decay * p[row, :] + alpha * bf16(x[row, :] * mult[row]): the weight update of the per-row scale modes
// (`normuon`, `aurora_ema_v2`: kernels/muon/muon_scaling.py:166-195, kernels/sm75/muon.py:381,431-434), x in the
// parameters' own (rows, cols) layout.  One warp per row.
template <bool kPF32>
__global__ void __launch_bounds__(256) muon_update_rows_kernel(const uint4* __restrict__ x, const float* __restrict__ mult,
                                                               long long rows, int vec_per_row, float decay, float alpha,
                                                               void* p) {
  const int lane = threadIdx.x & 31;
  for (long long row = blockIdx.x * 8LL + (threadIdx.x >> 5); row < rows; row += gridDim.x * 8LL) {
    const float s = mult[row];
    const uint4* src = x + row * vec_per_row;
    for (int c = lane; c < vec_per_row; c += 32) {
      float o[8], w[8];
      unpack8(src[c], o);
      const long long pi = (row * vec_per_row + c) * 8;
      if (kPF32) {
        float4* pp = reinterpret_cast<float4*>(reinterpret_cast<float*>(p) + pi);
        const float4 a = pp[0], b = pp[1];
        w[0] = a.x; w[1] = a.y; w[2] = a.z; w[3] = a.w; w[4] = b.x; w[5] = b.y; w[6] = b.z; w[7] = b.w;
#pragma unroll
        for (int t = 0; t < 8; ++t) w[t] = w[t] * decay + alpha * round_bf16(o[t] * s);
        pp[0] = make_float4(w[0], w[1], w[2], w[3]);
        pp[1] = make_float4(w[4], w[5], w[6], w[7]);
      } else {
        uint4* pp = reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(p) + pi);
        unpack8(*pp, w);
#pragma unroll
        for (int t = 0; t < 8; ++t) w[t] = round_bf16(w[t] * decay) + alpha * round_bf16(o[t] * s);
        *pp = pack8(w);
      }
    }
  }
}

// norms[e] = bf16(max(sqrt(sum_i rowss[e, i]), eps)) as a float: the per-matrix Frobenius norm the iteration divides
// by (kernels/sm75/muon.py:78,82).  One CTA per matrix, fixed summation order (reruns are bit-identical).
__global__ void __launch_bounds__(256) muon_stack_norms_kernel(const float* __restrict__ rowss, int r, float eps,
                                                               float* __restrict__ norms) {
  __shared__ float part[256];
  const float* src = rowss + static_cast<long long>(blockIdx.x) * r;
  float s = 0.0f;
  for (int i = threadIdx.x; i < r; i += 256) s += src[i];
  part[threadIdx.x] = s;
  __syncthreads();
  for (int w = 128; w > 0; w >>= 1) {
    if (threadIdx.x < w) part[threadIdx.x] += part[threadIdx.x + w];
    __syncthreads();
  }
  if (threadIdx.x == 0) norms[blockIdx.x] = round_bf16(fmaxf(sqrtf(part[0]), eps));
}

// Stack in the layout of the iteration, rows kept: xp (E, Rp, c), xp[e, i, :] = bf16(x[e, i, :] / norms[e]) for
// i < r and zero rows up to Rp (kernels/sm75/muon.py:82).  One warp per output row.
__global__ void __launch_bounds__(256) muon_pack_rows_kernel(const uint4* __restrict__ x, const float* __restrict__ norms,
                                                             int E, int r, int Rp, int vec_per_row,
                                                             uint4* __restrict__ xp) {
  const int lane = threadIdx.x & 31;
  const long long total = static_cast<long long>(E) * Rp;
  for (long long orow = blockIdx.x * 8LL + (threadIdx.x >> 5); orow < total; orow += gridDim.x * 8LL) {
    const int e = static_cast<int>(orow / Rp), i = static_cast<int>(orow % Rp);
    uint4* dst = xp + orow * vec_per_row;
    if (i >= r) {
      for (int c = lane; c < vec_per_row; c += 32) dst[c] = make_uint4(0u, 0u, 0u, 0u);
      continue;
    }
    const float nrm = norms[e];
    const uint4* src = x + (static_cast<long long>(e) * r + i) * vec_per_row;
    for (int c = lane; c < vec_per_row; c += 32) {
      float f[8];
      unpack8(src[c], f);
#pragma unroll
      for (int j = 0; j < 8; ++j) f[j] = f[j] / nrm;
      dst[c] = pack8(f);
    }
  }
}

// A 64 x 64 bf16 tile in shared memory for transposing with 16-byte accesses on both sides: 64 rows of 32 words
// (bf16 pairs); word w of row r sits at w ^ ((r >> 3) << 2), which keeps 8-value vectors whole and makes the
// column-wise reads of the second phase conflict-free.  Thread v (0..511, two per thread) owns the vector of row
// v >> 3 that starts at column 8 * (v & 7), in the source for the first phase and in the destination for the second.
struct TransposeTile {
  uint32_t w[64 * 32];
  __device__ __forceinline__ void put(int r, int c8, const uint4& v) {
    *reinterpret_cast<uint4*>(&w[r * 32 + ((c8 >> 1) ^ ((r >> 3) << 2))]) = v;
  }
  // the 8 values of destination row r, columns c8 .. c8+7 = source column r, rows c8 .. c8+7
  __device__ __forceinline__ void get_transposed(int r, int c8, float (&f)[8]) const {
    const __nv_bfloat16* h = reinterpret_cast<const __nv_bfloat16*>(w);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const int sr = c8 + j;
      f[j] = __bfloat162float(h[2 * (sr * 32 + ((r >> 1) ^ ((sr >> 3) << 2))) + (r & 1)]);
    }
  }
};

// Tall matrices (r > c) iterate on the transpose (kernels/sm75/muon.py:79-81): xp (E, Rp, r),
// xp[e, j, i] = bf16(x[e, i, j] / norms[e]) for j < c, zero rows for c <= j < Rp.  grid = (ceil(r/64), Rp/64, E).
__global__ void __launch_bounds__(256) muon_pack_transpose_kernel(const __nv_bfloat16* __restrict__ x,
                                                                  const float* __restrict__ norms, int r, int c, int Rp,
                                                                  __nv_bfloat16* __restrict__ xp) {
  __shared__ __align__(16) TransposeTile tile;
  const int e = blockIdx.z, i0 = blockIdx.x * 64, j0 = blockIdx.y * 64;
  const float nrm = norms[e];
  const __nv_bfloat16* src = x + static_cast<long long>(e) * r * c;
#pragma unroll
  for (int k = 0; k < 2; ++k) {
    const int v = threadIdx.x + 256 * k, i = i0 + (v >> 3), j = j0 + (v & 7) * 8;
    uint4 q = make_uint4(0u, 0u, 0u, 0u);
    if (i < r && j < c) {                                  // c is a multiple of 8: the vector is inside or outside
      float f[8];
      unpack8(*reinterpret_cast<const uint4*>(src + static_cast<long long>(i) * c + j), f);
#pragma unroll
      for (int t = 0; t < 8; ++t) f[t] = f[t] / nrm;
      q = pack8(f);
    }
    tile.put(v >> 3, (v & 7) * 8, q);
  }
  __syncthreads();
  __nv_bfloat16* dst = xp + static_cast<long long>(e) * Rp * r;
#pragma unroll
  for (int k = 0; k < 2; ++k) {
    const int v = threadIdx.x + 256 * k, j = j0 + (v >> 3), i = i0 + (v & 7) * 8;
    if (i < r) {
      float f[8];
      tile.get_transposed(v >> 3, (v & 7) * 8, f);
      *reinterpret_cast<uint4*>(dst + static_cast<long long>(j) * r + i) = pack8(f);
    }
  }
}

// out = bf16(alpha * x + beta * y + diag * I) over a stack of ld x ld matrices (ld = 0: plain vectors, no identity
// term).  One pass builds the whole left factor of an iteration: the reference's X <- a X + (b A + c A A) X
// (kernels/sm75/muon.py:85-86) is evaluated as ((b A + c A A) + a I) X, so the a X term rides on the GEMM and costs no
// pass over X.  out may alias x or y.
__global__ void __launch_bounds__(256) axpby_bf16_kernel(const uint4* x, float alpha, const uint4* y, float beta,
                                                         float diag, int ld, uint4* out, long long nvec) {
  for (long long i = blockIdx.x * 256LL + threadIdx.x; i < nvec; i += gridDim.x * 256LL) {
    float a[8], b[8];
    unpack8(x[i], a);
    unpack8(y[i], b);
#pragma unroll
    for (int j = 0; j < 8; ++j) a[j] = alpha * a[j] + beta * b[j];
    if (ld > 0) {
      const long long e0 = i * 8;                       // ld is a multiple of 8: the 8 elements share a row
      const int col0 = static_cast<int>(e0 % ld), row = static_cast<int>((e0 / ld) % ld);
      if (row >= col0 && row < col0 + 8) {
#pragma unroll
        for (int j = 0; j < 8; ++j)
          if (col0 + j == row) a[j] += diag;
      }
    }
    out[i] = pack8(a);
  }
}

template <bool kPF32>
__device__ __forceinline__ float load_param(const void* p, long long i) {
  return kPF32 ? reinterpret_cast<const float*>(p)[i] : __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(p)[i]);
}
template <bool kPF32>
__device__ __forceinline__ float round_param(float v) { return kPF32 ? v : round_bf16(v); }
template <bool kPF32>
__device__ __forceinline__ void store_param(void* p, long long i, float v) {
  if (kPF32) reinterpret_cast<float*>(p)[i] = v;
  else reinterpret_cast<__nv_bfloat16*>(p)[i] = __float2bfloat16_rn(v);
}

// p = round(round(p * decay) + alpha * bf16(gain * o)), o = the orthogonalised stack read back from the iteration's
// layout (kernels/sm75/muon.py:381,431-434; gain: kernels/muon/muon_scaling.py:112).  Rows kept: o = xp[e, i, j].
template <bool kPF32>
__global__ void __launch_bounds__(256) muon_apply_rows_kernel(const __nv_bfloat16* __restrict__ xp, int E, int r, int c,
                                                              int Rp, float gain, float decay, float alpha, void* p) {
  const long long total = static_cast<long long>(E) * r * (c / 2);
  for (long long t = blockIdx.x * 256LL + threadIdx.x; t < total; t += gridDim.x * 256LL) {
    const int j = static_cast<int>(t % (c / 2)) * 2;
    const long long row = t / (c / 2);
    const int e = static_cast<int>(row / r), i = static_cast<int>(row % r);
    const float2 o = __bfloat1622float2(
        *reinterpret_cast<const __nv_bfloat162*>(xp + (static_cast<long long>(e) * Rp + i) * c + j));
    const long long pi = row * c + j;
    store_param<kPF32>(p, pi, round_param<kPF32>(load_param<kPF32>(p, pi) * decay) + alpha * round_bf16(gain * o.x));
    store_param<kPF32>(p, pi + 1,
                       round_param<kPF32>(load_param<kPF32>(p, pi + 1) * decay) + alpha * round_bf16(gain * o.y));
  }
}

// Transposed stack: o[e, i, j] = xp[e, j, i] with xp (E, Rp, r).  grid = (ceil(r/64), ceil(c/64), E).
template <bool kPF32>
__global__ void __launch_bounds__(256) muon_apply_transpose_kernel(const __nv_bfloat16* __restrict__ xp, int r, int c,
                                                                   int Rp, float gain, float decay, float alpha,
                                                                   void* p) {
  __shared__ __align__(16) TransposeTile tile;
  const int e = blockIdx.z, i0 = blockIdx.x * 64, j0 = blockIdx.y * 64;
  const __nv_bfloat16* src = xp + static_cast<long long>(e) * Rp * r;
#pragma unroll
  for (int k = 0; k < 2; ++k) {
    const int v = threadIdx.x + 256 * k, j = j0 + (v >> 3), i = i0 + (v & 7) * 8;
    uint4 q = make_uint4(0u, 0u, 0u, 0u);
    if (j < c && i < r) q = *reinterpret_cast<const uint4*>(src + static_cast<long long>(j) * r + i);
    tile.put(v >> 3, (v & 7) * 8, q);
  }
  __syncthreads();
#pragma unroll
  for (int k = 0; k < 2; ++k) {
    const int v = threadIdx.x + 256 * k, i = i0 + (v >> 3), j = j0 + (v & 7) * 8;
    if (i < r && j < c) {
      float o[8], w[8];
      tile.get_transposed(v >> 3, (v & 7) * 8, o);
      const long long pi = (static_cast<long long>(e) * r + i) * c + j;
      if (kPF32) {
        float4* pp = reinterpret_cast<float4*>(reinterpret_cast<float*>(p) + pi);
        const float4 a = pp[0], b = pp[1];
        w[0] = a.x; w[1] = a.y; w[2] = a.z; w[3] = a.w; w[4] = b.x; w[5] = b.y; w[6] = b.z; w[7] = b.w;
#pragma unroll
        for (int t = 0; t < 8; ++t) w[t] = w[t] * decay + alpha * round_bf16(gain * o[t]);
        pp[0] = make_float4(w[0], w[1], w[2], w[3]);
        pp[1] = make_float4(w[4], w[5], w[6], w[7]);
      } else {
        uint4* pp = reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(p) + pi);
        unpack8(*pp, w);
#pragma unroll
        for (int t = 0; t < 8; ++t) w[t] = round_bf16(w[t] * decay) + alpha * round_bf16(gain * o[t]);
        *pp = pack8(w);
      }
    }
  }
}

// a[e, i, j] = a[e, j, i] for every 64 x 64 block strictly below the block diagonal of each n x n matrix: completes a
// symmetric product of which only the tiles reaching the upper triangle were computed.  grid = (n/64, n/64, E).
__global__ void __launch_bounds__(256) mirror_upper_kernel(__nv_bfloat16* __restrict__ a, int n) {
  const int bi = blockIdx.y, bj = blockIdx.x;           // destination block (row bi, column bj)
  if (bi <= bj) return;
  __shared__ __align__(16) TransposeTile tile;          // source block (bj, bi)
  __nv_bfloat16* m = a + static_cast<long long>(blockIdx.z) * n * n;
#pragma unroll
  for (int k = 0; k < 2; ++k) {
    const int v = threadIdx.x + 256 * k, r = v >> 3, c8 = (v & 7) * 8;
    tile.put(r, c8, *reinterpret_cast<const uint4*>(m + static_cast<long long>(bj * 64 + r) * n + bi * 64 + c8));
  }
  __syncthreads();
#pragma unroll
  for (int k = 0; k < 2; ++k) {
    const int v = threadIdx.x + 256 * k, r = v >> 3, c8 = (v & 7) * 8;
    float f[8];
    tile.get_transposed(r, c8, f);                       // bf16 -> float -> bf16 is exact
    *reinterpret_cast<uint4*>(m + static_cast<long long>(bi * 64 + r) * n + bj * 64 + c8) = pack8(f);
  }
}

static int stream_grid(long long work_items, int per_cta) {
  long long grid = (work_items + per_cta - 1) / per_cta;
  const long long cap = static_cast<long long>(num_sms()) * 16;
  if (grid > cap) grid = cap;
  return static_cast<int>(grid < 1 ? 1 : grid);
}

}  // namespace b200moe

using namespace b200moe;

#define MUON_CHECK_DIMS(who, E, r, c, Rp, transposed)                                                             \
  B200_CHECK_ARG((E) >= 1 && (E) <= 65535 && (r) > 0 && (c) > 0 && (r) % 8 == 0 && (c) % 8 == 0 &&                 \
                     (r) < (1LL << 24) && (c) < (1LL << 24),                                                       \
                 B200MOE_E_BAD_SHAPE, who ": a stack of %d matrices of %lld x %lld (both must be multiples of 8)",  \
                 (int)(E), (long long)(r), (long long)(c));                                                        \
  B200_CHECK_ARG((Rp) % B200MOE_TILE_M == 0 && (Rp) >= ((transposed) ? (c) : (r)) && (Rp) < (1LL << 24),           \
                 B200MOE_E_BAD_SHAPE, who ": padded rows %lld must be a multiple of %d covering the smaller side", \
                 (long long)(Rp), B200MOE_TILE_M)

extern "C" {

int b200moe_muon_momentum(const void* grad, int grad_f32, void* mom, void* u, int64_t n, float mu, int nesterov,
                          b200moe_stream_t stream) {
  B200_CHECK_ARG(grad && mom && u, B200MOE_E_NULL, "muon_momentum: null pointer");
  B200_CHECK_ARG(n >= 0 && n % 8 == 0, B200MOE_E_BAD_SHAPE, "muon_momentum: n = %lld must be a multiple of 8", (long long)n);
  B200_CHECK_ARG(aligned16(grad) && aligned16(mom) && aligned16(u), B200MOE_E_ALIGN, "muon_momentum: pointers must be 16-byte aligned");
  if (n == 0) return 0;
  const long long nvec = n / 8;
  const int grid = stream_grid(nvec, 256);
  if (grad_f32)
    muon_momentum_kernel<true><<<grid, 256, 0, (cudaStream_t)stream>>>(grad, (uint4*)mom, (uint4*)u, nvec, mu, nesterov);
  else
    muon_momentum_kernel<false><<<grid, 256, 0, (cudaStream_t)stream>>>(grad, (uint4*)mom, (uint4*)u, nvec, mu, nesterov);
  B200_CUDA(cudaGetLastError());
  return 0;
}

int b200moe_muon_row_sumsq(const void* x, int64_t rows, int64_t cols, float* rowss, b200moe_stream_t stream) {
  B200_CHECK_ARG(x && rowss, B200MOE_E_NULL, "muon_row_sumsq: null pointer");
  B200_CHECK_ARG(rows >= 0 && cols > 0 && cols % 8 == 0 && cols < (1LL << 24), B200MOE_E_BAD_SHAPE,
                 "muon_row_sumsq: cols = %lld must be a multiple of 8", (long long)cols);
  B200_CHECK_ARG(aligned16(x), B200MOE_E_ALIGN, "muon_row_sumsq: x must be 16-byte aligned");
  if (rows == 0) return 0;
  muon_row_sumsq_kernel<<<stream_grid(rows, 8), 256, 0, (cudaStream_t)stream>>>((const uint4*)x, rows, (int)(cols / 8), rowss);
  B200_CUDA(cudaGetLastError());
  return 0;
}

int b200moe_muon_prescale_rows(const void* x, const float* rowss, int64_t rows, int64_t cols, float tgt, float eps,
                               void* out, float* rowss_out, b200moe_stream_t stream) {
  B200_CHECK_ARG(x && rowss && out && rowss_out, B200MOE_E_NULL, "muon_prescale_rows: null pointer");
  B200_CHECK_ARG(rows >= 0 && cols > 0 && cols % 8 == 0 && cols < (1LL << 24), B200MOE_E_BAD_SHAPE,
                 "muon_prescale_rows: cols = %lld must be a multiple of 8", (long long)cols);
  B200_CHECK_ARG(aligned16(x) && aligned16(out), B200MOE_E_ALIGN, "muon_prescale_rows: pointers must be 16-byte aligned");
  if (rows == 0) return 0;
  muon_prescale_rows_kernel<<<stream_grid(rows, 8), 256, 0, (cudaStream_t)stream>>>(
      (const uint4*)x, rowss, rows, (int)(cols / 8), tgt, eps, (uint4*)out, rowss_out);
  B200_CUDA(cudaGetLastError());
  return 0;
}

int b200moe_muon_scale_rows(const void* x, const float* mult, int64_t rows, int64_t cols, void* out, float* rowss_out,
                            b200moe_stream_t stream) {
  B200_CHECK_ARG(x && mult && out && rowss_out, B200MOE_E_NULL, "muon_scale_rows: null pointer");
  B200_CHECK_ARG(rows >= 0 && cols > 0 && cols % 8 == 0 && cols < (1LL << 24), B200MOE_E_BAD_SHAPE,
                 "muon_scale_rows: cols = %lld must be a multiple of 8", (long long)cols);
  B200_CHECK_ARG(aligned16(x) && aligned16(out), B200MOE_E_ALIGN, "muon_scale_rows: pointers must be 16-byte aligned");
  if (rows == 0) return 0;
  muon_scale_rows_kernel<<<stream_grid(rows, 8), 256, 0, (cudaStream_t)stream>>>((const uint4*)x, mult, rows, (int)(cols / 8),
                                                                                 (uint4*)out, rowss_out);
  B200_CUDA(cudaGetLastError());
  return 0;
}

int b200moe_muon_update_rows(const void* x, const float* mult, int64_t rows, int64_t cols, float decay, float alpha, void* p,
                             int p_f32, b200moe_stream_t stream) {
  B200_CHECK_ARG(x && mult && p, B200MOE_E_NULL, "muon_update_rows: null pointer");
  B200_CHECK_ARG(rows >= 0 && cols > 0 && cols % 8 == 0 && cols < (1LL << 24), B200MOE_E_BAD_SHAPE,
                 "muon_update_rows: cols = %lld must be a multiple of 8", (long long)cols);
  B200_CHECK_ARG(aligned16(x) && aligned16(p), B200MOE_E_ALIGN, "muon_update_rows: pointers must be 16-byte aligned");
  if (rows == 0) return 0;
  const int grid = stream_grid(rows, 8);
  if (p_f32)
    muon_update_rows_kernel<true><<<grid, 256, 0, (cudaStream_t)stream>>>((const uint4*)x, mult, rows, (int)(cols / 8), decay, alpha, p);
  else
    muon_update_rows_kernel<false><<<grid, 256, 0, (cudaStream_t)stream>>>((const uint4*)x, mult, rows, (int)(cols / 8), decay, alpha, p);
  B200_CUDA(cudaGetLastError());
  return 0;
}

int b200moe_muon_normalise_pack(const void* x, const float* rowss, int E, int64_t r, int64_t c, int64_t Rp,
                                int transposed, float eps, float* norms, void* xp, b200moe_stream_t stream) {
  B200_CHECK_ARG(x && rowss && norms && xp, B200MOE_E_NULL, "muon_normalise_pack: null pointer");
  MUON_CHECK_DIMS("muon_normalise_pack", E, r, c, Rp, transposed);
  B200_CHECK_ARG(aligned16(x) && aligned16(xp), B200MOE_E_ALIGN, "muon_normalise_pack: pointers must be 16-byte aligned");
  muon_stack_norms_kernel<<<E, 256, 0, (cudaStream_t)stream>>>(rowss, (int)r, eps, norms);
  if (transposed) {
    dim3 grid((unsigned)((r + 63) / 64), (unsigned)(Rp / 64), (unsigned)E);
    muon_pack_transpose_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>((const __nv_bfloat16*)x, norms, (int)r, (int)c,
                                                                       (int)Rp, (__nv_bfloat16*)xp);
  } else {
    muon_pack_rows_kernel<<<stream_grid((long long)E * Rp, 8), 256, 0, (cudaStream_t)stream>>>(
        (const uint4*)x, norms, E, (int)r, (int)Rp, (int)(c / 8), (uint4*)xp);
  }
  B200_CUDA(cudaGetLastError());
  return 0;
}

int b200moe_axpby_bf16(const void* x, float alpha, const void* y, float beta, float diag, int64_t ld, void* out,
                       int64_t n, b200moe_stream_t stream) {
  B200_CHECK_ARG(x && y && out, B200MOE_E_NULL, "axpby_bf16: null pointer");
  B200_CHECK_ARG(n >= 0 && n % 8 == 0, B200MOE_E_BAD_SHAPE, "axpby_bf16: n = %lld must be a multiple of 8", (long long)n);
  B200_CHECK_ARG(ld >= 0 && ld % 8 == 0 && ld < (1LL << 24) && (ld == 0 || n % (ld * ld) == 0), B200MOE_E_BAD_SHAPE,
                 "axpby_bf16: ld = %lld must be a multiple of 8 and n a whole number of ld x ld matrices", (long long)ld);
  B200_CHECK_ARG(aligned16(x) && aligned16(y) && aligned16(out), B200MOE_E_ALIGN, "axpby_bf16: pointers must be 16-byte aligned");
  if (n == 0) return 0;
  axpby_bf16_kernel<<<stream_grid(n / 8, 256), 256, 0, (cudaStream_t)stream>>>((const uint4*)x, alpha, (const uint4*)y, beta,
                                                                               diag, (int)ld, (uint4*)out, n / 8);
  B200_CUDA(cudaGetLastError());
  return 0;
}

int b200moe_mirror_upper(void* a, int E, int64_t n, b200moe_stream_t stream) {
  B200_CHECK_ARG(a, B200MOE_E_NULL, "mirror_upper: null pointer");
  B200_CHECK_ARG(E >= 1 && E <= 65535 && n > 0 && n % 64 == 0 && n < (1LL << 22), B200MOE_E_BAD_SHAPE,
                 "mirror_upper: %d matrices of order %lld (must be a multiple of 64)", E, (long long)n);
  B200_CHECK_ARG(aligned16(a), B200MOE_E_ALIGN, "mirror_upper: pointer must be 16-byte aligned");
  dim3 grid((unsigned)(n / 64), (unsigned)(n / 64), (unsigned)E);
  mirror_upper_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>((__nv_bfloat16*)a, (int)n);
  B200_CUDA(cudaGetLastError());
  return 0;
}

int b200moe_muon_apply(const void* xp, int E, int64_t r, int64_t c, int64_t Rp, int transposed, float gain, float decay,
                       float alpha, void* p, int p_f32, b200moe_stream_t stream) {
  B200_CHECK_ARG(xp && p, B200MOE_E_NULL, "muon_apply: null pointer");
  MUON_CHECK_DIMS("muon_apply", E, r, c, Rp, transposed);
  B200_CHECK_ARG(aligned16(xp) && aligned16(p), B200MOE_E_ALIGN, "muon_apply: pointers must be 16-byte aligned");
  const cudaStream_t s = (cudaStream_t)stream;
  const __nv_bfloat16* o = (const __nv_bfloat16*)xp;
  if (transposed) {
    dim3 grid((unsigned)((r + 63) / 64), (unsigned)((c + 63) / 64), (unsigned)E);
    if (p_f32) muon_apply_transpose_kernel<true><<<grid, 256, 0, s>>>(o, (int)r, (int)c, (int)Rp, gain, decay, alpha, p);
    else muon_apply_transpose_kernel<false><<<grid, 256, 0, s>>>(o, (int)r, (int)c, (int)Rp, gain, decay, alpha, p);
  } else {
    const int grid = stream_grid((long long)E * r * (c / 2), 256);
    if (p_f32) muon_apply_rows_kernel<true><<<grid, 256, 0, s>>>(o, E, (int)r, (int)c, (int)Rp, gain, decay, alpha, p);
    else muon_apply_rows_kernel<false><<<grid, 256, 0, s>>>(o, E, (int)r, (int)c, (int)Rp, gain, decay, alpha, p);
  }
  B200_CUDA(cudaGetLastError());
  return 0;
}

}  // extern "C"
