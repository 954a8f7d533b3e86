// Weighted combine (forward), its backward, both as gather-reduce passes over 16-byte vectors.
// Deterministic: every output element is produced by exactly one thread, no atomics.
#include <cuda_bf16.h>

#include "common.cuh"
#include "ptx.cuh"

namespace b200moe {

__device__ __forceinline__ void fma8(float (&acc)[8], const uint4& v, float w) {
  const float2 a = unpack_bf16x2(v.x), b = unpack_bf16x2(v.y), c = unpack_bf16x2(v.z), d = unpack_bf16x2(v.w);
  acc[0] += w * a.x; acc[1] += w * a.y; acc[2] += w * b.x; acc[3] += w * b.y;
  acc[4] += w * c.x; acc[5] += w * c.y; acc[6] += w * d.x; acc[7] += w * d.y;
}

constexpr int kVecBatch = 4;   // 16-byte vectors a lane keeps in flight per row it reads

// out[t] = sum_j w[t,j] * rows[slot_row[t*k+j]]  (fp32 accumulate in slot order j = 0..k-1)
__global__ void __launch_bounds__(256)
combine_kernel(const uint4* __restrict__ rows, const float* __restrict__ w, const int* __restrict__ slot_row,
               long long T, int k, int vec_per_row, uint4* __restrict__ out) {
  __shared__ int s_row[B200MOE_MAX_TOPK];
  __shared__ float s_w[B200MOE_MAX_TOPK];
  for (long long t = blockIdx.x; t < T; t += gridDim.x) {
    __syncthreads();
    if (threadIdx.x < k) {
      s_row[threadIdx.x] = slot_row[t * k + threadIdx.x];
      s_w[threadIdx.x] = (w != nullptr) ? w[t * k + threadIdx.x] : 1.0f;
    }
    __syncthreads();
    for (int c = threadIdx.x; c < vec_per_row; c += blockDim.x) {
      float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
      for (int j = 0; j < k; ++j) {
        if (s_row[j] < 0) continue;   // a slot without a row (its expert index was out of range) adds nothing
        const uint4 v = rows[static_cast<long long>(s_row[j]) * vec_per_row + c];
        fma8(acc, v, s_w[j]);
      }
      uint4 o;
      o.x = pack_bf16x2(acc[0], acc[1]);
      o.y = pack_bf16x2(acc[2], acc[3]);
      o.z = pack_bf16x2(acc[4], acc[5]);
      o.w = pack_bf16x2(acc[6], acc[7]);
      out[t * vec_per_row + c] = o;
    }
  }
}

// grad_eo[r] = bf16(go[tok] * w[slot]);  grad_w[slot] = sum_h go[tok,h] * eo[r,h]  (fp32)
// One warp per routed row, 2 * kVecBatch independent 16-byte loads in flight per lane; the dot product is
// reduced by shuffles in a fixed order.
__global__ void __launch_bounds__(256)
combine_bwd_kernel(const uint4* __restrict__ go, const uint4* __restrict__ eo, const float* __restrict__ w,
                   const int* __restrict__ row_slot, const int* __restrict__ total_rows, int k, int vec_per_row,
                   uint4* __restrict__ grad_eo, float* __restrict__ grad_w) {
  const int lane = threadIdx.x & 31;
  const long long warps = (static_cast<long long>(gridDim.x) * blockDim.x) >> 5;
  const int total = *total_rows;
  for (long long r = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5; r < total; r += warps) {
    const int slot = row_slot[r];
    uint4* dst = grad_eo + r * vec_per_row;
    if (slot < 0) {
      for (int c = lane; c < vec_per_row; c += 32) dst[c] = make_uint4(0u, 0u, 0u, 0u);
      continue;
    }
    const float wt = w[slot];
    const uint4* g = go + static_cast<long long>(slot / k) * vec_per_row;
    const uint4* e = eo + r * vec_per_row;
    float dot = 0.0f;
    for (int c0 = 0; c0 < vec_per_row; c0 += 32 * kVecBatch) {
      uint4 gv[kVecBatch], ev[kVecBatch];
#pragma unroll
      for (int i = 0; i < kVecBatch; ++i) {
        const int c = c0 + 32 * i + lane;
        gv[i] = c < vec_per_row ? g[c] : make_uint4(0u, 0u, 0u, 0u);
        ev[i] = c < vec_per_row ? e[c] : make_uint4(0u, 0u, 0u, 0u);
      }
#pragma unroll
      for (int i = 0; i < kVecBatch; ++i) {
        const int c = c0 + 32 * i + lane;
        const float2 g0 = unpack_bf16x2(gv[i].x), g1 = unpack_bf16x2(gv[i].y), g2 = unpack_bf16x2(gv[i].z),
                     g3 = unpack_bf16x2(gv[i].w);
        const float2 e0 = unpack_bf16x2(ev[i].x), e1 = unpack_bf16x2(ev[i].y), e2 = unpack_bf16x2(ev[i].z),
                     e3 = unpack_bf16x2(ev[i].w);
        dot += g0.x * e0.x + g0.y * e0.y + g1.x * e1.x + g1.y * e1.y + g2.x * e2.x + g2.y * e2.y + g3.x * e3.x +
               g3.y * e3.y;
        if (c < vec_per_row) {
          uint4 o;
          o.x = pack_bf16x2(g0.x * wt, g0.y * wt);
          o.y = pack_bf16x2(g1.x * wt, g1.y * wt);
          o.z = pack_bf16x2(g2.x * wt, g2.y * wt);
          o.w = pack_bf16x2(g3.x * wt, g3.y * wt);
          dst[c] = o;
        }
      }
    }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, off);
    if (lane == 0) grad_w[slot] = dot;
  }
}

}  // namespace b200moe

using namespace b200moe;

extern "C" {

int b200moe_combine(const void* rows, const float* w, const int32_t* slot_row, int64_t T, int k, int64_t H,
                    void* out, b200moe_stream_t stream) {
  B200_CHECK_ARG(rows && slot_row && out, B200MOE_E_NULL, "combine: null pointer");
  B200_CHECK_ARG(H > 0 && H % 8 == 0, B200MOE_E_BAD_SHAPE, "combine: H = %lld must be a multiple of 8", (long long)H);
  B200_CHECK_ARG(k >= 1 && k <= B200MOE_MAX_TOPK, B200MOE_E_BAD_SHAPE, "combine: k = %d", k);
  B200_CHECK_ARG(aligned16(rows) && aligned16(out), B200MOE_E_ALIGN, "combine: pointers must be 16-byte aligned");
  if (T <= 0) return 0;
  long long grid = T;
  const long long cap = static_cast<long long>(num_sms()) * 16;
  if (grid > cap) grid = cap;
  combine_kernel<<<static_cast<int>(grid), 256, 0, (cudaStream_t)stream>>>(
      reinterpret_cast<const uint4*>(rows), w, slot_row, T, k, static_cast<int>(H / 8), reinterpret_cast<uint4*>(out));
  B200_CUDA(cudaGetLastError());
  return 0;
}

int b200moe_combine_bwd(const void* grad_out, const void* eo, const float* w, const int32_t* row_slot,
                        const int32_t* total_rows, int k, int64_t H, int64_t rows_cap, void* grad_eo, float* grad_w,
                        b200moe_stream_t stream) {
  B200_CHECK_ARG(grad_out && eo && w && row_slot && total_rows && grad_eo && grad_w, B200MOE_E_NULL,
                 "combine_bwd: null pointer");
  B200_CHECK_ARG(H > 0 && H % 8 == 0, B200MOE_E_BAD_SHAPE, "combine_bwd: H = %lld must be a multiple of 8", (long long)H);
  B200_CHECK_ARG(k >= 1, B200MOE_E_BAD_SHAPE, "combine_bwd: k = %d", k);
  B200_CHECK_ARG(aligned16(grad_out) && aligned16(eo) && aligned16(grad_eo), B200MOE_E_ALIGN,
                 "combine_bwd: pointers must be 16-byte aligned");
  if (rows_cap <= 0) return 0;
  long long grid = (rows_cap + 7) / 8;   // one warp per routed row, 8 warps per CTA
  const long long cap = static_cast<long long>(num_sms()) * 8;
  if (grid > cap) grid = cap;
  combine_bwd_kernel<<<static_cast<int>(grid), 256, 0, (cudaStream_t)stream>>>(
      reinterpret_cast<const uint4*>(grad_out), reinterpret_cast<const uint4*>(eo), w, row_slot, total_rows, k,
      static_cast<int>(H / 8), reinterpret_cast<uint4*>(grad_eo), grad_w);
  B200_CUDA(cudaGetLastError());
  return 0;
}

}  // extern "C"
