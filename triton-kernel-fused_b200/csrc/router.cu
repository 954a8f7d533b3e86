// Router epilogue kernels: sigmoid + selection bias + in-register warp-level top-k + renormalise
// (forward), the matching Jacobian (backward), the bias update and the split-K slice reduction.
// One warp owns one token; lane l holds experts l, l+32, ... (at most 8 values for E <= 256).
#include <cuda_bf16.h>

#include "common.cuh"
#include "ptx.cuh"

namespace b200moe {

constexpr int kMaxVpl = B200MOE_MAX_EXPERTS / 32;  // values per lane
constexpr float kKnockOut = -1e30f;

template <int KIND>
__device__ __forceinline__ float load_in(const void* p, long long i) {
  if (KIND == B200MOE_LOGITS_BF16) return __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(p)[i]);
  return reinterpret_cast<const float*>(p)[i];
}

__device__ __forceinline__ float sigmoid_f(float x) { return 1.0f / (1.0f + expf(-x)); }

template <int KIND>
__global__ void __launch_bounds__(256)
router_topk_fwd_kernel(const void* __restrict__ input, const float* __restrict__ bias, long long T, int E,
                       int k, int norm, float scale, long long* __restrict__ idx_out,
                       float* __restrict__ w_out, int* __restrict__ counts) {
  __shared__ int hist[B200MOE_MAX_EXPERTS];
  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;
  const int wpb = blockDim.x >> 5;
  for (int e = threadIdx.x; e < E; e += blockDim.x) hist[e] = 0;
  __syncthreads();

  float b[kMaxVpl];
#pragma unroll
  for (int i = 0; i < kMaxVpl; ++i) {
    const int e = lane + 32 * i;
    b[i] = (bias != nullptr && e < E) ? bias[e] : 0.0f;
  }

  for (long long t = static_cast<long long>(blockIdx.x) * wpb + warp; t < T;
       t += static_cast<long long>(gridDim.x) * wpb) {
    float sc[kMaxVpl], sel[kMaxVpl];
#pragma unroll
    for (int i = 0; i < kMaxVpl; ++i) {
      const int e = lane + 32 * i;
      if (e < E) {
        const float v = load_in<KIND>(input, t * E + e);
        sc[i] = (KIND == B200MOE_SCORES_F32) ? v : sigmoid_f(v);
        sel[i] = sc[i] + b[i];
      } else {
        sc[i] = 0.0f;
        sel[i] = kKnockOut;
      }
    }
    int my_idx = 0;
    float my_w = 0.0f;
    for (int j = 0; j < k; ++j) {
      // lane-local argmax: ascending i = ascending expert id, strict '>' keeps the lowest index
      float bv = sel[0];
      int bi = lane;
#pragma unroll
      for (int i = 1; i < kMaxVpl; ++i) {
        if (sel[i] > bv) {
          bv = sel[i];
          bi = lane + 32 * i;
        }
      }
      // warp argmax, ties to the lowest expert id
#pragma unroll
      for (int off = 16; off > 0; off >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, bv, off);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, off);
        if (ov > bv || (ov == bv && oi < bi)) {
          bv = ov;
          bi = oi;
        }
      }
      // owner lane hands out the unbiased score and knocks the pick out
      float wv = 0.0f;
#pragma unroll
      for (int i = 0; i < kMaxVpl; ++i) {
        if (bi == lane + 32 * i) {
          wv = sc[i];
          sel[i] = kKnockOut;
        }
      }
      wv = __shfl_sync(0xffffffffu, wv, bi & 31);
      if (lane == j) {
        my_idx = bi;
        my_w = wv;
      }
      if (counts != nullptr && lane == 0 && bi < E) atomicAdd(&hist[bi], 1);
    }
    if (norm && k > 1) {
      float tsum = 0.0f;
      for (int j = 0; j < k; ++j) tsum += __shfl_sync(0xffffffffu, my_w, j);  // fixed order
      tsum += 1e-20f;
      my_w = my_w / tsum;
    }
    my_w = my_w * scale;
    if (lane < k) {
      idx_out[t * k + lane] = my_idx;
      w_out[t * k + lane] = my_w;
    }
  }
  if (counts != nullptr) {
    __syncthreads();
    for (int e = threadIdx.x; e < E; e += blockDim.x) {
      const int c = hist[e];
      if (c != 0) atomicAdd(&counts[e], c);
    }
  }
}

template <int KIND>
__global__ void __launch_bounds__(256)
router_topk_bwd_kernel(const void* __restrict__ logits, const long long* __restrict__ idx,
                       const float* __restrict__ grad_w, long long T, int E, int k, int norm, float scale,
                       __nv_bfloat16* __restrict__ grad_logits) {
  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;
  const int wpb = blockDim.x >> 5;
  for (long long t = static_cast<long long>(blockIdx.x) * wpb + warp; t < T;
       t += static_cast<long long>(gridDim.x) * wpb) {
    float s[kMaxVpl], gs[kMaxVpl];
#pragma unroll
    for (int i = 0; i < kMaxVpl; ++i) {
      const int e = lane + 32 * i;
      s[i] = (e < E) ? sigmoid_f(load_in<KIND>(logits, t * E + e)) : 0.0f;
      gs[i] = 0.0f;
    }
    float tsum = 0.0f, dot = 0.0f;
    if (norm && k > 1) {
      for (int j = 0; j < k; ++j) {
        const int ik = static_cast<int>(idx[t * k + j]);
        const float gk = grad_w[t * k + j];
        const float wk = (ik >= 0 && ik < E) ? sigmoid_f(load_in<KIND>(logits, t * E + ik)) : 0.0f;
        tsum += wk;
        dot += gk * wk;
      }
      tsum += 1e-20f;
    }
    for (int j = 0; j < k; ++j) {
      const int ik = static_cast<int>(idx[t * k + j]);
      const float gk = grad_w[t * k + j];
      const float graw = (norm && k > 1) ? (scale / tsum) * (gk - dot / tsum) : gk * scale;
#pragma unroll
      for (int i = 0; i < kMaxVpl; ++i)
        if (ik == lane + 32 * i) gs[i] += graw;
    }
#pragma unroll
    for (int i = 0; i < kMaxVpl; ++i) {
      const int e = lane + 32 * i;
      if (e < E) grad_logits[t * E + e] = __float2bfloat16_rn(gs[i] * (s[i] * (1.0f - s[i])));
    }
  }
}

__global__ void router_bias_update_kernel(float* bias, const int* counts, int E, float u) {
  __shared__ float red[32];
  float part = 0.0f;
  for (int e = threadIdx.x; e < E; e += blockDim.x) part += static_cast<float>(counts[e]);
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) part += __shfl_xor_sync(0xffffffffu, part, off);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = part;
  __syncthreads();
  float total = 0.0f;
  for (int i = 0; i < (blockDim.x >> 5); ++i) total += red[i];
  const float mean = total / static_cast<float>(E);
  for (int e = threadIdx.x; e < E; e += blockDim.x) {
    const float d = mean - static_cast<float>(counts[e]);
    const float sg = (d > 0.0f) ? 1.0f : (d < 0.0f ? -1.0f : 0.0f);
    bias[e] += u * sg;
  }
}

// D[i] = bf16( sum_s P[s][i] ), 4 elements per thread
__global__ void __launch_bounds__(256)
splitk_reduce_kernel(const float* __restrict__ P, long long slices, long long elems,
                     __nv_bfloat16* __restrict__ D) {
  const long long i4 = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) * 4;
  if (i4 >= elems) return;
  float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
  for (long long s = 0; s < slices; ++s) {
    const float4 v = *reinterpret_cast<const float4*>(P + s * elems + i4);
    acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
  }
  uint2 o;
  o.x = pack_bf16x2(acc.x, acc.y);
  o.y = pack_bf16x2(acc.z, acc.w);
  *reinterpret_cast<uint2*>(D + i4) = o;
}

static int grid_for_tokens(long long T) {
  long long g = (T + 7) / 8;
  const long long cap = static_cast<long long>(num_sms()) * 8;
  if (g > cap) g = cap;
  if (g < 1) g = 1;
  return static_cast<int>(g);
}

}  // namespace b200moe

using namespace b200moe;

extern "C" {

int b200moe_router_topk_fwd(const void* input, int input_kind, const float* bias, int64_t T, int E, int k,
                            int norm_topk, float scale, int64_t* idx, float* w, int32_t* counts,
                            b200moe_stream_t stream) {
  B200_CHECK_ARG(input && idx && w, B200MOE_E_NULL, "router_topk_fwd: null pointer");
  B200_CHECK_ARG(E >= 1 && E <= B200MOE_MAX_EXPERTS, B200MOE_E_UNSUPPORTED,
                 "router_topk_fwd: E = %d, supported 1..%d", E, B200MOE_MAX_EXPERTS);
  B200_CHECK_ARG(k >= 1 && k <= E && k <= B200MOE_MAX_TOPK, B200MOE_E_BAD_SHAPE,
                 "router_topk_fwd: top_k = %d must be in 1..min(E=%d, %d)", k, E, B200MOE_MAX_TOPK);
  B200_CHECK_ARG(T >= 0, B200MOE_E_BAD_SHAPE, "router_topk_fwd: T = %lld", (long long)T);
  cudaStream_t st = (cudaStream_t)stream;
  if (counts != nullptr) B200_CUDA(cudaMemsetAsync(counts, 0, sizeof(int32_t) * E, st));
  if (T == 0) return 0;
  const int grid = grid_for_tokens(T);
  long long* idx_ll = reinterpret_cast<long long*>(idx);
  switch (input_kind) {
    case B200MOE_LOGITS_BF16:
      router_topk_fwd_kernel<B200MOE_LOGITS_BF16><<<grid, 256, 0, st>>>(input, bias, T, E, k, norm_topk, scale, idx_ll, w, counts);
      break;
    case B200MOE_LOGITS_F32:
      router_topk_fwd_kernel<B200MOE_LOGITS_F32><<<grid, 256, 0, st>>>(input, bias, T, E, k, norm_topk, scale, idx_ll, w, counts);
      break;
    case B200MOE_SCORES_F32:
      router_topk_fwd_kernel<B200MOE_SCORES_F32><<<grid, 256, 0, st>>>(input, bias, T, E, k, norm_topk, scale, idx_ll, w, counts);
      break;
    default:
      set_error("router_topk_fwd: unknown input_kind %d", input_kind);
      return B200MOE_E_UNSUPPORTED;
  }
  B200_CUDA(cudaGetLastError());
  return 0;
}

int b200moe_router_topk_bwd(const void* logits, int input_kind, const int64_t* idx, const float* grad_w, int64_t T,
                            int E, int k, int norm_topk, float scale, void* grad_logits, b200moe_stream_t stream) {
  B200_CHECK_ARG(logits && idx && grad_w && grad_logits, B200MOE_E_NULL, "router_topk_bwd: null pointer");
  B200_CHECK_ARG(E >= 1 && E <= B200MOE_MAX_EXPERTS, B200MOE_E_UNSUPPORTED,
                 "router_topk_bwd: E = %d, supported 1..%d", E, B200MOE_MAX_EXPERTS);
  B200_CHECK_ARG(k >= 1 && k <= E && k <= B200MOE_MAX_TOPK, B200MOE_E_BAD_SHAPE, "router_topk_bwd: top_k = %d", k);
  if (T <= 0) return 0;
  cudaStream_t st = (cudaStream_t)stream;
  const int grid = grid_for_tokens(T);
  const long long* idx_ll = reinterpret_cast<const long long*>(idx);
  __nv_bfloat16* gl = reinterpret_cast<__nv_bfloat16*>(grad_logits);
  switch (input_kind) {
    case B200MOE_LOGITS_BF16:
      router_topk_bwd_kernel<B200MOE_LOGITS_BF16><<<grid, 256, 0, st>>>(logits, idx_ll, grad_w, T, E, k, norm_topk, scale, gl);
      break;
    case B200MOE_LOGITS_F32:
      router_topk_bwd_kernel<B200MOE_LOGITS_F32><<<grid, 256, 0, st>>>(logits, idx_ll, grad_w, T, E, k, norm_topk, scale, gl);
      break;
    default:
      set_error("router_topk_bwd: input_kind %d has no backward (logits are required)", input_kind);
      return B200MOE_E_UNSUPPORTED;
  }
  B200_CUDA(cudaGetLastError());
  return 0;
}

int b200moe_router_bias_update(float* bias, const int32_t* counts, int E, float u, b200moe_stream_t stream) {
  B200_CHECK_ARG(bias && counts, B200MOE_E_NULL, "router_bias_update: null pointer");
  B200_CHECK_ARG(E >= 1, B200MOE_E_BAD_SHAPE, "router_bias_update: E = %d", E);
  if (!(u > 0.0f)) return 0;
  router_bias_update_kernel<<<1, 256, 0, (cudaStream_t)stream>>>(bias, counts, E, u);
  B200_CUDA(cudaGetLastError());
  return 0;
}

int b200moe_splitk_reduce(const float* P, int64_t slices, int64_t elems, void* D, b200moe_stream_t stream) {
  B200_CHECK_ARG(P && D, B200MOE_E_NULL, "splitk_reduce: null pointer");
  B200_CHECK_ARG(slices >= 1 && elems > 0 && elems % 4 == 0, B200MOE_E_BAD_SHAPE,
                 "splitk_reduce: slices = %lld, elems = %lld (must be a multiple of 4)", (long long)slices,
                 (long long)elems);
  const long long threads = elems / 4;
  const int grid = static_cast<int>((threads + 255) / 256);
  splitk_reduce_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>(P, slices, elems, reinterpret_cast<__nv_bfloat16*>(D));
  B200_CUDA(cudaGetLastError());
  return 0;
}

}  // extern "C"
