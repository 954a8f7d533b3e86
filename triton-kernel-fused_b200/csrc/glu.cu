// PolyGLU activations with a per-expert activation code, as separate row kernels (the path used when
// an expert stack is not pure SiLU-GLU; the pure stack runs fused in the GEMM epilogues).
//   codes: 0 SiLU, 1 ReLU^2, 2 NormSiLU, 5 SiTU (gamma * tanh(alpha g) * sigmoid(g)), 6 NormReLU^2,
//          7 NormSiTU; the Norm codes first divide the gate row by rms = sqrt(mean(g^2) + 1e-6).
//   codes 3 (Identity) and 4 (Zero) are expert KINDS without weights: their rows are copied / zeroed.
// Semantics follow kernels/sm75/moe.py:163-232 (_glu_fwd_row_kernel, _glu_bwd_row_kernel) and
// :859-881 (_act_eager) of the reference; math in fp32, bf16 in and out.  One CTA per padded row.
#include <cuda_bf16.h>

#include "common.cuh"
#include "ptx.cuh"

namespace b200moe {

constexpr float kRmsEps = 1e-6f;   // _NS_EPS, kernels/sm75/moe.py:80

__device__ __forceinline__ float block_sum(float v, float* red) {
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) v += __shfl_xor_sync(0xffffffffu, v, off);
  __syncthreads();
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
  __syncthreads();
  float s = 0.0f;
  for (int i = 0; i < (blockDim.x >> 5); ++i) s += red[i];
  return s;
}

__device__ __forceinline__ float sigmoidf_(float x) { return 1.0f / (1.0f + expf(-x)); }
__device__ __forceinline__ float tanh_via_sigmoid(float x) { return 2.0f / (1.0f + expf(-2.0f * x)) - 1.0f; }
__device__ __forceinline__ bool is_norm(int code) { return code == 2 || code == 6 || code == 7; }

// activation value f(gn) (times gamma for SiTU) for the forward; gn = gate or gate / rms
__device__ __forceinline__ float act_value(int code, float gate, float gn, float alpha, float gamma) {
  const float sig = sigmoidf_(gn);
  if (code == 1 || code == 6) {
    const float r = fmaxf(gn, 0.0f);
    return r * r;
  }
  if (code == 5) return gamma * tanh_via_sigmoid(alpha * gate) * sig;
  if (code == 7) return tanh_via_sigmoid(gn) * sig;
  return gn * sig;   // codes 0 and 2
}

__global__ void __launch_bounds__(256)
glu_fwd_rows_kernel(const __nv_bfloat16* __restrict__ gate_up, const int* __restrict__ tile_expert,
                    const int* __restrict__ codes, const float* __restrict__ params, const int* __restrict__ total_rows,
                    int I, __nv_bfloat16* __restrict__ inter) {
  __shared__ float red[8];
  const int total = *total_rows;
  for (long long r = blockIdx.x; r < total; r += gridDim.x) {
    const int e = tile_expert[r / B200MOE_TILE_M];
    const int code = codes[e];
    const float alpha = (params != nullptr && code == 5) ? params[2 * e] : 1.0f;
    const float gamma = (params != nullptr && code == 5) ? params[2 * e + 1] : 1.0f;
    const __nv_bfloat16* g = gate_up + r * (2LL * I);
    const __nv_bfloat16* u = g + I;
    float inv_r = 1.0f;
    if (is_norm(code)) {
      float ss = 0.0f;
      for (int c = threadIdx.x; c < I; c += blockDim.x) {
        const float v = __bfloat162float(g[c]);
        ss += v * v;
      }
      ss = block_sum(ss, red);
      inv_r = 1.0f / sqrtf(ss / static_cast<float>(I) + kRmsEps);
    }
    for (int c = threadIdx.x; c < I; c += blockDim.x) {
      const float gate = __bfloat162float(g[c]);
      const float up = __bfloat162float(u[c]);
      inter[r * static_cast<long long>(I) + c] = __float2bfloat16_rn(act_value(code, gate, gate * inv_r, alpha, gamma) * up);
    }
  }
}

// grad_gate_up = [grad_gate | grad_up]; optional per-row d(alpha), d(gamma) for learnable SiTU.
__global__ void __launch_bounds__(256)
glu_bwd_rows_kernel(const __nv_bfloat16* __restrict__ grad_inter, const __nv_bfloat16* __restrict__ gate_up,
                    const int* __restrict__ tile_expert, const int* __restrict__ codes,
                    const float* __restrict__ params, const int* __restrict__ total_rows, int I,
                    __nv_bfloat16* __restrict__ grad_gate_up, float* __restrict__ row_da, float* __restrict__ row_dg) {
  __shared__ float red[8];
  const int total = *total_rows;
  for (long long r = blockIdx.x; r < total; r += gridDim.x) {
    const int e = tile_expert[r / B200MOE_TILE_M];
    const int code = codes[e];
    const float alpha = (params != nullptr && code == 5) ? params[2 * e] : 1.0f;
    const float gamma = (params != nullptr && code == 5) ? params[2 * e + 1] : 1.0f;
    const __nv_bfloat16* g = gate_up + r * (2LL * I);
    const __nv_bfloat16* u = g + I;
    const __nv_bfloat16* go = grad_inter + r * static_cast<long long>(I);
    __nv_bfloat16* gg = grad_gate_up + r * (2LL * I);
    const bool norm = is_norm(code);
    float rr = 1.0f, S = 0.0f;
    if (norm) {
      float ss = 0.0f;
      for (int c = threadIdx.x; c < I; c += blockDim.x) {
        const float v = __bfloat162float(g[c]);
        ss += v * v;
      }
      ss = block_sum(ss, red);
      rr = sqrtf(ss / static_cast<float>(I) + kRmsEps);
    }
    // derivative of the activation w.r.t. gn, and the activation itself
    auto deriv = [&](float gate, float gn, float& act) -> float {
      const float sig = sigmoidf_(gn);
      if (code == 1 || code == 6) {
        const float rl = fmaxf(gn, 0.0f);
        act = rl * rl;
        return 2.0f * rl;
      }
      if (code == 5) {
        const float t5 = tanh_via_sigmoid(alpha * gate);
        act = gamma * t5 * sig;
        return gamma * (alpha * (1.0f - t5 * t5) * sig + t5 * sig * (1.0f - sig));
      }
      if (code == 7) {
        const float tg = tanh_via_sigmoid(gn);
        act = tg * sig;
        return (1.0f - tg * tg) * sig + tg * sig * (1.0f - sig);
      }
      act = gn * sig;
      return sig * (1.0f + gn * (1.0f - sig));
    };
    if (norm) {   // RMS coupling term S = sum(go * up * f'(gn) * gn)
      float part = 0.0f;
      for (int c = threadIdx.x; c < I; c += blockDim.x) {
        const float gate = __bfloat162float(g[c]);
        const float gn = gate / rr;
        float act;
        const float d = deriv(gate, gn, act);
        part += __bfloat162float(go[c]) * __bfloat162float(u[c]) * d * gn;
      }
      S = block_sum(part, red);
    }
    float da = 0.0f, dg = 0.0f;
    for (int c = threadIdx.x; c < I; c += blockDim.x) {
      const float gate = __bfloat162float(g[c]);
      const float up = __bfloat162float(u[c]);
      const float gi = __bfloat162float(go[c]);
      const float gn = norm ? gate / rr : gate;
      float act;
      const float d = deriv(gate, gn, act);
      const float gu_ = gi * up;
      const float grad_gate = norm ? (gu_ * d - (S / static_cast<float>(I)) * gn) / rr : gu_ * d;
      gg[c] = __float2bfloat16_rn(grad_gate);
      gg[I + c] = __float2bfloat16_rn(gi * act);
      if (row_da != nullptr && code == 5) {
        const float sig = sigmoidf_(gate);
        const float t5 = tanh_via_sigmoid(alpha * gate);
        da += gu_ * gamma * gate * (1.0f - t5 * t5) * sig;
        dg += gu_ * t5 * sig;
      }
    }
    if (row_da != nullptr) {
      da = block_sum(da, red);
      dg = block_sum(dg, red);
      if (threadIdx.x == 0) {
        row_da[r] = da;
        row_dg[r] = dg;
      }
    }
  }
}

// out[e] = (sum of row_da over the rows of e, sum of row_dg): deterministic, one CTA per expert
__global__ void __launch_bounds__(256)
expert_row_sums_kernel(const float* __restrict__ row_da, const float* __restrict__ row_dg, const int* __restrict__ poffs,
                       float* __restrict__ out) {
  __shared__ float red[8];
  const int e = blockIdx.x;
  float a = 0.0f, b = 0.0f;
  for (int r = poffs[e] + threadIdx.x; r < poffs[e + 1]; r += blockDim.x) {
    a += row_da[r];
    b += row_dg[r];
  }
  a = block_sum(a, red);
  b = block_sum(b, red);
  if (threadIdx.x == 0) {
    out[2 * e] = a;
    out[2 * e + 1] = b;
  }
}

// rows of the special experts (those after the first `first_special` experts):
// dst[r] = src[r] for Identity (code 3), 0 otherwise (Zero, code 4)
__global__ void __launch_bounds__(256)
special_rows_kernel(const uint4* __restrict__ src, const int* __restrict__ tile_expert, const int* __restrict__ codes,
                    const int* __restrict__ poffs, int first_special, int num_experts, int vec_per_row,
                    uint4* __restrict__ dst) {
  const int r0 = poffs[first_special], r1 = poffs[num_experts];
  for (long long r = r0 + blockIdx.x; r < r1; r += gridDim.x) {
    const int code = codes[tile_expert[r / B200MOE_TILE_M]];
    for (int c = threadIdx.x; c < vec_per_row; c += blockDim.x)
      dst[r * vec_per_row + c] = (code == 3) ? src[r * vec_per_row + c] : make_uint4(0u, 0u, 0u, 0u);
  }
}

static int rows_grid(long long rows_cap) {
  long long g = rows_cap;
  const long long cap = static_cast<long long>(num_sms()) * 16;
  if (g > cap) g = cap;
  return static_cast<int>(g < 1 ? 1 : g);
}

}  // namespace b200moe

using namespace b200moe;

extern "C" {

int b200moe_glu_fwd_rows(const void* gate_up, const int32_t* tile_expert, const int32_t* act_codes,
                         const float* act_params, const int32_t* total_rows, int64_t rows_cap, int64_t I, void* inter,
                         b200moe_stream_t stream) {
  B200_CHECK_ARG(gate_up && tile_expert && act_codes && total_rows && inter, B200MOE_E_NULL, "glu_fwd_rows: null pointer");
  B200_CHECK_ARG(I > 0, B200MOE_E_BAD_SHAPE, "glu_fwd_rows: I = %lld", (long long)I);
  if (rows_cap <= 0) return 0;
  glu_fwd_rows_kernel<<<rows_grid(rows_cap), 256, 0, (cudaStream_t)stream>>>(
      reinterpret_cast<const __nv_bfloat16*>(gate_up), tile_expert, act_codes, act_params, total_rows, static_cast<int>(I),
      reinterpret_cast<__nv_bfloat16*>(inter));
  B200_CUDA(cudaGetLastError());
  return 0;
}

int b200moe_glu_bwd_rows(const void* grad_inter, const void* gate_up, const int32_t* tile_expert,
                         const int32_t* act_codes, const float* act_params, const int32_t* total_rows, int64_t rows_cap,
                         int64_t I, void* grad_gate_up, float* row_da, float* row_dg, b200moe_stream_t stream) {
  B200_CHECK_ARG(grad_inter && gate_up && tile_expert && act_codes && total_rows && grad_gate_up, B200MOE_E_NULL,
                 "glu_bwd_rows: null pointer");
  B200_CHECK_ARG((row_da == nullptr) == (row_dg == nullptr), B200MOE_E_NULL, "glu_bwd_rows: row_da and row_dg go together");
  B200_CHECK_ARG(I > 0, B200MOE_E_BAD_SHAPE, "glu_bwd_rows: I = %lld", (long long)I);
  if (rows_cap <= 0) return 0;
  glu_bwd_rows_kernel<<<rows_grid(rows_cap), 256, 0, (cudaStream_t)stream>>>(
      reinterpret_cast<const __nv_bfloat16*>(grad_inter), reinterpret_cast<const __nv_bfloat16*>(gate_up), tile_expert,
      act_codes, act_params, total_rows, static_cast<int>(I), reinterpret_cast<__nv_bfloat16*>(grad_gate_up), row_da, row_dg);
  B200_CUDA(cudaGetLastError());
  return 0;
}

int b200moe_expert_row_sums(const float* row_da, const float* row_dg, const int32_t* poffs, int E, float* out,
                            b200moe_stream_t stream) {
  B200_CHECK_ARG(row_da && row_dg && poffs && out, B200MOE_E_NULL, "expert_row_sums: null pointer");
  B200_CHECK_ARG(E >= 1, B200MOE_E_BAD_SHAPE, "expert_row_sums: E = %d", E);
  expert_row_sums_kernel<<<E, 256, 0, (cudaStream_t)stream>>>(row_da, row_dg, poffs, out);
  B200_CUDA(cudaGetLastError());
  return 0;
}

int b200moe_special_rows(const void* src, const int32_t* tile_expert, const int32_t* act_codes, const int32_t* poffs,
                         int first_special, int num_experts, int64_t H, int64_t rows_cap, void* dst,
                         b200moe_stream_t stream) {
  B200_CHECK_ARG(src && tile_expert && act_codes && poffs && dst, B200MOE_E_NULL, "special_rows: null pointer");
  B200_CHECK_ARG(H > 0 && H % 8 == 0 && first_special >= 0 && first_special <= num_experts, B200MOE_E_BAD_SHAPE,
                 "special_rows: H = %lld, first_special = %d, num_experts = %d", (long long)H, first_special, num_experts);
  B200_CHECK_ARG(aligned16(src) && aligned16(dst), B200MOE_E_ALIGN, "special_rows: pointers must be 16-byte aligned");
  if (rows_cap <= 0 || first_special == num_experts) return 0;
  special_rows_kernel<<<rows_grid(rows_cap), 256, 0, (cudaStream_t)stream>>>(
      reinterpret_cast<const uint4*>(src), tile_expert, act_codes, poffs, first_special, num_experts,
      static_cast<int>(H / 8), reinterpret_cast<uint4*>(dst));
  B200_CUDA(cudaGetLastError());
  return 0;
}

}  // extern "C"
