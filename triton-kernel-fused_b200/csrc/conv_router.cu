// Causal-conv router front end: the K-tap causal Conv1d(H -> E) of the reference's `fused_router`
// (kernels/sm75/router.py:172-218: F.conv1d(x^T, W, padding=K-1)[..., :S]) becomes ONE dense tcgen05
// GEMM over an unfolded operand:
//   xu[(b,s), j*H + h] = x[b, s-(K-1)+j, h]  (zero where the tap reaches before the sequence start)
//   logits = xu (B*S, K*H) @ Wf^T,  Wf[e, j*H + h] = W[e, h, j]
// and the backward folds grad_xu back: grad_x[b,s,h] = sum_j grad_xu[(b, s+(K-1)-j), j*H + h].
// Both kernels are pure copies / K-term sums over 16-byte vectors (HBM-bound).
#include <cuda_bf16.h>

#include "common.cuh"
#include "ptx.cuh"

namespace b200moe {

__global__ void __launch_bounds__(256)
conv_unfold_kernel(const uint4* __restrict__ x, long long B, long long S, int K, int vec_h, uint4* __restrict__ xu) {
  const long long rows = B * S;
  for (long long r = blockIdx.x; r < rows; r += gridDim.x) {
    const long long s = r % S;
    for (int c = threadIdx.x; c < K * vec_h; c += blockDim.x) {
      const int j = c / vec_h, v = c - j * vec_h;
      const long long sj = s - (K - 1) + j;
      xu[r * (static_cast<long long>(K) * vec_h) + c] =
          (sj >= 0) ? x[(r - s + sj) * vec_h + v] : make_uint4(0u, 0u, 0u, 0u);
    }
  }
}

__global__ void __launch_bounds__(256)
conv_fold_kernel(const uint4* __restrict__ gxu, long long B, long long S, int K, int vec_h, uint4* __restrict__ gx) {
  const long long rows = B * S;
  for (long long r = blockIdx.x; r < rows; r += gridDim.x) {
    const long long s = r % S;
    for (int v = threadIdx.x; v < vec_h; v += blockDim.x) {
      float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
      for (int j = 0; j < K; ++j) {
        const long long sr = s + (K - 1) - j;     // the output row that read x[b,s] through tap j
        if (sr < S) {
          const uint4 q = gxu[(r - s + sr) * (static_cast<long long>(K) * vec_h) + j * vec_h + v];
          const float2 a = unpack_bf16x2(q.x), b = unpack_bf16x2(q.y), c = unpack_bf16x2(q.z), d = unpack_bf16x2(q.w);
          acc[0] += a.x; acc[1] += a.y; acc[2] += b.x; acc[3] += b.y;
          acc[4] += c.x; acc[5] += c.y; acc[6] += d.x; acc[7] += d.y;
        }
      }
      uint4 o;
      o.x = pack_bf16x2(acc[0], acc[1]);
      o.y = pack_bf16x2(acc[2], acc[3]);
      o.z = pack_bf16x2(acc[4], acc[5]);
      o.w = pack_bf16x2(acc[6], acc[7]);
      gx[r * vec_h + v] = o;
    }
  }
}

}  // namespace b200moe

using namespace b200moe;

static int conv_check(const char* who, const void* a, const void* b, int64_t B, int64_t S, int64_t H, int K) {
  B200_CHECK_ARG(a && b, B200MOE_E_NULL, "%s: null pointer", who);
  B200_CHECK_ARG(B >= 1 && S >= 1 && H > 0 && H % 8 == 0 && K >= 1 && K <= 64, B200MOE_E_BAD_SHAPE,
                 "%s: B = %lld, S = %lld, H = %lld (multiple of 8), K = %d (1..64)", who, (long long)B, (long long)S,
                 (long long)H, K);
  B200_CHECK_ARG(aligned16(a) && aligned16(b), B200MOE_E_ALIGN, "%s: pointers must be 16-byte aligned", who);
  return 0;
}

extern "C" {

int b200moe_conv_unfold(const void* x, int64_t B, int64_t S, int64_t H, int K, void* xu, b200moe_stream_t stream) {
  int rc = conv_check("conv_unfold", x, xu, B, S, H, K);
  if (rc) return rc;
  long long grid = B * S;
  const long long cap = static_cast<long long>(num_sms()) * 16;
  if (grid > cap) grid = cap;
  conv_unfold_kernel<<<static_cast<int>(grid), 256, 0, (cudaStream_t)stream>>>(
      reinterpret_cast<const uint4*>(x), B, S, K, static_cast<int>(H / 8), reinterpret_cast<uint4*>(xu));
  B200_CUDA(cudaGetLastError());
  return 0;
}

int b200moe_conv_fold(const void* grad_xu, int64_t B, int64_t S, int64_t H, int K, void* grad_x,
                      b200moe_stream_t stream) {
  int rc = conv_check("conv_fold", grad_xu, grad_x, B, S, H, K);
  if (rc) return rc;
  long long grid = B * S;
  const long long cap = static_cast<long long>(num_sms()) * 16;
  if (grid > cap) grid = cap;
  conv_fold_kernel<<<static_cast<int>(grid), 256, 0, (cudaStream_t)stream>>>(
      reinterpret_cast<const uint4*>(grad_xu), B, S, K, static_cast<int>(H / 8), reinterpret_cast<uint4*>(grad_x));
  B200_CUDA(cudaGetLastError());
  return 0;
}

}  // extern "C"
