// Expert-parallel exchange kernels over peer memory (NVLink): every transfer is a plain load from a
// peer GPU's buffer (pointers of a symmetric allocation), fused with the gather / combine it feeds,
// so rows cross NVLink once and no staging copy or library collective touches the payload.
//
//   ep_plan             from the all-gathered (W,E) count matrix: this rank's padded expert segments,
//                       where each source rank's block starts inside them, and where this rank's own
//                       blocks start on their owners
//   ep_gather_pull      owner side, forward: x_s[row] = x of the source rank's token, zero pad rows
//   ep_combine_pull     home side: out[t] = sum_j w * rows of the owners (forward combine, and the
//                       grad_hidden un-permute with w = 1, plus the grad of the routing weights)
//   ep_combine_bwd_pull owner side, backward: grad_eo[row] = w * grad_out of the source's token
// Kernels only READ peer memory; each phase is separated from the next by a cross-rank barrier
// that the host side issues (the kernels themselves never wait on a peer).
#include <cuda_bf16.h>

#include "common.cuh"
#include "ptx.cuh"

namespace b200moe {

constexpr int kMaxRanks = 16;

struct PeerPtrs {
  const void* p[kMaxRanks];
};

// One CTA, one thread per global expert (E <= 256).
__global__ void __launch_bounds__(B200MOE_MAX_EXPERTS)
ep_plan_kernel(const int* __restrict__ counts_all, int W, int rank, int E, int* __restrict__ poffs_l,
               int* __restrict__ counts_l, int* __restrict__ tile_expert_l, int* __restrict__ src_base,
               int* __restrict__ dest_base) {
  __shared__ int s_tot[B200MOE_MAX_EXPERTS];
  __shared__ int s_start[B200MOE_MAX_EXPERTS + 1];   // padded start of expert e inside its owner
  const int e = threadIdx.x;
  const int El = E / W;
  int before_me = 0;
  if (e < E) {
    int tot = 0;
    for (int s = 0; s < W; ++s) {
      const int c = counts_all[s * E + e];
      if (s < rank) before_me += c;
      tot += c;
    }
    s_tot[e] = tot;
  }
  __syncthreads();
  if (e < W) {   // thread d scans the experts of owner d
    int run = 0;
    for (int j = 0; j < El; ++j) {
      const int g = e * El + j;
      s_start[g] = run;
      run += ((s_tot[g] + B200MOE_TILE_M - 1) / B200MOE_TILE_M) * B200MOE_TILE_M;
    }
    if (e == rank) poffs_l[El] = run;
  }
  __syncthreads();
  if (e < E) {
    dest_base[e] = s_start[e] + before_me;
    if (e / El == rank) {
      const int j = e - rank * El;
      const int p0 = s_start[e];
      const int p1 = p0 + ((s_tot[e] + B200MOE_TILE_M - 1) / B200MOE_TILE_M) * B200MOE_TILE_M;
      poffs_l[j] = p0;
      counts_l[j] = s_tot[e];
      int run = p0;
      for (int s = 0; s < W; ++s) {
        src_base[s * El + j] = run;
        run += counts_all[s * E + e];
      }
      for (int t = p0 / B200MOE_TILE_M; t < p1 / B200MOE_TILE_M; ++t) tile_expert_l[t] = j;
    }
  }
}

// One warp per padded row of this rank.
__global__ void __launch_bounds__(256)
ep_gather_pull_kernel(PeerPtrs x_peers, PeerPtrs order_peers, PeerPtrs offs_peers, const int* __restrict__ counts_l,
                      const int* __restrict__ poffs_l, const int* __restrict__ tile_expert_l,
                      const int* __restrict__ src_base, int W, int rank, int El, int k, int vec_per_row,
                      uint4* __restrict__ x_s, int* __restrict__ row_src, int* __restrict__ row_slot_src) {
  const int lane = threadIdx.x & 31;
  const long long warp0 = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  const long long nwarps = (static_cast<long long>(gridDim.x) * blockDim.x) >> 5;
  const int total = poffs_l[El];
  for (long long r = warp0; r < total; r += nwarps) {
    int src = -1, slot = 0;
    if (lane == 0) {
      const int j = tile_expert_l[r / B200MOE_TILE_M];
      const int i = static_cast<int>(r) - poffs_l[j];
      if (i < counts_l[j]) {
        int s = 0;
        while (s + 1 < W && src_base[(s + 1) * El + j] <= static_cast<int>(r)) ++s;
        // skip sources whose block is empty: the largest s with src_base <= r is the owner of r
        const int within = static_cast<int>(r) - src_base[s * El + j];
        const int* offs_s = reinterpret_cast<const int*>(offs_peers.p[s]);
        const int* order_s = reinterpret_cast<const int*>(order_peers.p[s]);
        const int e = rank * El + j;
        slot = order_s[offs_s[e] + within];
        src = s;
      }
    }
    src = __shfl_sync(0xffffffffu, src, 0);
    slot = __shfl_sync(0xffffffffu, slot, 0);
    uint4* dst = x_s + r * vec_per_row;
    if (src < 0) {
      for (int c = lane; c < vec_per_row; c += 32) dst[c] = make_uint4(0u, 0u, 0u, 0u);
    } else {
      const uint4* srow = reinterpret_cast<const uint4*>(x_peers.p[src]) + static_cast<long long>(slot / k) * vec_per_row;
      // peer loads have microseconds of latency: keep 8 of them in flight per lane
      for (int c0 = lane; c0 < vec_per_row; c0 += 32 * 8) {
        uint4 v[8];
#pragma unroll
        for (int i = 0; i < 8; ++i)
          if (c0 + 32 * i < vec_per_row) v[i] = srow[c0 + 32 * i];
#pragma unroll
        for (int i = 0; i < 8; ++i)
          if (c0 + 32 * i < vec_per_row) dst[c0 + 32 * i] = v[i];
      }
    }
    if (lane == 0) {
      row_src[r] = src;
      row_slot_src[r] = slot;
    }
  }
}

__device__ __forceinline__ void fma8(float (&acc)[8], const uint4& v, float w) {
  const float2 a = unpack_bf16x2(v.x), b = unpack_bf16x2(v.y), c = unpack_bf16x2(v.z), d = unpack_bf16x2(v.w);
  acc[0] += w * a.x; acc[1] += w * a.y; acc[2] += w * b.x; acc[3] += w * b.y;
  acc[4] += w * c.x; acc[5] += w * c.y; acc[6] += w * d.x; acc[7] += w * d.y;
}

// One CTA per token: out[t] = sum_j w[t,j] * rows_peer[owner(e_j)][dest_base[e_j] + slot_pos - offs[e_j]]
__global__ void __launch_bounds__(256)
ep_combine_pull_kernel(PeerPtrs rows_peers, const float* __restrict__ w, const long long* __restrict__ idx,
                       const int* __restrict__ slot_pos, const int* __restrict__ offs,
                       const int* __restrict__ dest_base, int El, long long T, int k, int vec_per_row,
                       uint4* __restrict__ out, PeerPtrs gw_peers, float* __restrict__ grad_w) {
  __shared__ int s_row[B200MOE_MAX_TOPK];
  __shared__ int s_owner[B200MOE_MAX_TOPK];
  __shared__ float s_w[B200MOE_MAX_TOPK];
  for (long long t = blockIdx.x; t < T; t += gridDim.x) {
    __syncthreads();
    if (threadIdx.x < k) {
      const long long s = t * k + threadIdx.x;
      const int e = static_cast<int>(idx[s]);
      const int row = dest_base[e] + slot_pos[s] - offs[e];
      const int owner = e / El;
      s_row[threadIdx.x] = row;
      s_owner[threadIdx.x] = owner;
      s_w[threadIdx.x] = (w != nullptr) ? w[s] : 1.0f;
      if (grad_w != nullptr) grad_w[s] = reinterpret_cast<const float*>(gw_peers.p[owner])[row];
    }
    __syncthreads();
    for (int c = threadIdx.x; c < vec_per_row; c += blockDim.x) {
      float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
      for (int j0 = 0; j0 < k; j0 += 8) {      // up to 8 peer loads in flight, summed in slot order
        uint4 v[8];
#pragma unroll
        for (int i = 0; i < 8; ++i)
          if (j0 + i < k)
            v[i] = reinterpret_cast<const uint4*>(rows_peers.p[s_owner[j0 + i]])[static_cast<long long>(s_row[j0 + i]) * vec_per_row + c];
#pragma unroll
        for (int i = 0; i < 8; ++i)
          if (j0 + i < k) fma8(acc, v[i], s_w[j0 + i]);
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

// One warp per padded row of this rank: grad_eo[r] = go_peer[src][slot/k] * w_peer[src][slot];
// gw_rows[r] = <go, eo[r]> (fp32); zero rows for pads.
__global__ void __launch_bounds__(256)
ep_combine_bwd_pull_kernel(PeerPtrs go_peers, PeerPtrs w_peers, const uint4* __restrict__ eo,
                           const int* __restrict__ row_src, const int* __restrict__ row_slot_src,
                           const int* __restrict__ total_rows, int k, int vec_per_row, uint4* __restrict__ grad_eo,
                           float* __restrict__ gw_rows) {
  const int lane = threadIdx.x & 31;
  const long long warp0 = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  const long long nwarps = (static_cast<long long>(gridDim.x) * blockDim.x) >> 5;
  const int total = *total_rows;
  for (long long r = warp0; r < total; r += nwarps) {
    const int src = row_src[r];
    uint4* dst = grad_eo + r * vec_per_row;
    if (src < 0) {
      for (int c = lane; c < vec_per_row; c += 32) dst[c] = make_uint4(0u, 0u, 0u, 0u);
      if (lane == 0) gw_rows[r] = 0.0f;
      continue;
    }
    const int slot = row_slot_src[r];
    const float wt = reinterpret_cast<const float*>(w_peers.p[src])[slot];
    const uint4* g = reinterpret_cast<const uint4*>(go_peers.p[src]) + static_cast<long long>(slot / k) * vec_per_row;
    const uint4* e = eo + r * vec_per_row;
    float dot = 0.0f;
    for (int c0 = lane; c0 < vec_per_row; c0 += 32 * 8) {
      uint4 gv[8], ev[8];
#pragma unroll
      for (int i = 0; i < 8; ++i)
        if (c0 + 32 * i < vec_per_row) {
          gv[i] = g[c0 + 32 * i];
          ev[i] = e[c0 + 32 * i];
        }
#pragma unroll
      for (int i = 0; i < 8; ++i)
        if (c0 + 32 * i < vec_per_row) {
          const float2 g0 = unpack_bf16x2(gv[i].x), g1 = unpack_bf16x2(gv[i].y), g2 = unpack_bf16x2(gv[i].z), g3 = unpack_bf16x2(gv[i].w);
          const float2 e0 = unpack_bf16x2(ev[i].x), e1 = unpack_bf16x2(ev[i].y), e2 = unpack_bf16x2(ev[i].z), e3 = unpack_bf16x2(ev[i].w);
          dot += g0.x * e0.x + g0.y * e0.y + g1.x * e1.x + g1.y * e1.y + g2.x * e2.x + g2.y * e2.y + g3.x * e3.x + g3.y * e3.y;
          uint4 o;
          o.x = pack_bf16x2(g0.x * wt, g0.y * wt);
          o.y = pack_bf16x2(g1.x * wt, g1.y * wt);
          o.z = pack_bf16x2(g2.x * wt, g2.y * wt);
          o.w = pack_bf16x2(g3.x * wt, g3.y * wt);
          dst[c0 + 32 * i] = o;
        }
    }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, off);
    if (lane == 0) gw_rows[r] = dot;
  }
}

static int load_peers(PeerPtrs* out, const void* const* host_ptrs, int W, const char* who) {
  B200_CHECK_ARG(host_ptrs != nullptr, B200MOE_E_NULL, "%s: null peer pointer table", who);
  for (int i = 0; i < kMaxRanks; ++i) out->p[i] = nullptr;
  for (int i = 0; i < W; ++i) {
    B200_CHECK_ARG(host_ptrs[i] != nullptr && aligned16(host_ptrs[i]), B200MOE_E_ALIGN,
                   "%s: peer pointer %d is null or not 16-byte aligned", who, i);
    out->p[i] = host_ptrs[i];
  }
  return 0;
}

static int grid_rows(long long rows, int per_sm) {
  long long g = rows;
  const long long cap = static_cast<long long>(num_sms()) * per_sm;
  if (g > cap) g = cap;
  return static_cast<int>(g < 1 ? 1 : g);
}

}  // namespace b200moe

using namespace b200moe;

#define CHECK_WORLD(who)                                                                                        \
  B200_CHECK_ARG(W >= 1 && W <= kMaxRanks && rank >= 0 && rank < W, B200MOE_E_BAD_SHAPE, who ": W = %d, rank = %d", \
                 W, rank)

extern "C" {

int b200moe_ep_plan(const int32_t* counts_all, int W, int rank, int E, int32_t* poffs_l, int32_t* counts_l,
                    int32_t* tile_expert_l, int32_t* src_base, int32_t* dest_base, b200moe_stream_t stream) {
  B200_CHECK_ARG(counts_all && poffs_l && counts_l && tile_expert_l && src_base && dest_base, B200MOE_E_NULL,
                 "ep_plan: null pointer");
  CHECK_WORLD("ep_plan");
  B200_CHECK_ARG(E >= W && E <= B200MOE_MAX_EXPERTS && E % W == 0, B200MOE_E_BAD_SHAPE,
                 "ep_plan: E = %d must be a multiple of W = %d and at most %d", E, W, B200MOE_MAX_EXPERTS);
  ep_plan_kernel<<<1, B200MOE_MAX_EXPERTS, 0, (cudaStream_t)stream>>>(counts_all, W, rank, E, poffs_l, counts_l,
                                                                       tile_expert_l, src_base, dest_base);
  B200_CUDA(cudaGetLastError());
  return 0;
}

int b200moe_ep_gather_pull(const void* const* x_peers, const void* const* order_peers, const void* const* offs_peers,
                           const int32_t* counts_l, const int32_t* poffs_l, const int32_t* tile_expert_l,
                           const int32_t* src_base, int W, int rank, int E, int k, int64_t H, int64_t rows_cap,
                           void* x_s, int32_t* row_src, int32_t* row_slot_src, b200moe_stream_t stream) {
  B200_CHECK_ARG(counts_l && poffs_l && tile_expert_l && src_base && x_s && row_src && row_slot_src, B200MOE_E_NULL,
                 "ep_gather_pull: null pointer");
  CHECK_WORLD("ep_gather_pull");
  B200_CHECK_ARG(H > 0 && H % 8 == 0 && k >= 1 && E % W == 0, B200MOE_E_BAD_SHAPE, "ep_gather_pull: H = %lld, k = %d",
                 (long long)H, k);
  PeerPtrs xp, op, fp;
  int rc = load_peers(&xp, x_peers, W, "ep_gather_pull(x)");
  if (rc) return rc;
  rc = load_peers(&op, order_peers, W, "ep_gather_pull(order)");
  if (rc) return rc;
  rc = load_peers(&fp, offs_peers, W, "ep_gather_pull(offs)");
  if (rc) return rc;
  if (rows_cap <= 0) return 0;
  ep_gather_pull_kernel<<<grid_rows((rows_cap + 7) / 8, 8), 256, 0, (cudaStream_t)stream>>>(
      xp, op, fp, counts_l, poffs_l, tile_expert_l, src_base, W, rank, E / W, k, static_cast<int>(H / 8),
      reinterpret_cast<uint4*>(x_s), row_src, row_slot_src);
  B200_CUDA(cudaGetLastError());
  return 0;
}

int b200moe_ep_combine_pull(const void* const* rows_peers, const float* w, const int64_t* idx, const int32_t* slot_pos,
                            const int32_t* offs, const int32_t* dest_base, int W, int E, int64_t T, int k, int64_t H,
                            void* out, const void* const* gw_peers, float* grad_w, b200moe_stream_t stream) {
  B200_CHECK_ARG(idx && slot_pos && offs && dest_base && out, B200MOE_E_NULL, "ep_combine_pull: null pointer");
  const int rank = 0;
  CHECK_WORLD("ep_combine_pull");
  B200_CHECK_ARG(H > 0 && H % 8 == 0 && k >= 1 && k <= B200MOE_MAX_TOPK && E % W == 0, B200MOE_E_BAD_SHAPE,
                 "ep_combine_pull: H = %lld, k = %d", (long long)H, k);
  B200_CHECK_ARG((gw_peers == nullptr) == (grad_w == nullptr), B200MOE_E_NULL,
                 "ep_combine_pull: gw_peers and grad_w go together");
  PeerPtrs rp, gp;
  int rc = load_peers(&rp, rows_peers, W, "ep_combine_pull(rows)");
  if (rc) return rc;
  for (int i = 0; i < kMaxRanks; ++i) gp.p[i] = nullptr;
  if (gw_peers != nullptr) {
    rc = load_peers(&gp, gw_peers, W, "ep_combine_pull(grad_w rows)");
    if (rc) return rc;
  }
  if (T <= 0) return 0;
  ep_combine_pull_kernel<<<grid_rows(T, 16), 256, 0, (cudaStream_t)stream>>>(
      rp, w, reinterpret_cast<const long long*>(idx), slot_pos, offs, dest_base, E / W, T, k, static_cast<int>(H / 8),
      reinterpret_cast<uint4*>(out), gp, grad_w);
  B200_CUDA(cudaGetLastError());
  return 0;
}

int b200moe_ep_combine_bwd_pull(const void* const* go_peers, const void* const* w_peers, const void* eo,
                                const int32_t* row_src, const int32_t* row_slot_src, const int32_t* total_rows, int W,
                                int k, int64_t H, int64_t rows_cap, void* grad_eo, float* gw_rows,
                                b200moe_stream_t stream) {
  B200_CHECK_ARG(eo && row_src && row_slot_src && total_rows && grad_eo && gw_rows, B200MOE_E_NULL,
                 "ep_combine_bwd_pull: null pointer");
  const int rank = 0;
  CHECK_WORLD("ep_combine_bwd_pull");
  B200_CHECK_ARG(H > 0 && H % 8 == 0 && k >= 1, B200MOE_E_BAD_SHAPE, "ep_combine_bwd_pull: H = %lld, k = %d",
                 (long long)H, k);
  PeerPtrs gp, wp;
  int rc = load_peers(&gp, go_peers, W, "ep_combine_bwd_pull(grad_out)");
  if (rc) return rc;
  rc = load_peers(&wp, w_peers, W, "ep_combine_bwd_pull(weights)");
  if (rc) return rc;
  if (rows_cap <= 0) return 0;
  ep_combine_bwd_pull_kernel<<<grid_rows((rows_cap + 7) / 8, 8), 256, 0, (cudaStream_t)stream>>>(
      gp, wp, reinterpret_cast<const uint4*>(eo), row_src, row_slot_src, total_rows, k, static_cast<int>(H / 8),
      reinterpret_cast<uint4*>(grad_eo), gw_rows);
  B200_CUDA(cudaGetLastError());
  return 0;
}

}  // extern "C"
