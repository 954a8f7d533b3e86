// Expert permutation as a stable counting sort on the device (no host sync):
//   1. hist : one warp per chunk of kChunk consecutive slots builds that chunk's per-expert histogram
//             (warp-aggregated: __match_any_sync groups equal experts, one shared-memory add per group)
//   2. scan : one CTA; thread e scans expert e over the chunks (exclusive, in place), then the CTA
//             scans counts -> compact offsets, padded offsets, tile table, pad-row markers
//   3. rank : one warp per chunk walks its slots in order; rank inside the expert = chunk base +
//             number of equal experts earlier in the chunk -> slot_row / row_slot / order
// Row r of expert e is therefore the r-th smallest slot index t*k+j with idx[t,j] == e, which is
// exactly what a stable sort of idx.flatten() gives.
#include "common.cuh"
#include "ptx.cuh"

namespace b200moe {

constexpr int kChunk = 512;          // slots per warp
constexpr int kWarpsPerBlock = 8;

__global__ void __launch_bounds__(kWarpsPerBlock * 32)
permute_hist_kernel(const long long* __restrict__ idx, long long M, int E, int* __restrict__ chunk_hist,
                    int* __restrict__ status) {
  extern __shared__ int sh[];  // kWarpsPerBlock * E
  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;
  int* h = sh + warp * E;
  const long long chunk = static_cast<long long>(blockIdx.x) * kWarpsPerBlock + warp;
  const long long nchunks = (M + kChunk - 1) / kChunk;
  if (chunk >= nchunks) return;
  for (int e = lane; e < E; e += 32) h[e] = 0;
  __syncwarp();
  const long long s0 = chunk * kChunk;
  for (int i = 0; i < kChunk; i += 32) {
    const long long s = s0 + i + lane;
    int e = -1;
    if (s < M) {
      const long long v = idx[s];
      if (v >= 0 && v < E) e = static_cast<int>(v);
      else atomicCAS(status, 0, ST_BAD_EXPERT_INDEX);
    }
    const unsigned peers = __match_any_sync(0xffffffffu, e);
    if (e >= 0 && (peers & ((1u << lane) - 1)) == 0) h[e] += __popc(peers);  // group leader
    __syncwarp();
  }
  for (int e = lane; e < E; e += 32) chunk_hist[chunk * E + e] = h[e];
}

__global__ void __launch_bounds__(B200MOE_MAX_EXPERTS)
permute_scan_kernel(int* __restrict__ chunk_hist, long long nchunks, int E, int* __restrict__ counts,
                    int* __restrict__ offs, int* __restrict__ poffs, int* __restrict__ row_slot,
                    int* __restrict__ tile_expert) {
  __shared__ int s_cnt[B200MOE_MAX_EXPERTS + 1];
  __shared__ int s_pad[B200MOE_MAX_EXPERTS + 1];
  const int e = threadIdx.x;
  int running = 0;
  if (e < E) {
    constexpr int B = 16;
    for (long long c0 = 0; c0 < nchunks; c0 += B) {
      int v[B];
#pragma unroll
      for (int i = 0; i < B; ++i) v[i] = (c0 + i < nchunks) ? chunk_hist[(c0 + i) * E + e] : 0;
#pragma unroll
      for (int i = 0; i < B; ++i) {
        if (c0 + i < nchunks) chunk_hist[(c0 + i) * E + e] = running;
        running += v[i];
      }
    }
    counts[e] = running;
    s_cnt[e] = running;
    s_pad[e] = ((running + B200MOE_TILE_M - 1) / B200MOE_TILE_M) * B200MOE_TILE_M;
  }
  __syncthreads();
  if (threadIdx.x == 0) {  // E <= 256: a serial scan is a few hundred cycles
    int a = 0, b = 0;
    for (int i = 0; i < E; ++i) {
      const int c = s_cnt[i], p = s_pad[i];
      s_cnt[i] = a;
      s_pad[i] = b;
      a += c;
      b += p;
    }
    s_cnt[E] = a;
    s_pad[E] = b;
  }
  __syncthreads();
  if (e < E) {
    offs[e] = s_cnt[e];
    poffs[e] = s_pad[e];
  }
  if (e == 0) {
    offs[E] = s_cnt[E];
    poffs[E] = s_pad[E];
  }
  if (e < E) {
    const int p0 = s_pad[e], p1 = s_pad[e + 1];
    for (int r = p0 + running; r < p1; ++r) row_slot[r] = -1;  // pad rows of this expert
    for (int t = p0 / B200MOE_TILE_M; t < p1 / B200MOE_TILE_M; ++t) tile_expert[t] = e;
  }
}

__global__ void __launch_bounds__(kWarpsPerBlock * 32)
permute_rank_kernel(const long long* __restrict__ idx, long long M, int E, const int* __restrict__ chunk_hist,
                    const int* __restrict__ offs, const int* __restrict__ poffs, int* __restrict__ slot_row,
                    int* __restrict__ row_slot, int* __restrict__ order, int* __restrict__ slot_pos) {
  extern __shared__ int sh[];
  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;
  int* base = sh + warp * E;
  const long long chunk = static_cast<long long>(blockIdx.x) * kWarpsPerBlock + warp;
  const long long nchunks = (M + kChunk - 1) / kChunk;
  if (chunk >= nchunks) return;
  for (int e = lane; e < E; e += 32) base[e] = chunk_hist[chunk * E + e];
  __syncwarp();
  const long long s0 = chunk * kChunk;
  for (int i = 0; i < kChunk; i += 32) {
    const long long s = s0 + i + lane;
    int e = -1;
    if (s < M) {
      const long long v = idx[s];
      if (v >= 0 && v < E) e = static_cast<int>(v);
    }
    const unsigned peers = __match_any_sync(0xffffffffu, e);
    int rank = 0;
    if (e >= 0) rank = base[e] + __popc(peers & ((1u << lane) - 1));
    __syncwarp();
    if (e >= 0 && (peers & ((1u << lane) - 1)) == 0) base[e] += __popc(peers);
    __syncwarp();
    if (e >= 0) {
      const int prow = poffs[e] + rank;
      slot_row[s] = prow;
      row_slot[prow] = static_cast<int>(s);
      if (order != nullptr) order[offs[e] + rank] = static_cast<int>(s);
      if (slot_pos != nullptr) slot_pos[s] = offs[e] + rank;
    } else if (s < M) {
      // an expert index outside [0, E) (the hist pass raised the status word): the slot owns no row.  -1 makes the
      // consumers of these tables skip it instead of following whatever the buffer held.
      slot_row[s] = -1;
      if (slot_pos != nullptr) slot_pos[s] = -1;
    }
  }
}

// x_s[r] = x[row_slot[r] / k] (16-byte vectors), zero rows for pads; rows >= *total_rows untouched
__global__ void __launch_bounds__(256)
gather_rows_kernel(const uint4* __restrict__ x, const int* __restrict__ row_slot,
                   const int* __restrict__ total_rows, int k, int vec_per_row, uint4* __restrict__ x_s) {
  const int total = *total_rows;
  for (long long r = blockIdx.x; r < total; r += gridDim.x) {
    const int slot = row_slot[r];
    uint4* dst = x_s + r * vec_per_row;
    if (slot < 0) {
      for (int c = threadIdx.x; c < vec_per_row; c += blockDim.x) dst[c] = make_uint4(0u, 0u, 0u, 0u);
    } else {
      const uint4* src = x + static_cast<long long>(slot / k) * vec_per_row;
      for (int c = threadIdx.x; c < vec_per_row; c += blockDim.x) dst[c] = src[c];
    }
  }
}

}  // namespace b200moe

using namespace b200moe;

extern "C" {

int64_t b200moe_padded_rows_cap(int64_t M, int E) {
  if (M < 0 || E < 1) return 0;
  return ((M + B200MOE_TILE_M - 1) / B200MOE_TILE_M + E) * B200MOE_TILE_M;
}

size_t b200moe_permute_ws_bytes(int64_t M, int E) {
  if (M < 0 || E < 1) return 0;
  const int64_t nchunks = (M + kChunk - 1) / kChunk;
  return static_cast<size_t>((nchunks > 0 ? nchunks : 1) * E) * sizeof(int32_t);
}

int b200moe_permute_build(const int64_t* idx, int64_t T, int k, int E, int32_t* counts, int32_t* offs,
                          int32_t* poffs, int32_t* slot_row, int32_t* row_slot, int32_t* tile_expert,
                          int32_t* order, int32_t* slot_pos, void* ws, size_t ws_bytes, int32_t* status,
                          b200moe_stream_t stream) {
  B200_CHECK_ARG(idx && counts && offs && poffs && slot_row && row_slot && tile_expert && ws && status,
                 B200MOE_E_NULL, "permute_build: null pointer");
  B200_CHECK_ARG(E >= 1 && E <= B200MOE_MAX_EXPERTS, B200MOE_E_UNSUPPORTED,
                 "permute_build: E = %d, supported 1..%d", E, B200MOE_MAX_EXPERTS);
  B200_CHECK_ARG(T >= 0 && k >= 1 && k <= B200MOE_MAX_TOPK, B200MOE_E_BAD_SHAPE,
                 "permute_build: T = %lld, k = %d", (long long)T, k);
  const int64_t M = T * k;
  B200_CHECK_ARG(b200moe_padded_rows_cap(M, E) < (1LL << 31), B200MOE_E_BAD_SHAPE,
                 "permute_build: %lld routed rows do not fit int32 tables", (long long)M);
  B200_CHECK_ARG(ws_bytes >= b200moe_permute_ws_bytes(M, E), B200MOE_E_WS_TOO_SMALL,
                 "permute_build: workspace %zu < %zu bytes", ws_bytes, b200moe_permute_ws_bytes(M, E));
  cudaStream_t st = (cudaStream_t)stream;
  const long long nchunks = (M + kChunk - 1) / kChunk;
  const int blocks = static_cast<int>((nchunks + kWarpsPerBlock - 1) / kWarpsPerBlock);
  const size_t shm = sizeof(int) * kWarpsPerBlock * E;
  int* hist = reinterpret_cast<int*>(ws);
  const long long* idx_ll = reinterpret_cast<const long long*>(idx);
  if (blocks > 0) {
    permute_hist_kernel<<<blocks, kWarpsPerBlock * 32, shm, st>>>(idx_ll, M, E, hist, status);
    B200_CUDA(cudaGetLastError());
  }
  permute_scan_kernel<<<1, B200MOE_MAX_EXPERTS, 0, st>>>(hist, nchunks, E, counts, offs, poffs, row_slot, tile_expert);
  B200_CUDA(cudaGetLastError());
  if (blocks > 0) {
    permute_rank_kernel<<<blocks, kWarpsPerBlock * 32, shm, st>>>(idx_ll, M, E, hist, offs, poffs, slot_row, row_slot,
                                                                   order, slot_pos);
    B200_CUDA(cudaGetLastError());
  }
  return 0;
}

int b200moe_gather_rows(const void* x, const int32_t* row_slot, const int32_t* total_rows, int k, int64_t H,
                        int64_t rows_cap, void* x_s, b200moe_stream_t stream) {
  B200_CHECK_ARG(x && row_slot && total_rows && x_s, B200MOE_E_NULL, "gather_rows: null pointer");
  B200_CHECK_ARG(H > 0 && H % 8 == 0, B200MOE_E_BAD_SHAPE, "gather_rows: H = %lld must be a multiple of 8", (long long)H);
  B200_CHECK_ARG(k >= 1, B200MOE_E_BAD_SHAPE, "gather_rows: k = %d", k);
  B200_CHECK_ARG(aligned16(x) && aligned16(x_s), B200MOE_E_ALIGN, "gather_rows: pointers must be 16-byte aligned");
  if (rows_cap <= 0) return 0;
  long long grid = rows_cap;
  const long long cap = static_cast<long long>(num_sms()) * 16;
  if (grid > cap) grid = cap;
  gather_rows_kernel<<<static_cast<int>(grid), 256, 0, (cudaStream_t)stream>>>(
      reinterpret_cast<const uint4*>(x), row_slot, total_rows, k, static_cast<int>(H / 8),
      reinterpret_cast<uint4*>(x_s));
  B200_CUDA(cudaGetLastError());
  return 0;
}

}  // extern "C"
