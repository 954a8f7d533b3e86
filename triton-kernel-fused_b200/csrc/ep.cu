// Expert-parallel exchange kernels over peer memory (NVLink): every transfer is a plain load from a
// peer GPU's buffer (pointers of a symmetric allocation), fused with the gather / combine it feeds,
// so rows cross NVLink once and no staging copy or library collective touches the payload.
//
//   ep_plan             from the all-gathered (W,E) count matrix: this rank's padded expert segments,
//                       where each source rank's block starts inside them, and where this rank's own
//                       blocks start on their owners
//   ep_gather_pull      owner side, forward: x_s[row] = x of the source rank's token, zero pad rows; a token
//                       routed to several experts of this rank crosses NVLink once and is written to all
//                       of its rows
//   ep_combine_pull     home side: out[t] = sum_j w * rows of the owners (forward combine, and the
//                       grad_hidden un-permute with w = 1, plus the grad of the routing weights)
//   ep_combine_bwd_pull owner side, backward: grad_eo[row] = w * grad_out of the source's token (again one
//                       transfer per token and owner), gw[row] = <grad_out, eo[row]>
// Kernels only READ peer memory; each phase is separated from the next by a cross-rank barrier
// that the host side issues (the kernels themselves never wait on a peer).
#include <cuda_bf16.h>

#include <mutex>

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
               int* __restrict__ dest_base, long long rows_cap, int* __restrict__ status) {
  __shared__ int s_tot[B200MOE_MAX_EXPERTS];
  __shared__ int s_start[B200MOE_MAX_EXPERTS + 1];   // padded start of expert e inside its owner
  __shared__ int s_over;                             // some owner's padded rows exceed rows_cap (same answer on every rank)
  if (threadIdx.x == 0) s_over = 0;
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
    if (rows_cap > 0 && run > rows_cap) s_over = 1;
  }
  __syncthreads();
  if (s_over != 0) {
    // Fixed-capacity buffers (no host read of the row count) and a routing decision that does not fit on some rank.
    // Every rank sees the same count matrix and takes this branch together: the step computes nothing (no segment has
    // rows, no source has a block: the pull kernels skip negative rows) and the status word reports it.
    if (e <= El) poffs_l[e] = 0;
    if (e < El) counts_l[e] = 0;
    if (e < W * El) src_base[e] = -(1 << 30);
    if (e < E) dest_base[e] = 0;
    if (e == 0 && status != nullptr) atomicCAS(status, 0, ST_EP_CAPACITY);
    return;
  }
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

// Rows that arrive on this rank, stored straight into pinned host memory: host_words[0] = the sum of every source's
// counts for the local experts, host_words[1 + j] = the padded row at which local expert j ENDS (the padded offsets
// b200moe_ep_plan computes on the device).  The host learns how large its buffers must be, and where a group of
// experts starts, by waiting for this kernel, without a device-to-host copy that would queue behind whatever
// transfer the copy engines are busy with.
__global__ void __launch_bounds__(B200MOE_MAX_EXPERTS)
ep_local_rows_kernel(const int* __restrict__ counts_all, int W, int rank, int E, volatile int* __restrict__ host_words) {
  __shared__ int s_cnt[B200MOE_MAX_EXPERTS];
  const int El = E / W;
  const int j = threadIdx.x;
  int v = 0;
  if (j < El)
    for (int s = 0; s < W; ++s) v += counts_all[s * E + rank * El + j];
  s_cnt[j] = v;
  __syncthreads();
  if (j < El) {   // El <= 256 terms per thread: not worth a scan
    int end = 0;
    for (int i = 0; i <= j; ++i) end += ((s_cnt[i] + B200MOE_TILE_M - 1) / B200MOE_TILE_M) * B200MOE_TILE_M;
    host_words[1 + j] = end;
  }
  if (j == 0) {
    int tot = 0;
    for (int i = 0; i < El; ++i) tot += s_cnt[i];
    host_words[0] = tot;
  }
  __threadfence_system();
}

// Every rank sends its routing tables (expert index, position inside the expert segment and routing weight of each
// slot; the segment offsets) to all ranks, itself included, with plain stores into slot `rank` of the replica arrays
// in the receivers' symmetric buffers.  The pull kernels then resolve (source rank, token) -> local row from LOCAL
// memory: the only peer reads left on their path are the payload rows.  1.5 MB per peer at 98 304 slots.
__global__ void __launch_bounds__(256)
ep_publish_kernel(const long long* __restrict__ idx, const int* __restrict__ spos, const float* __restrict__ w,
                  const int* __restrict__ offs, long long M, int E, int rank, long long slot_stride, int offs_stride,
                  const __grid_constant__ PeerPtrs tab_idx,
                  const __grid_constant__ PeerPtrs tab_spos, const __grid_constant__ PeerPtrs tab_w,
                  const __grid_constant__ PeerPtrs tab_offs) {
  const int p = blockIdx.y;    // receiving rank
  long long* d_idx = reinterpret_cast<long long*>(const_cast<void*>(tab_idx.p[p])) + rank * slot_stride;
  int* d_spos = reinterpret_cast<int*>(const_cast<void*>(tab_spos.p[p])) + rank * slot_stride;
  float* d_w = reinterpret_cast<float*>(const_cast<void*>(tab_w.p[p])) + rank * slot_stride;
  int* d_offs = reinterpret_cast<int*>(const_cast<void*>(tab_offs.p[p])) + rank * offs_stride;
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < M; i += stride) {
    d_idx[i] = idx[i];
    d_spos[i] = spos[i];
    d_w[i] = w[i];
  }
  if (blockIdx.x == 0)
    for (int e = threadIdx.x; e <= E; e += blockDim.x) d_offs[e] = offs[e];
}

// The rows of this rank that a (source rank, token) pair feeds: lane j < k looks at slot j of the token in
// the source's routing tables (peer reads) and, when that expert lives here, computes the padded row
//   src_base[source][local expert] + (position of the slot inside its expert segment at the source).
// Returns the ballot of lanes with a local slot; `row` is valid on those lanes.
__device__ __forceinline__ unsigned local_rows_of_token(const long long* __restrict__ idx_s,
                                                        const int* __restrict__ spos_s,
                                                        const int* __restrict__ offs_s,
                                                        const int* __restrict__ src_base, int s, long long t, int k,
                                                        int rank, int El, int e_lo, int e_hi, int lane, int& row) {
  bool local = false;
  row = 0;
  if (lane < k) {
    const long long ev = idx_s[t * k + lane];
    // an index below 0 or past the last expert belongs to no rank; [e_lo, e_hi) = the local experts this launch serves
    if (ev >= 0 && ev / El == rank && ev - static_cast<long long>(rank) * El >= e_lo &&
        ev - static_cast<long long>(rank) * El < e_hi) {
      const int e = static_cast<int>(ev);
      const int sp = spos_s[t * k + lane];
      if (sp >= 0) {                    // -1: the source's permutation gave the slot no row
        row = src_base[s * El + (e - rank * El)] + sp - offs_s[e];
        local = row >= 0;               // negative: the plan refused the step (fixed capacity exceeded)
      }
    }
  }
  return __ballot_sync(0xffffffffu, local);
}

// pad rows [poffs[j] + counts[j], poffs[j+1]) of every local expert, one warp per row
template <typename F>
__device__ __forceinline__ void for_each_pad_row(const int* __restrict__ counts_l, const int* __restrict__ poffs_l,
                                                 int e_lo, int e_hi, long long warp0, long long nwarps, F f) {
  for (int j = e_lo; j < e_hi; ++j) {
    const int p0 = poffs_l[j] + counts_l[j], p1 = poffs_l[j + 1];
    for (long long r = p0 + warp0; r < p1; r += nwarps) f(r);
  }
}

// One warp per (source rank, token): the token row is loaded once (from the peer's x) and stored to each of
// its rows here.  Tasks are numbered token-major so that neighbouring warps read from different peers.
// THREADS = 256 for a launch over the whole GPU; 1024 when the launch is confined to a few SMs beside a persistent
// GEMM (one CTA per SM: a GEMM CTA takes a whole SM's shared memory, so the two never share an SM, and a pull of
// `n` CTAs takes at most `n` SMs away from the GEMM whichever of the two is placed first)
template <int THREADS>
__global__ void __launch_bounds__(THREADS)
ep_gather_pull_kernel(const __grid_constant__ PeerPtrs x_peers, const __grid_constant__ PeerPtrs idx_peers,
                      const __grid_constant__ PeerPtrs spos_peers, const __grid_constant__ PeerPtrs offs_peers,
                      const int* __restrict__ counts_l, const int* __restrict__ poffs_l,
                      const int* __restrict__ src_base, int W, int rank, int El, int e_lo, int e_hi, long long T, int k,
                      int vec_per_row, uint4* __restrict__ x_s, int* __restrict__ row_rank, int* __restrict__ row_slot) {
  const int lane = threadIdx.x & 31;
  const long long warp0 = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  const long long nwarps = (static_cast<long long>(gridDim.x) * blockDim.x) >> 5;
  for (long long task = warp0; task < T * W; task += nwarps) {
    const int s = static_cast<int>(task % W);
    const long long t = task / W;
    int row;
    const unsigned mask = local_rows_of_token(reinterpret_cast<const long long*>(idx_peers.p[s]),
                                              reinterpret_cast<const int*>(spos_peers.p[s]),
                                              reinterpret_cast<const int*>(offs_peers.p[s]), src_base, s, t, k, rank,
                                              El, e_lo, e_hi, lane, row);
    if (mask == 0u) continue;
    if (row_rank != nullptr && ((mask >> lane) & 1u)) {   // where the result rows of this row go back to
      row_rank[row] = s;
      row_slot[row] = static_cast<int>(t * k + lane);
    }
    const uint4* srow = reinterpret_cast<const uint4*>(x_peers.p[s]) + t * vec_per_row;
    // peer loads have microseconds of latency: keep 8 of them in flight per lane
    for (int c0 = lane; c0 < vec_per_row; c0 += 32 * 8) {
      uint4 v[8];
#pragma unroll
      for (int i = 0; i < 8; ++i)
        if (c0 + 32 * i < vec_per_row) v[i] = srow[c0 + 32 * i];
      for (unsigned m = mask; m != 0u; m &= m - 1) {
        const int r = __shfl_sync(0xffffffffu, row, __ffs(m) - 1);
        uint4* dst = x_s + static_cast<long long>(r) * vec_per_row;
#pragma unroll
        for (int i = 0; i < 8; ++i)
          if (c0 + 32 * i < vec_per_row) dst[c0 + 32 * i] = v[i];
      }
    }
  }
  for_each_pad_row(counts_l, poffs_l, e_lo, e_hi, warp0, nwarps, [&](long long r) {
    uint4* dst = x_s + r * vec_per_row;
    for (int c = lane; c < vec_per_row; c += 32) dst[c] = make_uint4(0u, 0u, 0u, 0u);
    if (row_rank != nullptr && lane == 0) {
      row_rank[r] = -1;
      row_slot[r] = 0;
    }
  });
}

__device__ __forceinline__ void fma8(float (&acc)[8], const uint4& v, float w) {
  const float2 a = unpack_bf16x2(v.x), b = unpack_bf16x2(v.y), c = unpack_bf16x2(v.z), d = unpack_bf16x2(v.w);
  acc[0] += w * a.x; acc[1] += w * a.y; acc[2] += w * b.x; acc[3] += w * b.y;
  acc[4] += w * c.x; acc[5] += w * c.y; acc[6] += w * d.x; acc[7] += w * d.y;
}

// out[t] = sum_j w[t,j] * rows_peer[owner(e_j)][dest_base[e_j] + slot_pos - offs[e_j]]
//
// A bulk-copy pipeline, so that a few SMs keep enough bytes in flight to fill NVLink and the kernel can run
// beside a persistent GEMM that leaves those SMs free.  One CTA per SM (its shared-memory ring fills the SM),
// 288 threads: warp 0 is the producer, warps 1-8 sum and store.  A work item is (token, 4 KB column chunk);
// its k source pieces are fetched with one cp.async.bulk each into a ring slot, counted on the slot's `full`
// barrier; the consumers add them in slot order j = 0..k-1 with the weights the producer left beside the data
// and release the slot.  The producer resolves the routing tables for 32/k items at a time (lane = item, slot)
// and one batch ahead, so those dependent loads are off the copy path.  Every wait is bounded.
constexpr int kPullChunk = 4096;          // bytes of one row piece
constexpr int kPullConsumers = 256;       // one 16-byte vector of the chunk per consumer thread
constexpr int kPullThreads = 32 + kPullConsumers;

__global__ void __launch_bounds__(kPullThreads, 1)
ep_combine_pull_kernel(const __grid_constant__ PeerPtrs rows_peers, const float* __restrict__ w,
                       const long long* __restrict__ idx, const int* __restrict__ slot_pos,
                       const int* __restrict__ offs, const int* __restrict__ dest_base, int El, int E, long long T, int k,
                       long long row_bytes, int nslots, uint8_t* __restrict__ out, int* __restrict__ status) {
  extern __shared__ uint8_t pull_smem_raw[];
  uint8_t* data = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(pull_smem_raw) + 127) & ~static_cast<uintptr_t>(127));
  float* sw = reinterpret_cast<float*>(data + static_cast<size_t>(nslots) * k * kPullChunk);   // [nslots][32]
  uint64_t* bars = reinterpret_cast<uint64_t*>(sw + nslots * 32);
  const uint32_t bar_full = smem_u32(bars), bar_empty = smem_u32(bars + nslots);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(bars + 2 * nslots);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    for (int s = 0; s < nslots; ++s) {
      mbar_init(bar_full + 8 * s, 1);
      mbar_init(bar_empty + 8 * s, kPullConsumers / 32);
    }
    *abort_flag = 0;
    fence_mbar_init();
  }
  __syncthreads();
  const int nchunk = static_cast<int>((row_bytes + kPullChunk - 1) / kPullChunk);
  const long long items = T * nchunk;
  if (warp == 0) {
    const int per = 32 / k;                  // items resolved per batch
    const int sub = lane / k, j = lane - sub * k;
    const bool active = sub < per;
    int slot = 0;
    uint32_t ph = 0;
    bool ok = true;
    // metadata of a batch: source address and weight of (item = first + sub * gridDim.x, slot j)
    auto resolve = [&](long long first, const uint8_t*& src, float& wj, uint32_t& bytes) {
      src = nullptr;
      wj = 0.0f;
      bytes = 0;
      const long long item = first + static_cast<long long>(sub) * gridDim.x;
      if (active && item < items) {
        const long long t = item / nchunk;
        const int ch = static_cast<int>(item - t * nchunk);
        const long long s = t * k + j;
        const long long ev = idx[s];
        const int e = static_cast<int>(ev);
        const long long off = static_cast<long long>(ch) * kPullChunk;
        bytes = static_cast<uint32_t>(row_bytes - off < kPullChunk ? row_bytes - off : kPullChunk);
        if (ev >= 0 && ev < E && slot_pos[s] >= 0) {
          const long long row = dest_base[e] + slot_pos[s] - offs[e];
          src = reinterpret_cast<const uint8_t*>(rows_peers.p[e / El]) + row * row_bytes + off;
          wj = (w != nullptr) ? w[s] : 1.0f;
        } else {
          // expert index out of range (the permutation raised the status word): the copy still has to deliver its
          // bytes to the barrier, so it reads row 0 of the first buffer; weight 0 makes the consumers skip the piece
          src = reinterpret_cast<const uint8_t*>(rows_peers.p[0]) + off;
          wj = 0.0f;
        }
      }
    };
    const long long stride = static_cast<long long>(per) * gridDim.x;
    const uint8_t* src;
    float wj;
    uint32_t bytes;
    resolve(blockIdx.x, src, wj, bytes);
    for (long long first = blockIdx.x; first < items && ok; first += stride) {
      const uint8_t* src_n;
      float wj_n;
      uint32_t bytes_n;
      resolve(first + stride, src_n, wj_n, bytes_n);   // next batch's tables are read during this batch's copies
      for (int b = 0; b < per; ++b) {
        if (first + static_cast<long long>(b) * gridDim.x >= items) break;
        int good = 1;
        if (lane == 0) good = mbar_wait(bar_empty + 8 * slot, ph ^ 1, abort_flag, ST_WAIT_PRODUCER) ? 1 : 0;
        good = __shfl_sync(0xffffffffu, good, 0);
        if (!good) {
          ok = false;
          break;
        }
        const uint32_t bytes_b = __shfl_sync(0xffffffffu, bytes, b * k);
        if (sub == b && active) sw[slot * 32 + j] = wj;
        __syncwarp();
        if (lane == 0) mbar_arrive_expect_tx(bar_full + 8 * slot, static_cast<uint32_t>(k) * bytes_b);
        __syncwarp();
        if (sub == b && active)
          bulk_load_1d(smem_u32(data + (static_cast<size_t>(slot) * k + j) * kPullChunk), src, bytes, bar_full + 8 * slot);
        if (++slot == nslots) {
          slot = 0;
          ph ^= 1;
        }
      }
      src = src_n;
      wj = wj_n;
      bytes = bytes_n;
    }
  } else {
    const int tid = threadIdx.x - 32;
    int slot = 0;
    uint32_t ph = 0;
    // items of this CTA in the producer's order: batches of `per`, item = first + b * gridDim.x
    const int per = 32 / k;
    const long long stride = static_cast<long long>(per) * gridDim.x;
    bool ok = true;
    for (long long first = blockIdx.x; first < items && ok; first += stride) {
      for (int b = 0; b < per; ++b) {
        const long long item = first + static_cast<long long>(b) * gridDim.x;
        if (item >= items) break;
        if (!mbar_wait(bar_full + 8 * slot, ph, abort_flag, ST_WAIT_EPILOGUE)) {
          ok = false;
          break;
        }
        const long long t = item / nchunk;
        const long long off = (item - t * nchunk) * kPullChunk;
        const int nvec = static_cast<int>((row_bytes - off < kPullChunk ? row_bytes - off : kPullChunk) >> 4);
        if (tid < nvec) {
          float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
          const uint8_t* base = data + static_cast<size_t>(slot) * k * kPullChunk + tid * 16;
          for (int jj = 0; jj < k; ++jj) {
            const float wjj = sw[slot * 32 + jj];
            if (wjj != 0.0f) fma8(acc, *reinterpret_cast<const uint4*>(base + static_cast<size_t>(jj) * kPullChunk), wjj);
          }
          uint4 o;
          o.x = pack_bf16x2(acc[0], acc[1]);
          o.y = pack_bf16x2(acc[2], acc[3]);
          o.z = pack_bf16x2(acc[4], acc[5]);
          o.w = pack_bf16x2(acc[6], acc[7]);
          *reinterpret_cast<uint4*>(out + t * row_bytes + off + tid * 16) = o;
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(bar_empty + 8 * slot);
        if (++slot == nslots) {
          slot = 0;
          ph ^= 1;
        }
      }
    }
  }
  __syncthreads();
  if (threadIdx.x == 0 && *abort_flag != 0 && status != nullptr) atomicCAS(status, 0, *abort_flag);
}

// grad of the routing weights: grad_w[t,j] = the owner's row dot product of that slot (a 4-byte peer read each)
__global__ void __launch_bounds__(256)
ep_pull_row_scalars_kernel(const __grid_constant__ PeerPtrs gw_peers, const long long* __restrict__ idx,
                           const int* __restrict__ slot_pos, const int* __restrict__ offs,
                           const int* __restrict__ dest_base, int El, int E, long long slots, float* __restrict__ grad_w) {
  for (long long s = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; s < slots;
       s += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long ev = idx[s];
    const int e = static_cast<int>(ev);
    grad_w[s] = (ev >= 0 && ev < E && slot_pos[s] >= 0)
                    ? reinterpret_cast<const float*>(gw_peers.p[e / El])[dest_base[e] + slot_pos[s] - offs[e]]
                    : 0.0f;   // a slot whose expert index is out of range owns no row
  }
}

// One warp per (source rank, token): grad_out of the token is loaded once from the peer; for each of its
// rows r here grad_eo[r] = grad_out * w_peer[slot] and gw_rows[r] = <grad_out, eo[r]> (fp32); pad rows zero.
// DOTS = false: no row dot products (eo ignored), twice the loads in flight per lane (KB = 8); THREADS as for
// ep_gather_pull_kernel.
template <int THREADS, int MINB, bool DOTS, int KB>
__global__ void __launch_bounds__(THREADS, MINB)
ep_combine_bwd_pull_kernel(const __grid_constant__ PeerPtrs go_peers, const __grid_constant__ PeerPtrs w_peers,
                           const __grid_constant__ PeerPtrs idx_peers, const __grid_constant__ PeerPtrs spos_peers,
                           const __grid_constant__ PeerPtrs offs_peers, const uint4* __restrict__ eo, const int* __restrict__ counts_l,
                           const int* __restrict__ poffs_l, const int* __restrict__ src_base, int W, int rank, int El,
                           int e_lo, int e_hi, long long T, int k, int vec_per_row, uint4* __restrict__ grad_eo,
                           float* __restrict__ gw_rows) {
  const int lane = threadIdx.x & 31;
  const long long warp0 = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  const long long nwarps = (static_cast<long long>(gridDim.x) * blockDim.x) >> 5;
  for (long long task = warp0; task < T * W; task += nwarps) {
    const int s = static_cast<int>(task % W);
    const long long t = task / W;
    int row;
    const unsigned mask = local_rows_of_token(reinterpret_cast<const long long*>(idx_peers.p[s]),
                                              reinterpret_cast<const int*>(spos_peers.p[s]),
                                              reinterpret_cast<const int*>(offs_peers.p[s]), src_base, s, t, k, rank,
                                              El, e_lo, e_hi, lane, row);
    if (mask == 0u) continue;
    float wt_lane = 0.0f;
    if ((mask >> lane) & 1u) wt_lane = reinterpret_cast<const float*>(w_peers.p[s])[t * k + lane];
    const uint4* g = reinterpret_cast<const uint4*>(go_peers.p[s]) + t * vec_per_row;
    float dot_lane = 0.0f;   // lane j keeps the row dot of slot j
    constexpr int kB = KB;   // 16-byte vectors per lane and row in flight
    const bool dots = DOTS && eo != nullptr;
    for (int c0 = lane; c0 < vec_per_row; c0 += 32 * kB) {
      uint4 gv[kB], ev[kB], ev_next[kB];
#pragma unroll
      for (int i = 0; i < kB; ++i)
        if (c0 + 32 * i < vec_per_row) gv[i] = g[c0 + 32 * i];
      unsigned m = mask;
      int j = __ffs(m) - 1;
      int r = __shfl_sync(0xffffffffu, row, j);
      if (dots) {
        const uint4* e = eo + static_cast<long long>(r) * vec_per_row;
#pragma unroll
        for (int i = 0; i < kB; ++i)
          if (c0 + 32 * i < vec_per_row) ev[i] = e[c0 + 32 * i];
      }
      while (m != 0u) {
        m &= m - 1;
        // the next slot's eo row is requested before this slot's arithmetic
        const int jn = m != 0u ? __ffs(m) - 1 : j;
        const int rn = __shfl_sync(0xffffffffu, row, jn);
        if (m != 0u && dots) {
          const uint4* e = eo + static_cast<long long>(rn) * vec_per_row;
#pragma unroll
          for (int i = 0; i < kB; ++i)
            if (c0 + 32 * i < vec_per_row) ev_next[i] = e[c0 + 32 * i];
        }
        const float wt = __shfl_sync(0xffffffffu, wt_lane, j);
        uint4* dst = grad_eo + static_cast<long long>(r) * vec_per_row;
        float dot = 0.0f;
#pragma unroll
        for (int i = 0; i < kB; ++i)
          if (c0 + 32 * i < vec_per_row) {
            const float2 g0 = unpack_bf16x2(gv[i].x), g1 = unpack_bf16x2(gv[i].y), g2 = unpack_bf16x2(gv[i].z), g3 = unpack_bf16x2(gv[i].w);
            if (dots) {
              const float2 e0 = unpack_bf16x2(ev[i].x), e1 = unpack_bf16x2(ev[i].y), e2 = unpack_bf16x2(ev[i].z), e3 = unpack_bf16x2(ev[i].w);
              dot += g0.x * e0.x + g0.y * e0.y + g1.x * e1.x + g1.y * e1.y + g2.x * e2.x + g2.y * e2.y + g3.x * e3.x + g3.y * e3.y;
            }
            uint4 o;
            o.x = pack_bf16x2(g0.x * wt, g0.y * wt);
            o.y = pack_bf16x2(g1.x * wt, g1.y * wt);
            o.z = pack_bf16x2(g2.x * wt, g2.y * wt);
            o.w = pack_bf16x2(g3.x * wt, g3.y * wt);
            dst[c0 + 32 * i] = o;
          }
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, off);
        if (lane == j) dot_lane += dot;   // chunks of the row in ascending order: a fixed summation order
#pragma unroll
        for (int i = 0; i < kB; ++i) ev[i] = ev_next[i];
        j = jn;
        r = rn;
      }
    }
    if (DOTS && gw_rows != nullptr && ((mask >> lane) & 1u)) gw_rows[row] = dot_lane;
  }
  for_each_pad_row(counts_l, poffs_l, e_lo, e_hi, warp0, nwarps, [&](long long r) {
    uint4* dst = grad_eo + r * vec_per_row;
    for (int c = lane; c < vec_per_row; c += 32) dst[c] = make_uint4(0u, 0u, 0u, 0u);
    if (gw_rows != nullptr && lane == 0) gw_rows[r] = 0.0f;
  });
}

// out[s] = <go[s / k], rows[s]> in fp32, one warp per slot (the routing-weight gradient where the expert
// outputs of a token sit in slot order at its home rank)
__global__ void __launch_bounds__(256)
slot_dots_kernel(const uint4* __restrict__ go, const uint4* __restrict__ rows, long long slots, int k, int vec_per_row,
                 float* __restrict__ out) {
  const int lane = threadIdx.x & 31;
  const long long nwarps = (static_cast<long long>(gridDim.x) * blockDim.x) >> 5;
  for (long long s = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5; s < slots; s += nwarps) {
    const uint4* g = go + (s / k) * vec_per_row;
    const uint4* e = rows + s * vec_per_row;
    float dot = 0.0f;
    for (int c0 = lane; c0 < vec_per_row; c0 += 32 * 4) {
      uint4 gv[4], ev[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const bool in = c0 + 32 * i < vec_per_row;
        gv[i] = in ? g[c0 + 32 * i] : make_uint4(0u, 0u, 0u, 0u);
        ev[i] = in ? e[c0 + 32 * i] : make_uint4(0u, 0u, 0u, 0u);
      }
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float2 g0 = unpack_bf16x2(gv[i].x), g1 = unpack_bf16x2(gv[i].y), g2 = unpack_bf16x2(gv[i].z), g3 = unpack_bf16x2(gv[i].w);
        const float2 e0 = unpack_bf16x2(ev[i].x), e1 = unpack_bf16x2(ev[i].y), e2 = unpack_bf16x2(ev[i].z), e3 = unpack_bf16x2(ev[i].w);
        dot += g0.x * e0.x + g0.y * e0.y + g1.x * e1.x + g1.y * e1.y + g2.x * e2.x + g2.y * e2.y + g3.x * e3.x + g3.y * e3.y;
      }
    }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, off);
    if (lane == 0) out[s] = dot;
  }
}

// Cross-rank barrier on a symmetric flag array (W unsigned words per rank, zero before the first use).
// Thread p of the one CTA announces this rank at peer p: a release store of `generation` into word `rank` of
// p's array (a plain peer store over NVLink); then it waits, with an acquire load of its OWN array's word p,
// until peer p's announcement of the same (or a later) generation shows up.  Every rank writes only its own
// word of every array, so no atomics are needed and generations only grow.  The wait is bounded by
// `limit_cycles` SM clocks: when it runs out the kernel raises ST_WAIT_PEER in `status` and returns normally,
// so a missing peer ends in a status code and a usable context, never in a hung GPU or a trap.
// Stream order makes the writes of earlier kernels of this stream (peer stores included) complete before the
// release store; the acquire load orders the kernels queued after the barrier behind the peers' writes.
__global__ void __launch_bounds__(kMaxRanks)
ep_barrier_kernel(const __grid_constant__ PeerPtrs flags_peers, int W, int rank, unsigned generation,
                  long long limit_cycles, int* __restrict__ status) {
  const int p = threadIdx.x;
  if (p >= W) return;
  unsigned* theirs = reinterpret_cast<unsigned*>(const_cast<void*>(flags_peers.p[p])) + rank;
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(theirs), "r"(generation) : "memory");
  const unsigned* mine = reinterpret_cast<const unsigned*>(flags_peers.p[rank]) + p;
  const long long t0 = clock64();
  for (unsigned it = 0;; ++it) {
    unsigned seen;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(seen) : "l"(mine) : "memory");
    if (static_cast<int>(seen - generation) >= 0) return;       // wrap-safe "seen >= generation"
    if ((it & 0x3f) == 0x3f && clock64() - t0 > limit_cycles) {
      atomicCAS(status, 0, ST_WAIT_PEER);
      return;
    }
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
                    int32_t* tile_expert_l, int32_t* src_base, int32_t* dest_base, int64_t rows_cap, int32_t* status,
                    b200moe_stream_t stream) {
  B200_CHECK_ARG(counts_all && poffs_l && counts_l && tile_expert_l && src_base && dest_base, B200MOE_E_NULL,
                 "ep_plan: null pointer");
  CHECK_WORLD("ep_plan");
  B200_CHECK_ARG(E >= W && E <= B200MOE_MAX_EXPERTS && E % W == 0, B200MOE_E_BAD_SHAPE,
                 "ep_plan: E = %d must be a multiple of W = %d and at most %d", E, W, B200MOE_MAX_EXPERTS);
  B200_CHECK_ARG(rows_cap <= 0 || (status != nullptr && rows_cap % B200MOE_TILE_M == 0), B200MOE_E_BAD_SHAPE,
                 "ep_plan: a row capacity (%lld) needs a status word and must be a multiple of %d", (long long)rows_cap,
                 B200MOE_TILE_M);
  ep_plan_kernel<<<1, B200MOE_MAX_EXPERTS, 0, (cudaStream_t)stream>>>(counts_all, W, rank, E, poffs_l, counts_l,
                                                                       tile_expert_l, src_base, dest_base, rows_cap,
                                                                       status);
  B200_CUDA(cudaGetLastError());
  return 0;
}

int b200moe_ep_local_rows(const int32_t* counts_all, int W, int rank, int E, int32_t* host_words,
                          b200moe_stream_t stream) {
  B200_CHECK_ARG(counts_all && host_words, B200MOE_E_NULL, "ep_local_rows: null pointer");
  CHECK_WORLD("ep_local_rows");
  B200_CHECK_ARG(E >= W && E <= B200MOE_MAX_EXPERTS && E % W == 0, B200MOE_E_BAD_SHAPE,
                 "ep_local_rows: E = %d must be a multiple of W = %d and at most %d", E, W, B200MOE_MAX_EXPERTS);
  void* dev_view = nullptr;   // the device's address of the pinned host words; fails (nothing launched) if not pinned
  B200_CUDA(cudaHostGetDevicePointer(&dev_view, host_words, 0));
  ep_local_rows_kernel<<<1, B200MOE_MAX_EXPERTS, 0, (cudaStream_t)stream>>>(counts_all, W, rank, E,
                                                                             reinterpret_cast<volatile int*>(dev_view));
  B200_CUDA(cudaGetLastError());
  return 0;
}

#define LOAD_PEERS(var, table, who)                 \
  PeerPtrs var;                                     \
  {                                                 \
    const int rc__ = load_peers(&var, table, W, who); \
    if (rc__) return rc__;                          \
  }

int b200moe_ep_publish(const int64_t* idx, const int32_t* slot_pos, const float* w, const int32_t* offs, int64_t M, int E,
                       int W, int rank, int64_t slot_stride, int offs_stride, const void* const* tab_idx_peers, const void* const* tab_spos_peers,
                       const void* const* tab_w_peers, const void* const* tab_offs_peers, b200moe_stream_t stream) {
  B200_CHECK_ARG(idx && slot_pos && w && offs, B200MOE_E_NULL, "ep_publish: null pointer");
  CHECK_WORLD("ep_publish");
  B200_CHECK_ARG(M >= 0 && E >= 1 && E <= B200MOE_MAX_EXPERTS, B200MOE_E_BAD_SHAPE, "ep_publish: M = %lld, E = %d", (long long)M, E);
  B200_CHECK_ARG(slot_stride >= M && slot_stride % 4 == 0 && offs_stride >= E + 1 && offs_stride % 4 == 0, B200MOE_E_BAD_SHAPE,
                 "ep_publish: strides %lld / %d must cover M = %lld / E + 1 = %d and be multiples of 4 elements",
                 (long long)slot_stride, offs_stride, (long long)M, E + 1);
  LOAD_PEERS(ti, tab_idx_peers, "ep_publish(idx tables)");
  LOAD_PEERS(ts, tab_spos_peers, "ep_publish(slot_pos tables)");
  LOAD_PEERS(tw, tab_w_peers, "ep_publish(weight tables)");
  LOAD_PEERS(to, tab_offs_peers, "ep_publish(offs tables)");
  long long bx = (M + 255) / 256;
  if (bx > 64) bx = 64;
  if (bx < 1) bx = 1;
  ep_publish_kernel<<<dim3(static_cast<unsigned>(bx), static_cast<unsigned>(W)), 256, 0, (cudaStream_t)stream>>>(
      reinterpret_cast<const long long*>(idx), slot_pos, w, offs, M, E, rank, slot_stride, offs_stride, ti, ts, tw, to);
  B200_CUDA(cudaGetLastError());
  return 0;
}

int b200moe_ep_gather_pull(const void* const* x_peers, const void* const* idx_peers, const void* const* spos_peers,
                           const void* const* offs_peers, const int32_t* counts_l, const int32_t* poffs_l,
                           const int32_t* src_base, int W, int rank, int E, int e_lo, int e_hi, int max_sms, int64_t T,
                           int k, int64_t H, void* x_s, int32_t* row_rank, int32_t* row_slot, b200moe_stream_t stream) {
  B200_CHECK_ARG(counts_l && poffs_l && src_base && x_s, B200MOE_E_NULL, "ep_gather_pull: null pointer");
  B200_CHECK_ARG((row_rank == nullptr) == (row_slot == nullptr), B200MOE_E_NULL,
                 "ep_gather_pull: row_rank and row_slot go together");
  CHECK_WORLD("ep_gather_pull");
  B200_CHECK_ARG(H > 0 && H % 8 == 0 && k >= 1 && k <= B200MOE_MAX_TOPK && E % W == 0 && T >= 0, B200MOE_E_BAD_SHAPE,
                 "ep_gather_pull: H = %lld, k = %d, T = %lld", (long long)H, k, (long long)T);
  LOAD_PEERS(xp, x_peers, "ep_gather_pull(x)");
  LOAD_PEERS(ip, idx_peers, "ep_gather_pull(idx)");
  LOAD_PEERS(sp, spos_peers, "ep_gather_pull(slot_pos)");
  LOAD_PEERS(fp, offs_peers, "ep_gather_pull(offs)");
  B200_CHECK_ARG(0 <= e_lo && e_lo <= e_hi && e_hi <= E / W && max_sms >= 0, B200MOE_E_BAD_SHAPE,
                 "ep_gather_pull: local expert range [%d, %d) of %d, max_sms = %d", e_lo, e_hi, E / W, max_sms);
  if (max_sms > 0 && max_sms < num_sms())
    ep_gather_pull_kernel<1024><<<max_sms, 1024, 0, (cudaStream_t)stream>>>(
        xp, ip, sp, fp, counts_l, poffs_l, src_base, W, rank, E / W, e_lo, e_hi, T, k, static_cast<int>(H / 8),
        reinterpret_cast<uint4*>(x_s), row_rank, row_slot);
  else
    ep_gather_pull_kernel<256><<<grid_rows((T * W + 7) / 8, 8), 256, 0, (cudaStream_t)stream>>>(
        xp, ip, sp, fp, counts_l, poffs_l, src_base, W, rank, E / W, e_lo, e_hi, T, k, static_cast<int>(H / 8),
        reinterpret_cast<uint4*>(x_s), row_rank, row_slot);
  B200_CUDA(cudaGetLastError());
  return 0;
}

int b200moe_ep_combine_pull(const void* const* rows_peers, const float* w, const int64_t* idx, const int32_t* slot_pos,
                            const int32_t* offs, const int32_t* dest_base, int W, int E, int64_t T, int k, int64_t H,
                            void* out, const void* const* gw_peers, float* grad_w, int32_t* status,
                            b200moe_stream_t stream) {
  B200_CHECK_ARG(idx && slot_pos && offs && dest_base && out, B200MOE_E_NULL, "ep_combine_pull: null pointer");
  const int rank = 0;
  CHECK_WORLD("ep_combine_pull");
  B200_CHECK_ARG(H > 0 && H % 8 == 0 && k >= 1 && k <= B200MOE_MAX_TOPK && E % W == 0, B200MOE_E_BAD_SHAPE,
                 "ep_combine_pull: H = %lld, k = %d", (long long)H, k);
  B200_CHECK_ARG((gw_peers == nullptr) == (grad_w == nullptr), B200MOE_E_NULL,
                 "ep_combine_pull: gw_peers and grad_w go together");
  B200_CHECK_ARG(aligned16(out), B200MOE_E_ALIGN, "ep_combine_pull: out must be 16-byte aligned");
  LOAD_PEERS(rp, rows_peers, "ep_combine_pull(rows)");
  if (T <= 0) return 0;
  if (gw_peers != nullptr) {
    LOAD_PEERS(gp, gw_peers, "ep_combine_pull(grad_w rows)");
    ep_pull_row_scalars_kernel<<<grid_rows((T * k + 255) / 256, 8), 256, 0, (cudaStream_t)stream>>>(
        gp, reinterpret_cast<const long long*>(idx), slot_pos, offs, dest_base, E / W, E, T * k, grad_w);
    B200_CUDA(cudaGetLastError());
  }
  // ring slots: as many (k pieces of 4 KB + 32 weights + 2 barriers) as fit in 227 KB, at most 16
  const size_t per_slot = static_cast<size_t>(k) * kPullChunk + 32 * sizeof(float) + 16;
  int nslots = static_cast<int>((232448 - 256) / per_slot);
  if (nslots > 16) nslots = 16;
  B200_CHECK_ARG(nslots >= 2, B200MOE_E_UNSUPPORTED, "ep_combine_pull: k = %d rows of 4 KB do not fit twice in shared memory", k);
  const size_t smem = nslots * per_slot + 128 + 16;
  static std::once_flag once;
  static cudaError_t attr_err = cudaSuccess;
  std::call_once(once, [] {
    attr_err = cudaFuncSetAttribute(ep_combine_pull_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 232448);
  });
  if (attr_err != cudaSuccess) return cuda_fail(attr_err, "cudaFuncSetAttribute(max dynamic smem)");
  const long long row_bytes = H * 2;
  const long long items = T * ((row_bytes + kPullChunk - 1) / kPullChunk);
  long long grid = exchange_sm_budget();
  if (grid > items) grid = items;
  ep_combine_pull_kernel<<<static_cast<int>(grid), kPullThreads, smem, (cudaStream_t)stream>>>(
      rp, w, reinterpret_cast<const long long*>(idx), slot_pos, offs, dest_base, E / W, E, T, k, row_bytes, nslots,
      reinterpret_cast<uint8_t*>(out), status);
  B200_CUDA(cudaGetLastError());
  return 0;
}

int b200moe_ep_combine_bwd_pull(const void* const* go_peers, const void* const* w_peers,
                                const void* const* idx_peers, const void* const* spos_peers,
                                const void* const* offs_peers, const void* eo, const int32_t* counts_l,
                                const int32_t* poffs_l, const int32_t* src_base, int W, int rank, int E, int e_lo,
                                int e_hi, int max_sms, int64_t T, int k, int64_t H, void* grad_eo, float* gw_rows,
                                b200moe_stream_t stream) {
  B200_CHECK_ARG(counts_l && poffs_l && src_base && grad_eo, B200MOE_E_NULL, "ep_combine_bwd_pull: null pointer");
  B200_CHECK_ARG((eo == nullptr) == (gw_rows == nullptr), B200MOE_E_NULL,
                 "ep_combine_bwd_pull: eo and gw_rows go together (both NULL: no row dot products)");
  CHECK_WORLD("ep_combine_bwd_pull");
  B200_CHECK_ARG(H > 0 && H % 8 == 0 && k >= 1 && k <= B200MOE_MAX_TOPK && E % W == 0 && T >= 0, B200MOE_E_BAD_SHAPE,
                 "ep_combine_bwd_pull: H = %lld, k = %d, T = %lld", (long long)H, k, (long long)T);
  LOAD_PEERS(gp, go_peers, "ep_combine_bwd_pull(grad_out)");
  LOAD_PEERS(wp, w_peers, "ep_combine_bwd_pull(weights)");
  LOAD_PEERS(ip, idx_peers, "ep_combine_bwd_pull(idx)");
  LOAD_PEERS(sp, spos_peers, "ep_combine_bwd_pull(slot_pos)");
  LOAD_PEERS(fp, offs_peers, "ep_combine_bwd_pull(offs)");
  B200_CHECK_ARG(0 <= e_lo && e_lo <= e_hi && e_hi <= E / W && max_sms >= 0, B200MOE_E_BAD_SHAPE,
                 "ep_combine_bwd_pull: local expert range [%d, %d) of %d, max_sms = %d", e_lo, e_hi, E / W, max_sms);
  const bool few_sms = max_sms > 0 && max_sms < num_sms();
#define B200_BWD_PULL(THREADS, MINB, DOTS, KB, GRID)                                                               \
  ep_combine_bwd_pull_kernel<THREADS, MINB, DOTS, KB><<<(GRID), THREADS, 0, (cudaStream_t)stream>>>(               \
      gp, wp, ip, sp, fp, reinterpret_cast<const uint4*>(eo), counts_l, poffs_l, src_base, W, rank, E / W, e_lo,   \
      e_hi, T, k, static_cast<int>(H / 8), reinterpret_cast<uint4*>(grad_eo), gw_rows)
  if (few_sms && eo == nullptr) B200_BWD_PULL(1024, 1, false, 8, max_sms);
  else if (few_sms) B200_BWD_PULL(768, 1, true, 4, max_sms);
  else B200_BWD_PULL(256, 3, true, 4, grid_rows((T * W + 7) / 8, 8));
#undef B200_BWD_PULL
  B200_CUDA(cudaGetLastError());
  return 0;
}

int b200moe_ep_barrier(const void* const* flags_peers, int W, int rank, uint32_t generation, int64_t limit_cycles,
                       int32_t* status, b200moe_stream_t stream) {
  B200_CHECK_ARG(status != nullptr, B200MOE_E_NULL, "ep_barrier: null status word");
  CHECK_WORLD("ep_barrier");
  B200_CHECK_ARG(limit_cycles >= 1000 && limit_cycles <= 40000000000LL, B200MOE_E_BAD_SHAPE,
                 "ep_barrier: limit_cycles = %lld outside [1e3, 4e10]", (long long)limit_cycles);
  B200_CHECK_ARG(flags_peers != nullptr, B200MOE_E_NULL, "ep_barrier: null peer pointer table");
  PeerPtrs fp;
  for (int i = 0; i < kMaxRanks; ++i) fp.p[i] = nullptr;
  for (int i = 0; i < W; ++i) {
    B200_CHECK_ARG(flags_peers[i] != nullptr && (reinterpret_cast<uintptr_t>(flags_peers[i]) & 3) == 0, B200MOE_E_ALIGN,
                   "ep_barrier: flag array %d is null or not 4-byte aligned", i);
    fp.p[i] = flags_peers[i];
  }
  ep_barrier_kernel<<<1, kMaxRanks, 0, (cudaStream_t)stream>>>(fp, W, rank, generation, limit_cycles, status);
  B200_CUDA(cudaGetLastError());
  return 0;
}

int b200moe_slot_dots(const void* grad_out, const void* rows, int64_t T, int k, int64_t H, float* out,
                      b200moe_stream_t stream) {
  B200_CHECK_ARG(grad_out && rows && out, B200MOE_E_NULL, "slot_dots: null pointer");
  B200_CHECK_ARG(H > 0 && H % 8 == 0 && k >= 1 && T >= 0, B200MOE_E_BAD_SHAPE, "slot_dots: H = %lld, k = %d", (long long)H, k);
  B200_CHECK_ARG(aligned16(grad_out) && aligned16(rows), B200MOE_E_ALIGN, "slot_dots: pointers must be 16-byte aligned");
  if (T == 0) return 0;
  slot_dots_kernel<<<grid_rows((T * k + 7) / 8, 8), 256, 0, (cudaStream_t)stream>>>(
      reinterpret_cast<const uint4*>(grad_out), reinterpret_cast<const uint4*>(rows), T * k, k, static_cast<int>(H / 8), out);
  B200_CUDA(cudaGetLastError());
  return 0;
}

}  // extern "C"
