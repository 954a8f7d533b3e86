// Pieces shared by the bf16 and the MXFP8 GEMM translation units: schedules, tile decoding,
// epilogue math, tensor-map encoding.
#pragma once
#include <cuda.h>

#include <mutex>

#include "common.cuh"
#include "ptx.cuh"

namespace b200moe {

enum : int { SCHED_DENSE = 0, SCHED_GROUPED_M = 1, SCHED_GROUPED_K = 2 };
// EPI_STORE_SYM: EPI_STORE for symmetric results (256-wide tiles), able to store the transposed chunks as well
enum : int { EPI_STORE = 0, EPI_SWIGLU = 1, EPI_GLU_BWD = 2, EPI_STORE_F32 = 3, EPI_AXPBY = 4, EPI_STORE_SYM = 5 };

constexpr int BM = 128;  // rows per CTA = TMEM lanes
constexpr int kEpiWarps = 8;
constexpr int kThreads = 64 + 32 * kEpiWarps;

struct GemmParams {
  int sched;
  int a_mn, b_mn;        // 1 = operand is MN-major
  int M;                 // DENSE: rows of D; GROUPED_K: rows of D[e] (= MN extent of A)
  int N;                 // columns of D (SwiGLU: I)
  int K;                 // reduction length (DENSE, GROUPED_M); total rows (GROUPED_K by chunks)
  int num_groups;        // experts (GROUPED_M/K) or K-chunks
  int k_chunk;           // GROUPED_K without poffs: rows per chunk (multiple of 64)
  const int* tile_expert;  // GROUPED_M: expert of each B200MOE_TILE_M-row tile
  const int* poffs;        // (num_groups+1) padded row offsets, multiples of B200MOE_TILE_M
  const int* counts;       // GROUPED_K, optional: live rows per group (pad rows past them are zero)
  void* D;
  long long ldd;
  long long d_group_stride;  // GROUPED_K: elements between D[e] and D[e+1]
  void* aux;                 // SwiGLU: inter (rows, I); GLU_BWD: saved gate_up (rows, 2I); AXPBY: C (rows, N)
  int I;
  // GROUPED_M with equal square groups (sym_rows rows and N = sym_rows columns each) whose result is symmetric:
  // only the tiles that reach the upper triangle of each group are computed (0 = all tiles); with sym_mirror the
  // epilogue also stores every chunk of a tile right of the diagonal tile a second time, transposed, so the
  // result arrives complete
  int sym_rows;
  int sym_mirror;
  // EPI_AXPBY (256-wide tiles): D = ax_alpha * (A B) + ax_beta * C + ax_diag * [column == row - poffs[group]]
  float ax_alpha, ax_beta, ax_diag;
  int* status;
  // optional, EPI_STORE with 256-wide tiles: output row r is not stored to D but sent to
  // push_base[push_rank[r]] + push_slot[r] * N elements (a peer GPU's buffer); rows with push_rank < 0 are dropped
  const int* push_rank;
  const int* push_slot;
  const long long* push_base;
  // optional, GLU epilogues of the POLY instantiations: activation code of each expert (0 SiLU, 1 ReLU^2,
  // 5 SiTU = tanh(g) * sigmoid(g)); nullptr in the plain instantiations, which are SiLU only
  const int* act_codes;
  // optional, GROUPED_M: only the row tiles of rows [row_lo, row_hi) are computed (multiples of B200MOE_TILE_M;
  // row_hi <= 0: every row).  Lets a caller run the rows of one group of experts while the rows of the next
  // group are still arriving.
  int row_lo, row_hi;
  // optional (conv_taps > 0): causal-convolution operand.  The operand's tensor map is {conv_C channels, conv_S
  // positions, batches} and every 64-wide k-block is loaded `shift` positions away from the tile's own, positions
  // outside [0, conv_S) reading as zero (the convolution's padding), so the unfolded (rows, taps * C) copy of the
  // input is never written.  DENSE: operand A, k-block kb = (tap, channel block), shift = conv_sign * (tap -
  // (conv_taps - 1)); row tiles must not straddle batches (conv_S % 128 == 0).  GROUPED_K by chunks (split-K
  // weight gradient): operand B, tap = tile column / conv_C, shift = tap - (conv_taps - 1); conv_S % 64 == 0.
  int conv_taps, conv_S, conv_C, conv_sign;
};

struct Tile {
  int m0, n0, g, k0, nkb;
};

// tiles of one symmetric group that reach its upper triangle: row tile mi covers columns from (mi*TM/TN)*TN on
__device__ __forceinline__ int sym_tiles_per_group(const GemmParams& p, int TN, int TM) {
  const int nt = (p.N + TN - 1) / TN;
  int n = 0;
  for (int mi = 0; mi * TM < p.sym_rows; ++mi) n += nt - (mi * TM) / TN;
  return n;
}

// `window`: the launch honours GemmParams::row_lo / row_hi (only the kernels whose entry points take a row window
// are compiled with it, so that the others carry no code or registers for it)
__device__ __forceinline__ int total_tiles(const GemmParams& p, int TN, int TM, bool window = false) {
  const int nt = (p.N + TN - 1) / TN;
  if (p.sched == SCHED_GROUPED_M && p.sym_rows > 0) return p.num_groups * sym_tiles_per_group(p, TN, TM);
  if (p.sched == SCHED_DENSE) return ((p.M + TM - 1) / TM) * nt;
  if (p.sched == SCHED_GROUPED_M) {
    const int rows = p.poffs[p.num_groups];
    return ((window && p.row_hi > 0 ? max(min(rows, p.row_hi) - p.row_lo, 0) : rows) / TM) * nt;
  }
  return ((p.M + TM - 1) / TM) * nt * p.num_groups;
}

// GROUPED_K with live-row counts: the groups in descending order of their reduction length, so that the
// static round-robin of tiles over the persistent CTAs deals the long tiles out evenly (an expert with many
// rows next to experts with few would otherwise leave most CTAs idle at the end).  Every thread of the CTA
// calls this before the barrier that precedes the role dispatch; `order` is a shared array of
// B200MOE_MAX_EXPERTS ints.  Returns nullptr when the plain order is used.
__device__ __forceinline__ const int* build_group_order(const GemmParams& p, int* order) {
  if (p.sched != SCHED_GROUPED_K || p.counts == nullptr || p.num_groups > B200MOE_MAX_EXPERTS) return nullptr;
  for (int i = threadIdx.x; i < p.num_groups; i += blockDim.x) {
    const int ci = p.counts[i];
    int rank = 0;
    for (int j = 0; j < p.num_groups; ++j) {
      const int cj = p.counts[j];
      rank += (cj > ci || (cj == ci && j < i)) ? 1 : 0;
    }
    order[rank] = i;
  }
  return order;
}

__device__ __forceinline__ Tile get_tile(const GemmParams& p, int tile, int TN, int TM, int BK = 64,
                                         const int* order = nullptr, int row_base = 0) {
  Tile t;
  const int nt = (p.N + TN - 1) / TN;
  if (p.sched == SCHED_GROUPED_K) {
    const int mt = (p.M + TM - 1) / TM;
    const int per = mt * nt;
    const int gi = tile / per;
    t.g = order != nullptr ? order[gi] : gi;
    const int r = tile - gi * per;
    t.m0 = (r / nt) * TM;
    t.n0 = (r % nt) * TN;
    int kb, ke;
    if (p.poffs != nullptr) {
      kb = p.poffs[t.g];
      ke = (p.counts != nullptr) ? kb + p.counts[t.g] : p.poffs[t.g + 1];   // skip all-zero k-blocks
    } else {
      kb = t.g * p.k_chunk;
      ke = min(p.K, kb + p.k_chunk);
    }
    t.k0 = kb;
    t.nkb = (ke - kb + BK - 1) / BK;
  } else if (p.sched == SCHED_GROUPED_M && p.sym_rows > 0) {
    const int per = sym_tiles_per_group(p, TN, TM);
    const int g = tile / per;
    int r = tile - g * per, mi = 0;
    for (;; ++mi) {                       // row tile mi owns nt - first(mi) consecutive indices
      const int len = nt - (mi * TM) / TN;
      if (r < len) break;
      r -= len;
    }
    t.m0 = g * p.sym_rows + mi * TM;
    t.n0 = ((mi * TM) / TN + r) * TN;
    t.g = g;
    t.k0 = 0;
    t.nkb = (p.K + BK - 1) / BK;
  } else {
    const int mi = tile / nt;
    t.m0 = mi * TM + row_base;   // first row of the launch's row window (0: every row)
    t.n0 = (tile - mi * nt) * TN;
    t.g = (p.sched == SCHED_GROUPED_M) ? p.tile_expert[t.m0 / B200MOE_TILE_M] : 0;
    t.k0 = 0;
    t.nkb = (p.K + BK - 1) / BK;
  }
  return t;
}

__device__ __forceinline__ uint4 pack8(const uint32_t* r) {
  uint4 o;
  o.x = pack_bf16x2(__uint_as_float(r[0]), __uint_as_float(r[1]));
  o.y = pack_bf16x2(__uint_as_float(r[2]), __uint_as_float(r[3]));
  o.z = pack_bf16x2(__uint_as_float(r[4]), __uint_as_float(r[5]));
  o.w = pack_bf16x2(__uint_as_float(r[6]), __uint_as_float(r[7]));
  return o;
}

// GLU activations of the fused epilogues, by activation code: 0 SiLU, 1 ReLU^2, 5 SiTU = tanh(g) * sigmoid(g)
// (the parameter-free codes of the reference that need no row reduction, kernels/sm75/moe.py:859-881).  The code is
// uniform over a tile (one expert per row tile), so the epilogues branch once per 32-column chunk and run a loop
// specialised for the code; code 0 uses the expressions the SiLU-only kernels have always used.
template <int CODE>
__device__ __forceinline__ float glu_fwd_val(float g, float u) {
  if constexpr (CODE == 1) {
    const float r = fmaxf(g, 0.0f);
    return r * r * u;
  } else {
    const float s = __fdividef(1.0f, 1.0f + __expf(-g));
    if constexpr (CODE == 5) {
      const float t = __fdividef(2.0f, 1.0f + __expf(-2.0f * g)) - 1.0f;
      return t * s * u;
    } else {
      return g * s * u;
    }
  }
}
// grad_gate = go * up * f'(g), grad_up = go * f(g)
template <int CODE>
__device__ __forceinline__ void glu_bwd_val(float g, float u, float go, float& grad_gate, float& grad_up) {
  if constexpr (CODE == 1) {
    const float r = fmaxf(g, 0.0f);
    grad_gate = go * u * (2.0f * r);
    grad_up = go * (r * r);
  } else {
    const float s = __fdividef(1.0f, 1.0f + __expf(-g));
    if constexpr (CODE == 5) {
      const float t = __fdividef(2.0f, 1.0f + __expf(-2.0f * g)) - 1.0f;
      const float d = (1.0f - t * t) * s + t * s * (1.0f - s);
      grad_gate = go * u * d;
      grad_up = go * (t * s);
    } else {
      const float d = s * (1.0f + g * (1.0f - s));
      grad_gate = go * u * d;
      grad_up = go * (g * s);
    }
  }
}

// Forward GLU on n packed pairs: pg / pu = bf16-rounded gate / up (the activation reads the rounded values, as the
// reference's separate activation kernel does, kernels/sm75/moe.py:163-184); oh = act(gate) * up
template <int CODE>
__device__ __forceinline__ void glu_fwd_pairs(const uint32_t* pg, const uint32_t* pu, uint32_t* oh, int n) {
#pragma unroll
  for (int i = 0; i < n; ++i) {
    const float2 gf = unpack_bf16x2(pg[i]);
    const float2 uf = unpack_bf16x2(pu[i]);
    oh[i] = pack_bf16x2(glu_fwd_val<CODE>(gf.x, uf.x), glu_fwd_val<CODE>(gf.y, uf.y));
  }
}
template <bool POLY>
__device__ __forceinline__ void glu_fwd_pairs_by_code(int code, const uint32_t* pg, const uint32_t* pu, uint32_t* oh,
                                                      int n) {
  if constexpr (POLY) {
    if (code == 1) return glu_fwd_pairs<1>(pg, pu, oh, n);
    if (code == 5) return glu_fwd_pairs<5>(pg, pu, oh, n);
  }
  glu_fwd_pairs<0>(pg, pu, oh, n);
}

// grad_gate = gi*up*f'(g), grad_up = gi*f(g) for 32 columns; gi (fp32 accumulator)
// is rounded to bf16 first because the reference materialises grad_inter in bf16
template <int CODE>
__device__ __forceinline__ void glu_bwd32_code(const uint32_t (&r)[32], const uint4 (&g)[4], const uint4 (&u)[4],
                                               uint32_t* og, uint32_t* ou) {
#pragma unroll
  for (int v = 0; v < 4; ++v) {
    const uint32_t gw[4] = {g[v].x, g[v].y, g[v].z, g[v].w};
    const uint32_t uw[4] = {u[v].x, u[v].y, u[v].z, u[v].w};
#pragma unroll
    for (int h = 0; h < 4; ++h) {
      const float2 gf = unpack_bf16x2(gw[h]);
      const float2 uf = unpack_bf16x2(uw[h]);
      const float go0 = bf16_round(__uint_as_float(r[v * 8 + 2 * h]));
      const float go1 = bf16_round(__uint_as_float(r[v * 8 + 2 * h + 1]));
      float gg0, gu0, gg1, gu1;
      glu_bwd_val<CODE>(gf.x, uf.x, go0, gg0, gu0);
      glu_bwd_val<CODE>(gf.y, uf.y, go1, gg1, gu1);
      og[4 * v + h] = pack_bf16x2(gg0, gg1);
      ou[4 * v + h] = pack_bf16x2(gu0, gu1);
    }
  }
}
template <bool POLY = false>
__device__ __forceinline__ void glu_bwd32(const uint32_t (&r)[32], const uint4 (&g)[4], const uint4 (&u)[4],
                                          uint32_t* og, uint32_t* ou, int code = 0) {
  if constexpr (POLY) {
    if (code == 1) return glu_bwd32_code<1>(r, g, u, og, ou);
    if (code == 5) return glu_bwd32_code<5>(r, g, u, og, ou);
  }
  glu_bwd32_code<0>(r, g, u, og, ou);
}

// the same with grad_inter already rounded and packed: gi[i] = columns (2i, 2i+1)
__device__ __forceinline__ void glu_bwd32_packed(const uint32_t* gi, const uint4 (&g)[4], const uint4 (&u)[4],
                                                 uint32_t* og, uint32_t* ou) {
#pragma unroll
  for (int v = 0; v < 4; ++v) {
    const uint32_t gw[4] = {g[v].x, g[v].y, g[v].z, g[v].w};
    const uint32_t uw[4] = {u[v].x, u[v].y, u[v].z, u[v].w};
#pragma unroll
    for (int h = 0; h < 4; ++h) {
      const float2 gf = unpack_bf16x2(gw[h]);
      const float2 uf = unpack_bf16x2(uw[h]);
      const float2 go = unpack_bf16x2(gi[4 * v + h]);
      const float s0 = __fdividef(1.0f, 1.0f + __expf(-gf.x));
      const float s1 = __fdividef(1.0f, 1.0f + __expf(-gf.y));
      const float d0 = s0 * (1.0f + gf.x * (1.0f - s0));
      const float d1 = s1 * (1.0f + gf.y * (1.0f - s1));
      og[4 * v + h] = pack_bf16x2(go.x * uf.x * d0, go.y * uf.y * d1);
      ou[4 * v + h] = pack_bf16x2(go.x * (gf.x * s0), go.y * (gf.y * s1));
    }
  }
}

// One lane = one row of a 32-row staging box: 64 bf16 (32 packed registers) go to the 128-byte
// swizzled position the TMA store expects (16-byte chunk j of row r sits at chunk j ^ (r & 7)).
constexpr int kStageOutBytes = 32 * 128;   // one epilogue warp's staging box: 32 rows x 64 bf16

// One lane = one row of a 32-row staging box: 64 bf16 (32 packed registers) go to the 128-byte
// swizzled position the TMA store expects (16-byte chunk j of row r sits at chunk j ^ (r & 7)).
__device__ __forceinline__ void stage_row(uint8_t* buf, int lane, const uint32_t* pk) {
#pragma unroll
  for (int j = 0; j < 8; ++j)
    *reinterpret_cast<uint4*>(buf + lane * 128 + ((j ^ (lane & 7)) << 4)) =
        make_uint4(pk[4 * j], pk[4 * j + 1], pk[4 * j + 2], pk[4 * j + 3]);
}
// make the staged box visible to the async proxy and let lane 0 issue the store
__device__ __forceinline__ void store_box(const CUtensorMap* tm, uint8_t* buf, int lane, int c0, int c1, int c2) {
  fence_proxy_async_smem();
  __syncwarp();
  if (lane == 0) {
    tma_store_3d(tm, smem_u32(buf), c0, c1, c2);
    bulk_commit_group();
  }
}
// the staging box may be overwritten again
__device__ __forceinline__ void staging_free(int lane) {
  if (lane == 0) bulk_wait_read_all();
  __syncwarp();
}

// ---------------------------------------------------------------------------- host side
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*,
                                  CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                  CUtensorMapFloatOOBfill);

static EncodeTiledFn get_encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  });
  return fn;
}

// bf16 (or byte) tensor seen as dims {inner, outer, groups}; strides in elements; 128B (or 64B) swizzle; zero OOB fill.
static int make_map(CUtensorMap* tm, const void* base, uint64_t inner, uint64_t outer, uint64_t groups,
                    uint64_t outer_stride, uint64_t group_stride, uint32_t box_inner, uint32_t box_outer,
                    int elem_bytes = 2, int swizzle_bytes = 128) {
  EncodeTiledFn fn = get_encode_fn();
  B200_CHECK_ARG(fn != nullptr, B200MOE_E_CUDA, "cuTensorMapEncodeTiled entry point not available");
  B200_CHECK_ARG(aligned16(base), B200MOE_E_ALIGN, "tensor base %p is not 16-byte aligned", base);
  B200_CHECK_ARG((outer_stride * elem_bytes) % 16 == 0 && (group_stride * elem_bytes) % 16 == 0, B200MOE_E_ALIGN,
                 "row/group strides must be multiples of 16 bytes (got %llu, %llu elements)",
                 (unsigned long long)outer_stride, (unsigned long long)group_stride);
  cuuint64_t dims[3] = {inner, outer, groups};
  cuuint64_t strides[2] = {outer_stride * elem_bytes, group_stride * elem_bytes};
  cuuint32_t box[3] = {box_inner, box_outer, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = fn(tm, elem_bytes == 2 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE,
                  swizzle_bytes == 0 ? CU_TENSOR_MAP_SWIZZLE_NONE : swizzle_bytes == 64 ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  B200_CHECK_ARG(r == CUDA_SUCCESS, B200MOE_E_CUDA,
                 "cuTensorMapEncodeTiled failed (%d): dims {%llu,%llu,%llu} box {%u,%u}", (int)r,
                 (unsigned long long)inner, (unsigned long long)outer, (unsigned long long)groups, box_inner,
                 box_outer);
  return 0;
}


static inline long long ceil_div(long long a, long long b) { return (a + b - 1) / b; }

}  // namespace b200moe

#define CHECK_DIM8(v) \
  B200_CHECK_ARG((v) > 0 && (v) % 8 == 0, B200MOE_E_BAD_SHAPE, #v " = %lld must be a positive multiple of 8", (long long)(v))
#define CHECK_I32(v) \
  B200_CHECK_ARG((v) >= 0 && (v) < (1LL << 31), B200MOE_E_BAD_SHAPE, #v " = %lld does not fit int32", (long long)(v))
