// MXFP8 GEMM for sm_100a: e4m3 operands with E8M0 block-32 scales, tcgen05.mma.kind::mxf8f6f4
// .block_scale, fp32 accumulation in TMEM, bf16 results.
//
// Both operands are K-major (the quantisers write transposed copies where a GEMM reduces over the
// other dimension).  One CTA computes a 128 x 128 tile; a k-block is 128 elements (one 128-byte
// swizzle row, four MMAs of K = 32).  Per k-block the producer brings in the A and B boxes by TMA
// plus the two 512-byte scale atoms (bulk copies); the MMA thread copies the atoms into tensor
// memory (tcgen05.cp 32x128b.warpx4: lane = row % 32, column = row / 32, byte = k-block % 4) and
// selects the byte with the scale-id fields of the instruction descriptor.
// Schedules and epilogues are the ones of the bf16 kernel (dense / grouped-M / grouped-K; store,
// SwiGLU over 64-interleaved gate|up weight rows, GLU backward).
#include <stdlib.h>

#include "gemm_common.cuh"
#include "mxfp8_quant.cuh"

namespace b200moe {

constexpr int FBN = 128;                 // tile columns
constexpr int FBK = 128;                 // k-block in elements = bytes
constexpr int kATile = BM * FBK;         // 16 KB
constexpr int kBTile = FBN * FBK;        // 16 KB
constexpr int kSfAtom = 512;
constexpr int kFStage = kATile + kBTile + 2 * kSfAtom;   // 33 KB, a multiple of 1024
constexpr int kFStages = 6;
constexpr int kSfTmemBase = 2 * FBN;     // accumulators use columns [0, 256)
constexpr int kFTmemCols = 512;
constexpr int kFSmemBytes = kFStages * kFStage + (2 * kFStages + 4) * 8 + 16 + 1024;

struct Fp8Params {
  GemmParams g;
  const uint8_t* sfa;       // scale atoms of A: row-block major, k-chunk minor
  const uint8_t* sfb;
  int sfa_kc, sfb_kc;       // k-chunks (of 128) per row-block
  int b_rows_per_group;     // rows of B per expert (GROUPED_M), multiple of 128
  // optional: the epilogue also emits its bf16 result quantised along the row (the producer of the
  // next GEMM's A operand): SwiGLU -> inter (I bytes per row), GLU backward -> grad_gate_up (2I per row)
  uint8_t* q_out;
  uint8_t* q_sf;
};

// shared-memory descriptor of a 32 x 16-byte scale atom: no swizzle, 8-row groups 128 bytes apart
__device__ __forceinline__ uint64_t sf_desc(uint32_t smem_addr) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((smem_addr & 0x3FFFF) >> 4);
  d |= static_cast<uint64_t>(128 >> 4) << 32;
  d |= 1ull << 46;
  return d;
}
__device__ __forceinline__ void tmem_cp_sf(uint32_t taddr, uint64_t desc) {
  asm volatile("tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], %1;" ::"r"(taddr), "l"(desc) : "memory");
}
__device__ __forceinline__ void umma_mxf8(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                          uint32_t sfa_tmem, uint32_t sfb_tmem, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %6, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::mxf8f6f4.block_scale [%0], %1, %2, %3, [%4], [%5], p;\n\t}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(sfa_tmem), "r"(sfb_tmem), "r"(accumulate)
      : "memory");
}
// Block-scaled instruction descriptor: e4m3 A/B (format 0), K-major, E8M0 scales.
//   bits 4-5 B scale id   bits 7-9 A format   bits 10-12 B format   bits 17-22 N >> 3
//   bit 23 scale format (1 = E8M0)   bits 24-28 M >> 4   bits 29-30 A scale id
__device__ __forceinline__ uint32_t idesc_mxf8(int n, uint32_t sf_id) {
  return (sf_id << 4) | (static_cast<uint32_t>(n >> 3) << 17) | (1u << 23) |
         (static_cast<uint32_t>(BM >> 4) << 24) | (sf_id << 29);
}

template <int EPI>
__global__ void __launch_bounds__(kThreads, 1)
gemm_mxfp8_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                  const Fp8Params fp) {
  const GemmParams& p = fp.g;
  constexpr int TN = FBN;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + kFStages * kFStage);
  const uint32_t bar_full = smem_u32(bars);
  const uint32_t bar_empty = smem_u32(bars + kFStages);
  const uint32_t bar_tfull = smem_u32(bars + 2 * kFStages);
  const uint32_t bar_tempty = smem_u32(bars + 2 * kFStages + 2);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * kFStages + 4);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kFStages; ++s) {
      mbar_init(bar_full + 8 * s, 1);
      mbar_init(bar_empty + 8 * s, 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(bar_tfull + 8 * b, 1);
      mbar_init(bar_tempty + 8 * b, kEpiWarps);
    }
    *abort_flag = 0;
    fence_mbar_init();
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmB);
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(tmem_slot), kFTmemCols);
    tmem_relinquish();
  }
  __shared__ int s_order[B200MOE_MAX_EXPERTS];
  const int* order = build_group_order(p, s_order);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const int total = total_tiles(p, TN, BM);

  if (warp == 0) {
    if (lane == 0) {   // ---------------------------------------------------------- producer
      int s = 0;
      uint32_t ph = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < total && ok; tile += gridDim.x) {
        const Tile t = get_tile(p, tile, TN, BM, FBK, order);
        const int gB = (p.sched == SCHED_GROUPED_M) ? t.g : 0;
        const long long rb_a = t.m0 >> 7;
        const long long rb_b = (static_cast<long long>(gB) * fp.b_rows_per_group + t.n0) >> 7;
        for (int kb = 0; kb < t.nkb; ++kb) {
          if (!mbar_wait(bar_empty + 8 * s, ph ^ 1, abort_flag, ST_WAIT_PRODUCER)) {
            ok = false;
            break;
          }
          const uint32_t full = bar_full + 8 * s;
          mbar_arrive_expect_tx(full, kFStage);
          const uint32_t sa = smem_u32(smem + s * kFStage);
          const int kk = t.k0 + kb * FBK;
          const long long kc = kk >> 7;
          tma_load_3d(sa, &tmA, full, kk, t.m0, 0);
          tma_load_3d(sa + kATile, &tmB, full, kk, t.n0, gB);
          bulk_load_1d(sa + kATile + kBTile, fp.sfa + (rb_a * fp.sfa_kc + kc) * kSfAtom, kSfAtom, full);
          bulk_load_1d(sa + kATile + kBTile + kSfAtom, fp.sfb + (rb_b * fp.sfb_kc + kc) * kSfAtom, kSfAtom, full);
          if (++s == kFStages) {
            s = 0;
            ph ^= 1;
          }
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {   // ---------------------------------------------------------- MMA issuer
      int s = 0, it = 0;
      uint32_t ph = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < total && ok; tile += gridDim.x, ++it) {
        const Tile t = get_tile(p, tile, TN, BM, FBK, order);
        const int buf = it & 1;
        if (!mbar_wait(bar_tempty + 8 * buf, ((it >> 1) & 1) ^ 1, abort_flag, ST_WAIT_MMA_TMEM)) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + buf * FBN;
        for (int kb = 0; kb < t.nkb; ++kb) {
          if (!mbar_wait(bar_full + 8 * s, ph, abort_flag, ST_WAIT_MMA_FULL)) {
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t sa = smem_u32(smem + s * kFStage);
          const uint32_t sb = sa + kATile;
          const uint32_t sfa_t = tmem_base + kSfTmemBase + 8 * s;
          const uint32_t sfb_t = sfa_t + 4;
          tmem_cp_sf(sfa_t, sf_desc(sa + kATile + kBTile));
          tmem_cp_sf(sfb_t, sf_desc(sa + kATile + kBTile + kSfAtom));
#pragma unroll
          for (int k = 0; k < FBK / 32; ++k) {
            const uint64_t da = umma_desc_sw128(sa + k * 32, 0, 1024);
            const uint64_t db = umma_desc_sw128(sb + k * 32, 0, 1024);
            umma_mxf8(d_tmem, da, db, idesc_mxf8(FBN, k), sfa_t, sfb_t, (kb | k) != 0);
          }
          umma_commit(bar_empty + 8 * s);
          if (++s == kFStages) {
            s = 0;
            ph ^= 1;
          }
        }
        if (!ok) break;
        if (t.nkb > 0) umma_commit(bar_tfull + 8 * buf);
        else mbar_arrive(bar_tfull + 8 * buf);
      }
    }
  } else {   // ---------------------------------------------------------------------- epilogue
    const int q = warp & 3;
    const int half = (warp - 2) >> 2;
    int it = 0;
    for (int tile = blockIdx.x; tile < total; tile += gridDim.x, ++it) {
      const Tile t = get_tile(p, tile, TN, BM, FBK, order);
      const int buf = it & 1;
      if (!mbar_wait(bar_tfull + 8 * buf, (it >> 1) & 1, abort_flag, ST_WAIT_EPILOGUE)) break;
      __syncwarp();
      tc_fence_after();
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + buf * FBN;
      const long long row = static_cast<long long>(t.m0) + q * 32 + lane;
      const bool have_acc = t.nkb > 0;
      if constexpr (EPI == EPI_STORE) {
        const bool row_ok = (p.sched == SCHED_GROUPED_M) || (row < p.M);
        const long long base = (p.sched == SCHED_GROUPED_K ? t.g * p.d_group_stride : 0) + row * p.ldd + t.n0;
#pragma unroll 1
        for (int c0 = half * 64; c0 < half * 64 + 64; c0 += 32) {
          if (t.n0 + c0 >= p.N) break;
          uint32_t r[32];
          if (have_acc) {
            tmem_ld32(taddr + c0, r);
            tmem_ld_wait();
          } else {
#pragma unroll
            for (int i = 0; i < 32; ++i) r[i] = 0u;
          }
          if (row_ok) {
            __nv_bfloat16* d = reinterpret_cast<__nv_bfloat16*>(p.D) + base + c0;
#pragma unroll
            for (int v = 0; v < 4; ++v)
              if (t.n0 + c0 + v * 8 < p.N) *reinterpret_cast<uint4*>(d + v * 8) = pack8(r + v * 8);
          }
        }
      } else if constexpr (EPI == EPI_SWIGLU) {
        // weight rows are 64-interleaved: accumulator columns [0,64) = gate, [64,128) = up of the
        // intermediate columns [n0/2, n0/2 + 64); this warp handles 32 of them
        const int I = p.I;
        const int col0 = t.n0 / 2 + half * 32;
        if (col0 < I) {
          __nv_bfloat16* gu = reinterpret_cast<__nv_bfloat16*>(p.D) + row * (2LL * I);
          __nv_bfloat16* it_out = reinterpret_cast<__nv_bfloat16*>(p.aux) + row * static_cast<long long>(I);
          uint32_t g[32], u[32], hq[16];
          tmem_ld32(taddr + half * 32, g);
          tmem_ld32(taddr + 64 + half * 32, u);
          tmem_ld_wait();
#pragma unroll
          for (int v = 0; v < 4; ++v) {
            const int col = col0 + v * 8;
            if (col < I) {
              uint32_t og[4], ou[4], oh[4];
#pragma unroll
              for (int h = 0; h < 4; ++h) {
                og[h] = pack_bf16x2(__uint_as_float(g[v * 8 + 2 * h]), __uint_as_float(g[v * 8 + 2 * h + 1]));
                ou[h] = pack_bf16x2(__uint_as_float(u[v * 8 + 2 * h]), __uint_as_float(u[v * 8 + 2 * h + 1]));
                const float2 gf = unpack_bf16x2(og[h]);
                const float2 uf = unpack_bf16x2(ou[h]);
                const float s0 = __fdividef(1.0f, 1.0f + __expf(-gf.x));
                const float s1 = __fdividef(1.0f, 1.0f + __expf(-gf.y));
                oh[h] = pack_bf16x2(gf.x * s0 * uf.x, gf.y * s1 * uf.y);
              }
              *reinterpret_cast<uint4*>(gu + col) = make_uint4(og[0], og[1], og[2], og[3]);
              *reinterpret_cast<uint4*>(gu + I + col) = make_uint4(ou[0], ou[1], ou[2], ou[3]);
              *reinterpret_cast<uint4*>(it_out + col) = make_uint4(oh[0], oh[1], oh[2], oh[3]);
#pragma unroll
              for (int h = 0; h < 4; ++h) hq[4 * v + h] = oh[h];
            }
          }
          if (fp.q_out != nullptr)   // I % 128 == 0: a chunk is one whole 32-element block of the row
            mx_quant_store32(hq, fp.q_out + row * static_cast<long long>(I) + col0, fp.q_sf, row, col0 >> 5, I >> 7);
        }
      } else {   // EPI_GLU_BWD: accumulator = grad_inter columns [n0, n0+128), this warp 64 of them
        const int I = p.I;
        const __nv_bfloat16* gu = reinterpret_cast<const __nv_bfloat16*>(p.aux) + row * (2LL * I);
        __nv_bfloat16* ggu = reinterpret_cast<__nv_bfloat16*>(p.D) + row * (2LL * I);
#pragma unroll 1
        for (int c0 = half * 64; c0 < half * 64 + 64; c0 += 32) {
          if (t.n0 + c0 >= I) break;
          uint4 g4[4], u4[4];
#pragma unroll
          for (int v = 0; v < 4; ++v) {
            const int col = t.n0 + c0 + v * 8;
            g4[v] = col < I ? __ldg(reinterpret_cast<const uint4*>(gu + col)) : make_uint4(0u, 0u, 0u, 0u);
            u4[v] = col < I ? __ldg(reinterpret_cast<const uint4*>(gu + I + col)) : make_uint4(0u, 0u, 0u, 0u);
          }
          uint32_t r[32], og[16], ou[16];
          tmem_ld32(taddr + c0, r);
          tmem_ld_wait();
          glu_bwd32(r, g4, u4, og, ou);
          if (fp.q_out != nullptr) {   // blocks of the (rows, 2I) grad_gate_up: gate half, then up half
            const int colq = t.n0 + c0;
            mx_quant_store32(og, fp.q_out + row * (2LL * I) + colq, fp.q_sf, row, colq >> 5, (2 * I) >> 7);
            mx_quant_store32(ou, fp.q_out + row * (2LL * I) + I + colq, fp.q_sf, row, (I + colq) >> 5, (2 * I) >> 7);
          }
#pragma unroll
          for (int v = 0; v < 4; ++v) {
            const int col = t.n0 + c0 + v * 8;
            if (col < I) {
              *reinterpret_cast<uint4*>(ggu + col) = make_uint4(og[4 * v], og[4 * v + 1], og[4 * v + 2], og[4 * v + 3]);
              *reinterpret_cast<uint4*>(ggu + I + col) = make_uint4(ou[4 * v], ou[4 * v + 1], ou[4 * v + 2], ou[4 * v + 3]);
            }
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_tempty + 8 * buf);
    }
  }

  tc_fence_before();
  __syncthreads();
  if (threadIdx.x == 0 && *abort_flag != 0 && p.status != nullptr) atomicCAS(p.status, 0, *abort_flag);
  if (warp == 1) {
    __syncwarp();
    tc_fence_after();
    tmem_dealloc(tmem_base, kFTmemCols);
  }
}

// ---------------------------------------------------------------------------------------------
// Pair variant: a cluster of two CTAs computes a 256 x 256 tile with cta_group::2 block-scaled MMAs.
// Each CTA stages its own 128 rows of A, its own 128 rows of B, the scale atom of its A rows and both
// scale atoms of the tile's B rows (every CTA needs the scales of all 256 columns).  The 256-column
// accumulator plus the scale columns fill tensor memory, so the accumulator is single-buffered: the
// epilogue of a tile runs while the producer already refills the stages of the next one.
constexpr int PBN = 256;
constexpr int kPStage = 34816;           // A 16 KB + B 16 KB + SFA 512 B + SFB 1 KB, rounded to 1 KB
// GLU backward keeps two boxes per epilogue warp (gate and up: loaded by TMA, overwritten in place, stored by
// TMA) and therefore one stage less
template <int EPI> struct PairCfg {
  static constexpr int kStages = (EPI == EPI_GLU_BWD) ? 4 : 5;
  static constexpr int kEpiBytes = kEpiWarps * kStageOutBytes * ((EPI == EPI_GLU_BWD) ? 2 : 1);
  // barriers: full, empty, sf per stage; tfull, tempty; two per epilogue warp (GLU-backward load sets)
  static constexpr int kSmemBytes = kStages * kPStage + kEpiBytes +
                                    (3 * kStages + 2 + 2 * kEpiWarps) * 8 + 16 + 1024;
};
constexpr int kPSfCols = 16;             // tensor-memory columns per stage: SFA 4 + SFB 8 (+4 spare)
constexpr int kPThreads = kThreads + 32;   // one more warp: the scale-copy issuer

// pair form of the 3-D load for the scale tensors {128 u32, k-chunks, row-blocks}
__device__ __forceinline__ void umma_mxf8_pair(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                               uint32_t sfa_tmem, uint32_t sfb_tmem, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %6, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::mxf8f6f4.block_scale [%0], %1, %2, %3, [%4], [%5], p;\n\t}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(sfa_tmem), "r"(sfb_tmem), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void tmem_cp_sf_pair(uint32_t taddr, uint64_t desc) {
  asm volatile("tcgen05.cp.cta_group::2.32x128b.warpx4 [%0], %1;" ::"r"(taddr), "l"(desc) : "memory");
}
__device__ __forceinline__ uint32_t idesc_mxf8_pair(uint32_t sf_id) {
  return (sf_id << 4) | (static_cast<uint32_t>(PBN >> 3) << 17) | (1u << 23) |
         (static_cast<uint32_t>(256 >> 4) << 24) | (sf_id << 29);
}

template <int EPI>
__global__ void __launch_bounds__(kPThreads, 1)
gemm_mxfp8_pair_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                       const __grid_constant__ CUtensorMap tmSFA, const __grid_constant__ CUtensorMap tmSFB,
                       const __grid_constant__ CUtensorMap tmD, const __grid_constant__ CUtensorMap tmD2,
                       const Fp8Params fp) {
  const GemmParams& p = fp.g;
  constexpr int TN = PBN, TM = 2 * BM;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  constexpr int kPStages = PairCfg<EPI>::kStages;
  constexpr int kPEpiBytes = PairCfg<EPI>::kEpiBytes;
  uint8_t* epi_smem = smem + kPStages * kPStage;          // 1 KB aligned: stages are multiples of 1 KB
  uint64_t* bars = reinterpret_cast<uint64_t*>(epi_smem + kPEpiBytes);
  const uint32_t bar_full = smem_u32(bars);
  const uint32_t bar_empty = smem_u32(bars + kPStages);
  const uint32_t bar_sf = smem_u32(bars + 2 * kPStages);   // scales of the stage are in tensor memory
  const uint32_t bar_tfull = smem_u32(bars + 3 * kPStages);
  const uint32_t bar_tempty = smem_u32(bars + 3 * kPStages + 1);
  const uint32_t bar_epi = smem_u32(bars + 3 * kPStages + 2);   // two per epilogue warp: GLU-backward loads landed
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 3 * kPStages + 2 + 2 * kEpiWarps);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int cta_rank = static_cast<int>(cluster_ctarank());
  const int first_tile = static_cast<int>(cluster_id_x());
  const int tile_step = static_cast<int>(num_clusters_x());

  if (threadIdx.x == 0) {
    for (int s = 0; s < kPStages; ++s) {
      mbar_init(bar_full + 8 * s, 1);
      mbar_init(bar_empty + 8 * s, 1);
      mbar_init(bar_sf + 8 * s, 1);
    }
    mbar_init(bar_tfull, 1);
    mbar_init(bar_tempty, 2 * kEpiWarps);
    for (int i = 0; i < 2 * kEpiWarps; ++i) mbar_init(bar_epi + 8 * i, 1);
    *abort_flag = 0;
    fence_mbar_init();
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmB);
    tma_prefetch_desc(&tmSFA);
    tma_prefetch_desc(&tmSFB);
  }
  if (warp == 1) {
    tmem_alloc_pair(smem_u32(tmem_slot), kFTmemCols);
    tmem_relinquish_pair();
  }
  __shared__ int s_order[B200MOE_MAX_EXPERTS];
  const int* order = build_group_order(p, s_order);
  tc_fence_before();
  __syncthreads();
  __syncwarp();
  cluster_sync_all();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const int total = total_tiles(p, TN, TM);

  if (warp == 0) {
    // ------------------------------------------------------------------------------ producer (each CTA)
    // The four boxes of a stage (A, B, the A scale atom, the two B scale atoms) are issued by four lanes in ONE
    // instruction, each lane with its own tensor map, destination and coordinates: four instructions from one lane
    // took longer than the MMAs of a stage, and the ring ran dry.
    if (lane < 4) {
      const CUtensorMap* tm = lane == 0 ? &tmA : lane == 1 ? &tmB : lane == 2 ? &tmSFA : &tmSFB;
      const uint32_t dst_off = lane == 0 ? 0u : lane == 1 ? kATile : lane == 2 ? kATile + kBTile : kATile + kBTile + kSfAtom;
      const uint32_t full0 = mapa_shared(bar_full, 0);              // the leader's barrier counts both CTAs
      const bool expects = (lane == 0 && cta_rank == 0);
      int s = 0;
      uint32_t ph = 0;
      bool ok = true;
      for (int tile = first_tile; tile < total && ok; tile += tile_step) {
        const Tile t = get_tile(p, tile, TN, TM, FBK, order);
        const int gB = (p.sched == SCHED_GROUPED_M) ? t.g : 0;
        const int m0 = t.m0 + BM * cta_rank;
        const int rb_a = m0 >> 7;
        const int rb_b = static_cast<int>((static_cast<long long>(gB) * fp.b_rows_per_group + t.n0) >> 7);
        // data boxes: (k, row, group); scale atoms: (0, k chunk of 128, 128-row block)
        const int c1_fixed = lane == 0 ? m0 : t.n0 + 128 * cta_rank;
        const int c2 = lane == 0 ? 0 : lane == 1 ? gB : lane == 2 ? rb_a : rb_b;
        for (int kb = 0; kb < t.nkb; ++kb) {
          if (!mbar_wait(bar_empty + 8 * s, ph ^ 1, abort_flag, ST_WAIT_PRODUCER)) {
            ok = false;
            break;
          }
          if (expects) mbar_arrive_expect_tx(bar_full + 8 * s, 2 * (kATile + kBTile + 3 * kSfAtom));
          const int kk = t.k0 + kb * FBK;
          tma_load_3d_pair(smem_u32(smem + s * kPStage) + dst_off, tm, full0 + 8 * s, lane < 2 ? kk : 0,
                           lane < 2 ? c1_fixed : (kk >> 7), c2);
          if (++s == kPStages) {
            s = 0;
            ph ^= 1;
          }
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0 && cta_rank == 0) {   // --------------------------------------------- MMA issuer (leader)
      int s = 0, it = 0;
      uint32_t ph = 0;
      bool ok = true;
      for (int tile = first_tile; tile < total && ok; tile += tile_step, ++it) {
        const Tile t = get_tile(p, tile, TN, TM, FBK, order);
        if (!mbar_wait(bar_tempty, (it & 1) ^ 1, abort_flag, ST_WAIT_MMA_TMEM)) break;
        tc_fence_after();
        for (int kb = 0; kb < t.nkb; ++kb) {
          // operands landed in shared memory (full) and the scale-copy warp moved the scales to tensor memory (sf)
          if (!mbar_wait(bar_full + 8 * s, ph, abort_flag, ST_WAIT_MMA_FULL) ||
              !mbar_wait(bar_sf + 8 * s, ph, abort_flag, ST_WAIT_MMA_FULL)) {
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t sa = smem_u32(smem + s * kPStage);
          const uint32_t sb = sa + kATile;
          const uint32_t sfa_t = tmem_base + PBN + kPSfCols * s;
          const uint32_t sfb_t = sfa_t + 4;
#pragma unroll
          for (int k = 0; k < FBK / 32; ++k) {
            const uint64_t da = umma_desc_sw128(sa + k * 32, 0, 1024);
            const uint64_t db = umma_desc_sw128(sb + k * 32, 0, 1024);
            umma_mxf8_pair(tmem_base, da, db, idesc_mxf8_pair(k), sfa_t, sfb_t, (kb | k) != 0);
          }
          umma_commit_pair(bar_empty + 8 * s);
          if (++s == kPStages) {
            s = 0;
            ph ^= 1;
          }
        }
        if (!ok) break;
        if (t.nkb > 0) {
          umma_commit_pair(bar_tfull);
        } else {
          mbar_arrive(bar_tfull);
          mbar_arrive_cluster(mapa_shared(bar_tfull, 1));
        }
      }
    }
  } else if (warp == 2 + kEpiWarps) {
    // ------------------------------------------------------------------------- scale-copy issuer (leader)
    // The three scale atoms of a stage go from shared to tensor memory (tcgen05.cp) from a thread of their
    // own, stages ahead of the MMAs, instead of in the MMA thread's instruction stream directly before the
    // MMAs that read them.  A stage's scale columns are free again once the stage itself was refilled: the
    // producer waited for the commit that followed the MMAs reading them.
    if (lane == 0 && cta_rank == 0) {
      int s = 0;
      uint32_t ph = 0;
      bool ok = true;
      for (int tile = first_tile; tile < total && ok; tile += tile_step) {
        const int nkb = get_tile(p, tile, TN, TM, FBK, order).nkb;
        for (int kb = 0; kb < nkb; ++kb) {
          if (!mbar_wait(bar_full + 8 * s, ph, abort_flag, ST_WAIT_MMA_FULL)) {
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t sf_s = smem_u32(smem + s * kPStage) + kATile + kBTile;
          const uint32_t sfa_t = tmem_base + PBN + kPSfCols * s;
          tmem_cp_sf_pair(sfa_t, sf_desc(sf_s));
          tmem_cp_sf_pair(sfa_t + 4, sf_desc(sf_s + kSfAtom));
          tmem_cp_sf_pair(sfa_t + 8, sf_desc(sf_s + 2 * kSfAtom));
          umma_commit_pair_local(bar_sf + 8 * s);
          if (++s == kPStages) {
            s = 0;
            ph ^= 1;
          }
        }
      }
    }
  } else {   // ---------------------------------------------------------------------- epilogue
    const int q = warp & 3;
    const int half = (warp - 2) >> 2;    // columns [128*half, 128*half + 128) of the tile
    const uint32_t tempty_leader = mapa_shared(bar_tempty, 0);
    uint32_t epi_phase = 0;   // parity of this warp's GLU-backward load barrier
    int it = 0;
    for (int tile = first_tile; tile < total; tile += tile_step, ++it) {
      const Tile t = get_tile(p, tile, TN, TM, FBK, order);
      const int row0 = t.m0 + BM * cta_rank + q * 32;
      const long long row = static_cast<long long>(row0) + lane;
      // GLU backward works on four 32-column sub-chunks per warp with two sets of (gate, up) boxes of 32 rows x
      // 32 columns (2 KB, 64-byte swizzle): a set is loaded by TMA, overwritten in place with grad_gate /
      // grad_up and stored by TMA while the other set is loading or being computed on.  The saved gate/up
      // values do not depend on the accumulator, so the first two loads go out before the MMAs are waited for.
      constexpr int kGluBox = 32 * 64;
      const int glu_col0 = t.n0 + half * 128;
      uint8_t* ebuf = epi_smem + (warp - 2) * (kPEpiBytes / kEpiWarps);
      const uint32_t ebar = bar_epi + 16 * (warp - 2);   // + 8 * set
      auto glu_load = [&](int sub) {   // tmD2 = saved gate_up seen as {I, rows, 2}, box {32, 32}
        const int set = sub & 1;
        if (lane == 0) {
          mbar_arrive_expect_tx(ebar + 8 * set, 2 * kGluBox);
          tma_load_3d(smem_u32(ebuf + set * 2 * kGluBox), &tmD2, ebar + 8 * set, glu_col0 + 32 * sub, row0, 0);
          tma_load_3d(smem_u32(ebuf + set * 2 * kGluBox + kGluBox), &tmD2, ebar + 8 * set, glu_col0 + 32 * sub, row0, 1);
        }
      };
      uint8_t* bufG = ebuf;   // staging box of the other epilogues
      if constexpr (EPI == EPI_GLU_BWD) {
        staging_free(lane);   // the previous tile's stores out of these boxes have been read
        if (glu_col0 < p.I) glu_load(0);
        if (glu_col0 + 32 < p.I) glu_load(1);
      }
      if (!mbar_wait(bar_tfull, it & 1, abort_flag, ST_WAIT_EPILOGUE)) break;
      __syncwarp();
      tc_fence_after();
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(q * 32) << 16);
      const bool have_acc = t.nkb > 0;
      uint8_t* sbuf = bufG;   // this warp's staging box
      const int grp = (p.sched == SCHED_GROUPED_K) ? t.g : 0;
      // The accumulator is single-buffered, so it is drained first: this warp's 32 rows x 128 columns are
      // rounded to bf16, packed into 64 registers, and the tensor memory goes back to the MMA warp before any
      // arithmetic or store; acc[16 s + i] = columns (32 s + 2i, 32 s + 2i + 1) of this warp's column half.
      uint32_t acc[64];
#pragma unroll
      for (int s2 = 0; s2 < 2; ++s2) {   // two tensor-memory loads in flight per wait
        uint32_t r0[32], r1[32];
        if (have_acc) {
          tmem_ld32(taddr + 128 * half + 64 * s2, r0);
          tmem_ld32(taddr + 128 * half + 64 * s2 + 32, r1);
          tmem_ld_wait();
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) r0[i] = r1[i] = 0u;
        }
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          acc[32 * s2 + i] = pack_bf16x2(__uint_as_float(r0[2 * i]), __uint_as_float(r0[2 * i + 1]));
          acc[32 * s2 + 16 + i] = pack_bf16x2(__uint_as_float(r1[2 * i]), __uint_as_float(r1[2 * i + 1]));
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(tempty_leader);
      // results are staged per warp as 32 rows x 64 columns and written by TMA stores (which clip at the
      // tensor's bounds)
      if constexpr (EPI == EPI_STORE) {
#pragma unroll
        for (int cc = 0; cc < 2; ++cc) {
          const int c = half * 128 + 64 * cc;
          if (t.n0 + c < p.N) {
            staging_free(lane);
            stage_row(sbuf, lane, acc + 32 * cc);
            store_box(&tmD, sbuf, lane, t.n0 + c, row0, grp);
          }
        }
      } else if constexpr (EPI == EPI_SWIGLU) {
        // weight rows are 64-interleaved: accumulator columns [128h, 128h+64) = gate and [128h+64, 128h+128) = up
        // of the intermediate columns [n0/2 + 64h, n0/2 + 64h + 64)
        const int I = p.I;
        const int col0 = t.n0 / 2 + 64 * half;
        if (col0 < I) {
          uint32_t oh[32];
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            const float2 gf = unpack_bf16x2(acc[i]);
            const float2 uf = unpack_bf16x2(acc[32 + i]);
            const float s0 = __fdividef(1.0f, 1.0f + __expf(-gf.x));
            const float s1 = __fdividef(1.0f, 1.0f + __expf(-gf.y));
            oh[i] = pack_bf16x2(gf.x * s0 * uf.x, gf.y * s1 * uf.y);
          }
          if (fp.q_out != nullptr) {   // the quantised `inter` for the down GEMM, two 32-element blocks
            mx_quant_store32(oh, fp.q_out + row * static_cast<long long>(I) + col0, fp.q_sf, row, col0 >> 5, I >> 7);
            mx_quant_store32(oh + 16, fp.q_out + row * static_cast<long long>(I) + col0 + 32, fp.q_sf, row,
                             (col0 + 32) >> 5, I >> 7);
          }
          staging_free(lane);
          stage_row(sbuf, lane, acc);
          store_box(&tmD, sbuf, lane, col0, row0, 0);    // gate half of gate_up
          staging_free(lane);
          stage_row(sbuf, lane, acc + 32);
          store_box(&tmD, sbuf, lane, col0, row0, 1);    // up half
          staging_free(lane);
          stage_row(sbuf, lane, oh);
          store_box(&tmD2, sbuf, lane, col0, row0, 0);   // inter
        }
      } else {   // EPI_GLU_BWD: accumulator = grad_inter columns [n0, n0+256), this warp 128 of them
        const int I = p.I;
        bool live = true;
#pragma unroll
        for (int sub = 0; sub < 4; ++sub) {
          const int col = glu_col0 + 32 * sub;
          live = live && col < I;                      // warp-uniform
          if (!live) continue;
          const int set = sub & 1;
          uint8_t* bG = ebuf + set * 2 * kGluBox;
          uint8_t* bU = bG + kGluBox;
          if (!mbar_wait(ebar + 8 * set, (epi_phase >> set) & 1u, abort_flag, ST_WAIT_EPILOGUE)) {
            live = false;
            continue;
          }
          epi_phase ^= 1u << set;
          uint4 g4[4], u4[4];
#pragma unroll
          for (int v = 0; v < 4; ++v) {              // this lane's row: 64 bytes, 64-byte swizzle
            const int off = lane * 64 + ((v ^ ((lane >> 1) & 3)) << 4);
            g4[v] = *reinterpret_cast<const uint4*>(bG + off);
            u4[v] = *reinterpret_cast<const uint4*>(bU + off);
          }
          uint32_t og[16], ou[16];
          glu_bwd32_packed(acc + 16 * sub, g4, u4, og, ou);
          if (fp.q_out != nullptr) {   // blocks of the (rows, 2I) grad_gate_up: gate half, then up half
            mx_quant_store32(og, fp.q_out + row * (2LL * I) + col, fp.q_sf, row, col >> 5, (2 * I) >> 7);
            mx_quant_store32(ou, fp.q_out + row * (2LL * I) + I + col, fp.q_sf, row, (I + col) >> 5, (2 * I) >> 7);
          }
#pragma unroll
          for (int v = 0; v < 4; ++v) {              // results replace the inputs in place
            const int off = lane * 64 + ((v ^ ((lane >> 1) & 3)) << 4);
            *reinterpret_cast<uint4*>(bG + off) = make_uint4(og[4 * v], og[4 * v + 1], og[4 * v + 2], og[4 * v + 3]);
            *reinterpret_cast<uint4*>(bU + off) = make_uint4(ou[4 * v], ou[4 * v + 1], ou[4 * v + 2], ou[4 * v + 3]);
          }
          fence_proxy_async_smem();
          __syncwarp();
          if (lane == 0) {
            tma_store_3d(&tmD, smem_u32(bG), col, row0, 0);   // grad_gate
            tma_store_3d(&tmD, smem_u32(bU), col, row0, 1);   // grad_up
            bulk_commit_group();
          }
          // once that store has read its boxes they are reloaded with the sub-chunk after the next one
          if (sub + 2 < 4 && glu_col0 + 32 * (sub + 2) < I) {
            staging_free(lane);
            glu_load(sub + 2);
          }
        }
      }
    }
    if (lane == 0) bulk_wait_all();   // every TMA store of this warp has completed
  }

  tc_fence_before();
  __syncthreads();
  __syncwarp();
  cluster_sync_all();
  if (threadIdx.x == 0 && *abort_flag != 0 && p.status != nullptr) atomicCAS(p.status, 0, *abort_flag);
  if (warp == 1) {
    __syncwarp();
    tc_fence_after();
    tmem_dealloc_pair(tmem_base, kFTmemCols);
  }
}

// scale atoms seen as a {128 x u32, k-chunks, row-blocks} tensor, no swizzle; box = `atoms` row-blocks
static int map_sf(CUtensorMap* tm, const void* sf, long long row_blocks, long long k_chunks, int atoms) {
  EncodeTiledFn fn = get_encode_fn();
  B200_CHECK_ARG(fn != nullptr, B200MOE_E_CUDA, "cuTensorMapEncodeTiled entry point not available");
  B200_CHECK_ARG(aligned16(sf), B200MOE_E_ALIGN, "scale buffer is not 16-byte aligned");
  cuuint64_t dims[3] = {128, (cuuint64_t)k_chunks, (cuuint64_t)row_blocks};
  cuuint64_t strides[2] = {512, (cuuint64_t)k_chunks * 512};
  cuuint32_t box[3] = {128, 1, (cuuint32_t)atoms};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = fn(tm, CU_TENSOR_MAP_DATA_TYPE_UINT32, 3, const_cast<void*>(sf), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  B200_CHECK_ARG(r == CUDA_SUCCESS, B200MOE_E_CUDA, "cuTensorMapEncodeTiled(scales) failed (%d)", (int)r);
  return 0;
}

template <int EPI>
static int launch_fp8_pair(const CUtensorMap& tmA, const CUtensorMap& tmB, const CUtensorMap& tmSFA,
                           const CUtensorMap& tmSFB, const CUtensorMap& tmD, const CUtensorMap& tmD2,
                           const Fp8Params& fp, int max_tiles, cudaStream_t stream) {
  static std::once_flag once;
  static cudaError_t attr_err = cudaSuccess;
  std::call_once(once, [] {
    attr_err = cudaFuncSetAttribute(gemm_mxfp8_pair_kernel<EPI>, cudaFuncAttributeMaxDynamicSharedMemorySize, PairCfg<EPI>::kSmemBytes);
  });
  if (attr_err != cudaSuccess) return cuda_fail(attr_err, "cudaFuncSetAttribute(max dynamic smem)");
  int pairs = gemm_cta_budget() / 2;
  if (max_tiles > 0 && max_tiles < pairs) pairs = max_tiles;
  if (pairs < 1) pairs = 1;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(pairs * 2, 1, 1);
  cfg.blockDim = dim3(kPThreads, 1, 1);
  cfg.dynamicSmemBytes = PairCfg<EPI>::kSmemBytes;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  B200_CUDA(cudaLaunchKernelEx(&cfg, gemm_mxfp8_pair_kernel<EPI>, tmA, tmB, tmSFA, tmSFB, tmD, tmD2, fp));
  return 0;
}

// B200MOE_MXFP8_1CTA=1 keeps the single-CTA 128x128 tiles (A/B measurements)
static bool fp8_pairs_enabled() {
  static int v = -1;
  static std::once_flag once;
  std::call_once(once, [] {
    const char* e = getenv("B200MOE_MXFP8_1CTA");
    v = (e != nullptr && e[0] == '1') ? 0 : 1;
  });
  return v == 1;
}

template <int EPI>
static int launch_fp8(const CUtensorMap& tmA, const CUtensorMap& tmB, const Fp8Params& fp, int max_tiles,
                      cudaStream_t stream) {
  static std::once_flag once;
  static cudaError_t attr_err = cudaSuccess;
  std::call_once(once, [] {
    attr_err = cudaFuncSetAttribute(gemm_mxfp8_kernel<EPI>, cudaFuncAttributeMaxDynamicSharedMemorySize, kFSmemBytes);
  });
  if (attr_err != cudaSuccess) return cuda_fail(attr_err, "cudaFuncSetAttribute(max dynamic smem)");
  int grid = gemm_cta_budget();
  if (max_tiles > 0 && max_tiles < grid) grid = max_tiles;
  if (grid < 1) grid = 1;
  gemm_mxfp8_kernel<EPI><<<grid, kThreads, kFSmemBytes, stream>>>(tmA, tmB, fp);
  B200_CUDA(cudaGetLastError());
  return 0;
}

// byte tensor {K, rows, groups}, box {128 bytes, 128 rows}
static int map_fp8(CUtensorMap* tm, const void* q, long long rows, long long K, long long groups) {
  return make_map(tm, q, K, rows, groups, K, rows * K, FBK, 128, 1);
}

// Launch with pair tiles when the output is at least one 256-wide tile (and pairs are enabled).
template <int EPI>
static int launch_any(const void* Aq, long long a_rows, const void* Bq, long long b_rows, long long b_groups,
                      long long K, const Fp8Params& fp, int max_tiles_1cta, cudaStream_t stream) {
  CUtensorMap tmA, tmB;
  int rc = map_fp8(&tmA, Aq, a_rows, K, 1);
  if (rc) return rc;
  rc = map_fp8(&tmB, Bq, b_rows, K, b_groups);
  if (rc) return rc;
  const bool pair = fp8_pairs_enabled() && fp.g.N >= PBN && fp.g.N % 128 == 0 &&
                    (fp.g.sched != SCHED_DENSE || fp.g.M >= 256);
  if (!pair) return launch_fp8<EPI>(tmA, tmB, fp, max_tiles_1cta, stream);
  CUtensorMap tmSFA, tmSFB;
  rc = map_sf(&tmSFA, fp.sfa, ceil_div(a_rows, 128), fp.sfa_kc, 1);
  if (rc) return rc;
  rc = map_sf(&tmSFB, fp.sfb, ceil_div(b_rows * b_groups, 128), fp.sfb_kc, 2);
  if (rc) return rc;
  // bf16 outputs as {columns, rows, groups} tensors, box {64, 32}, for the TMA-store epilogue
  CUtensorMap tmD, tmD2 = tmA;
  const GemmParams& g = fp.g;
  if (EPI == EPI_STORE) {
    const long long rows = (g.sched == SCHED_GROUPED_K || g.sched == SCHED_DENSE) ? g.M : a_rows;
    const long long groups = (g.sched == SCHED_GROUPED_K) ? g.num_groups : 1;
    rc = make_map(&tmD, g.D, g.N, rows, groups, g.ldd, g.sched == SCHED_GROUPED_K ? g.d_group_stride : rows * g.ldd, 64, 32);
  } else {
    if (EPI == EPI_SWIGLU) {
      rc = make_map(&tmD, g.D, g.I, a_rows, 2, 2LL * g.I, g.I, 64, 32);          // gate and up halves of gate_up
      if (rc == 0) rc = make_map(&tmD2, g.aux, g.I, a_rows, 1, g.I, a_rows * g.I, 64, 32);
    } else {   // GLU backward: boxes {32 columns, 32 rows}, 64-byte swizzle, for the in-place epilogue
      rc = make_map(&tmD, g.D, g.I, a_rows, 2, 2LL * g.I, g.I, 32, 32, 2, 64);   // grad_gate_up halves
      if (rc == 0) rc = make_map(&tmD2, g.aux, g.I, a_rows, 2, 2LL * g.I, g.I, 32, 32, 2, 64);   // saved gate_up
    }
  }
  if (rc) return rc;
  return launch_fp8_pair<EPI>(tmA, tmB, tmSFA, tmSFB, tmD, tmD2, fp, max_tiles_1cta > 0 ? (max_tiles_1cta + 3) / 4 : 0,
                              stream);
}

}  // namespace b200moe

using namespace b200moe;

#define CHECK_K128(v) \
  B200_CHECK_ARG((v) > 0 && (v) % 128 == 0, B200MOE_E_BAD_SHAPE, #v " = %lld must be a positive multiple of 128", (long long)(v))

extern "C" {

int b200moe_mxfp8_gemm_nt(const void* Aq, const void* Asf, const void* Bq, const void* Bsf, void* D, int64_t M,
                          int64_t N, int64_t K, int32_t* status, b200moe_stream_t stream) {
  B200_CHECK_ARG(Aq && Asf && Bq && Bsf && D, B200MOE_E_NULL, "mxfp8_gemm_nt: null pointer");
  CHECK_K128(K); CHECK_DIM8(N); CHECK_I32(M); CHECK_I32(N); CHECK_I32(K);
  if (M == 0) return 0;
  Fp8Params fp{};
  fp.g.sched = SCHED_DENSE; fp.g.M = (int)M; fp.g.N = (int)N; fp.g.K = (int)K; fp.g.num_groups = 1;
  fp.g.D = D; fp.g.ldd = N; fp.g.status = status;
  fp.sfa = (const uint8_t*)Asf; fp.sfb = (const uint8_t*)Bsf; fp.sfa_kc = fp.sfb_kc = (int)(K / 128);
  return launch_any<EPI_STORE>(Aq, M, Bq, N, 1, K, fp, (int)(ceil_div(M, BM) * ceil_div(N, FBN)), (cudaStream_t)stream);
}

/* grouped-M: D(rows of e, N) = A(rows of e) * B[e]^T; B is an (E*N, K) stack, N %% 128 == 0.
 * epilogue: 0 store, 1 SwiGLU (B rows 64-interleaved gate|up, N = 2I, D = gate_up, aux = inter),
 * 2 GLU backward (N = I, aux = saved gate_up, D = grad_gate_up). */
int b200moe_mxfp8_expert_gemm(int epilogue, const void* Aq, const void* Asf, const void* Bq, const void* Bsf,
                              const int32_t* tile_expert, const int32_t* poffs, int64_t rows_cap, int E, int64_t N,
                              int64_t K, int64_t I, void* D, void* aux, void* q_out, void* q_sf, int32_t* status,
                              b200moe_stream_t stream) {
  B200_CHECK_ARG(Aq && Asf && Bq && Bsf && D && tile_expert && poffs, B200MOE_E_NULL, "mxfp8_expert_gemm: null pointer");
  B200_CHECK_ARG((q_out == nullptr) == (q_sf == nullptr), B200MOE_E_NULL, "mxfp8_expert_gemm: q_out and q_sf go together");
  B200_CHECK_ARG(q_out == nullptr || (epilogue != EPI_STORE && I % 128 == 0 && aligned16(q_out)), B200MOE_E_BAD_SHAPE,
                 "mxfp8_expert_gemm: quantised output needs the SwiGLU / GLU-backward epilogue and I %% 128 == 0");
  CHECK_K128(K); CHECK_K128(N); CHECK_I32(rows_cap);
  B200_CHECK_ARG(rows_cap % B200MOE_TILE_M == 0, B200MOE_E_BAD_SHAPE, "mxfp8_expert_gemm: rows_cap %% %d != 0", B200MOE_TILE_M);
  B200_CHECK_ARG(E >= 1 && E * N < (1LL << 31), B200MOE_E_BAD_SHAPE, "mxfp8_expert_gemm: E = %d", E);
  Fp8Params fp{};
  fp.g.sched = SCHED_GROUPED_M; fp.g.N = (int)N; fp.g.K = (int)K; fp.g.num_groups = E;
  fp.g.tile_expert = tile_expert; fp.g.poffs = poffs; fp.g.D = D; fp.g.ldd = N; fp.g.aux = aux; fp.g.I = (int)I;
  fp.g.status = status;
  fp.sfa = (const uint8_t*)Asf; fp.sfb = (const uint8_t*)Bsf; fp.sfa_kc = fp.sfb_kc = (int)(K / 128);
  fp.b_rows_per_group = (int)N;
  fp.q_out = (uint8_t*)q_out; fp.q_sf = (uint8_t*)q_sf;
  switch (epilogue) {
    case EPI_STORE: return launch_any<EPI_STORE>(Aq, rows_cap, Bq, N, E, K, fp, 0, (cudaStream_t)stream);
    case EPI_SWIGLU:
      B200_CHECK_ARG(aux && N == 2 * I && I % 64 == 0, B200MOE_E_BAD_SHAPE, "mxfp8_expert_gemm: SwiGLU needs N = 2I, I %% 64 == 0");
      return launch_any<EPI_SWIGLU>(Aq, rows_cap, Bq, N, E, K, fp, 0, (cudaStream_t)stream);
    case EPI_GLU_BWD:
      B200_CHECK_ARG(aux && N == I, B200MOE_E_BAD_SHAPE, "mxfp8_expert_gemm: GLU backward needs N = I");
      return launch_any<EPI_GLU_BWD>(Aq, rows_cap, Bq, N, E, K, fp, 0, (cudaStream_t)stream);
    default:
      set_error("mxfp8_expert_gemm: unknown epilogue %d", epilogue);
      return B200MOE_E_UNSUPPORTED;
  }
}

/* grouped-K (wgrad): out[e] (Na,Nb) = At[:, rows of e] * Bt[:, rows of e]^T with At (Na, rows_cap) and
 * Bt (Nb, rows_cap) the transposed-quantised operands (K = padded token rows). */
int b200moe_mxfp8_expert_wgrad(const void* Atq, const void* Atsf, const void* Btq, const void* Btsf,
                               const int32_t* poffs, const int32_t* counts, int64_t rows_cap, int E, int64_t Na,
                               int64_t Nb, void* out, int32_t* status, b200moe_stream_t stream) {
  B200_CHECK_ARG(Atq && Atsf && Btq && Btsf && poffs && out, B200MOE_E_NULL, "mxfp8_expert_wgrad: null pointer");
  CHECK_K128(rows_cap); CHECK_DIM8(Na); CHECK_DIM8(Nb); CHECK_I32(Na); CHECK_I32(Nb); CHECK_I32(rows_cap);
  Fp8Params fp{};
  fp.g.sched = SCHED_GROUPED_K; fp.g.M = (int)Na; fp.g.N = (int)Nb; fp.g.K = (int)rows_cap; fp.g.num_groups = E;
  fp.g.poffs = poffs; fp.g.counts = counts; fp.g.D = out; fp.g.ldd = Nb; fp.g.d_group_stride = Na * Nb;
  fp.g.status = status;
  fp.sfa = (const uint8_t*)Atsf; fp.sfb = (const uint8_t*)Btsf; fp.sfa_kc = fp.sfb_kc = (int)(rows_cap / 128);
  return launch_any<EPI_STORE>(Atq, Na, Btq, Nb, 1, rows_cap, fp,
                               (int)std::min<long long>(1 << 30, E * ceil_div(Na, BM) * ceil_div(Nb, FBN)),
                               (cudaStream_t)stream);
}

}  // extern "C"
