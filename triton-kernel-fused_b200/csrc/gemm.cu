// Persistent bf16 GEMM for sm_100a: TMA -> 128B-swizzled shared-memory ring -> tcgen05.mma with the
// fp32 accumulator in TMEM (double buffered) -> epilogue warps read TMEM and store.
//
// One kernel serves every contraction of the MoE block:
//   schedule  DENSE      D(M,N)            = A * B          (router projections)
//             GROUPED_M  D(rows of e, N)   = A(rows of e) * B[e]   (expert forward + dgrad)
//             GROUPED_K  D[e](M,N)         = A(rows of e)^T * B(rows of e)   (expert wgrad, split-K)
//   operand majors: K-major (reduction index contiguous) or MN-major (row/column index contiguous)
//   epilogues: bf16 store, SwiGLU (gate|up -> gate_up + inter), GLU backward, fp32 store.
//   CTAS = 1: one CTA computes a 128 x BN tile.
//   CTAS = 2: a CTA pair (cluster of 2) computes a 256 x 256 tile with tcgen05 cta_group::2: each CTA
//             stages its own 128 rows of A and its own 128 columns of B, the leader CTA issues the
//             MMAs for both, each CTA's TMEM holds its 128 rows of the accumulator.  This halves
//             the L2 -> shared-memory traffic per FLOP and leaves room for 6 stages instead of 4.
//
// Warp roles (320 threads): warp 0 = TMA producer (one lane), warp 1 = TMEM owner + MMA issuer (one
// lane), warps 2-9 = epilogue (TMEM lane quarter = warp_id % 4, two warps per quarter split the
// columns).
#include <cuda.h>
#include <stdlib.h>

#include <mutex>
#include <type_traits>

#include "gemm_common.cuh"

namespace b200moe {

constexpr int BK = 64;   // k-block: 64 bf16 = one 128-byte swizzle row

// BN = 256 kernels with a bf16 result stage it in shared memory and write it with TMA stores
template <int BN, int EPI>
__host__ __device__ constexpr bool tma_epilogue() { return BN == 256 && EPI != EPI_STORE_F32; }

// EPI_WARP_BYTES: shared memory each epilogue warp owns (0: none, 4 KB: one output staging box,
// 8 KB: the GLU-backward gate and up boxes that are loaded by TMA and overwritten in place)
constexpr int kGluBoxBytes = 32 * 64;   // GLU backward: one 32 rows x 32 columns bf16 box

template <int BN, int EPI>
__host__ __device__ constexpr int epi_warp_bytes() {
  return !tma_epilogue<BN, EPI>() ? 0 : (EPI == EPI_GLU_BWD ? 2 * kStageOutBytes : kStageOutBytes);
}

template <int BN, int CTAS, int EPI_WARP_BYTES = 0>
struct Cfg {
  static constexpr int A_BYTES = BM * BK * 2;
  static constexpr int B_BYTES = (BN / CTAS) * BK * 2;   // per CTA
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int EPI_BYTES = kEpiWarps * EPI_WARP_BYTES;
  static constexpr int kBudget = 232448 - 1024 - 256;       // 227 KB minus alignment slack and barriers
  static constexpr int kFit = (kBudget - EPI_BYTES) / STAGE_BYTES;
  static constexpr int NSTAGE = kFit > 8 ? 8 : kFit;
  static constexpr int TMEM_COLS = 2 * BN;  // two accumulators; 128, 256 or 512 (power of two >= 32)
  static constexpr int BAR_BYTES = (2 * NSTAGE + 4 + 2 * kEpiWarps) * 8 + 16;
  static constexpr int SMEM_BYTES = NSTAGE * STAGE_BYTES + EPI_BYTES + BAR_BYTES + 1024;  // + alignment slack
  static constexpr int TILE_ROWS = BM * CTAS;
};


// POLY: the variant of the kernel.  GLU epilogues: per-expert activation codes 0 / 1 / 5 (p.act_codes); false =
// SiLU for every expert.  Store epilogues (EPI_STORE, EPI_STORE_F32): a convolution operand (p.conv_taps), compiled
// only into the instantiations the conv-router entry points launch, so that the expert GEMMs carry no code for it.
template <int BN, int EPI, int CTAS, bool POLY = false>
__global__ void __launch_bounds__(kThreads, 1)
gemm_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
            const __grid_constant__ CUtensorMap tmD, const __grid_constant__ CUtensorMap tmD2,
            const GemmParams p) {
  constexpr bool TMA_EPI = tma_epilogue<BN, EPI>();
  using C = Cfg<BN, CTAS, epi_warp_bytes<BN, EPI>()>;
  constexpr int TN = (EPI == EPI_SWIGLU) ? BN / 2 : BN;   // output columns one tile covers
  constexpr int TM = C::TILE_ROWS;
  constexpr int NSTAGE = C::NSTAGE;
  constexpr int BNC = BN / CTAS;                          // B columns staged by one CTA

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint8_t* epi_smem = smem + NSTAGE * C::STAGE_BYTES;   // 1024-aligned: stages are multiples of 8 KB
  uint64_t* bars = reinterpret_cast<uint64_t*>(epi_smem + C::EPI_BYTES);
  const uint32_t bar_full = smem_u32(bars);
  const uint32_t bar_empty = smem_u32(bars + NSTAGE);
  const uint32_t bar_tfull = smem_u32(bars + 2 * NSTAGE);
  const uint32_t bar_tempty = smem_u32(bars + 2 * NSTAGE + 2);
  const uint32_t bar_epi = smem_u32(bars + 2 * NSTAGE + 4);   // two per epilogue warp (GLU backward load sets)
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * NSTAGE + 4 + 2 * kEpiWarps);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t cta_rank = (CTAS == 2) ? cluster_ctarank() : 0u;   // 0 = leader of the pair
  const int first_tile = (CTAS == 2) ? static_cast<int>(cluster_id_x()) : static_cast<int>(blockIdx.x);
  const int tile_step = (CTAS == 2) ? static_cast<int>(num_clusters_x()) : static_cast<int>(gridDim.x);

  if (threadIdx.x == 0) {
    for (int s = 0; s < NSTAGE; ++s) {
      mbar_init(bar_full + 8 * s, 1);
      mbar_init(bar_empty + 8 * s, 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(bar_tfull + 8 * b, 1);
      mbar_init(bar_tempty + 8 * b, kEpiWarps * CTAS);
    }
    for (int w = 0; w < 2 * kEpiWarps; ++w) mbar_init(bar_epi + 8 * w, 1);
    *abort_flag = 0;
    fence_mbar_init();
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmB);
  }
  if (warp == 1) {
    if constexpr (CTAS == 2) {
      tmem_alloc_pair(smem_u32(tmem_slot), C::TMEM_COLS);
      tmem_relinquish_pair();
    } else {
      tmem_alloc(smem_u32(tmem_slot), C::TMEM_COLS);
      tmem_relinquish();
    }
  }
  __shared__ int s_order[B200MOE_MAX_EXPERTS];
  const int* order = build_group_order(p, s_order);
  tc_fence_before();
  __syncthreads();
  if constexpr (CTAS == 2) {   // peer barriers are initialised before any remote arrive
    __syncwarp();
    cluster_sync_all();
  }
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  constexpr bool WINDOW = (EPI == EPI_SWIGLU || EPI == EPI_GLU_BWD);   // entry points with a row window
  constexpr bool CONV = POLY && (EPI == EPI_STORE || EPI == EPI_STORE_F32);   // launched by the conv-router entry points
  const int total = total_tiles(p, TN, TM, WINDOW);
  const int row_base = (WINDOW && p.row_hi > 0) ? p.row_lo : 0;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer (each CTA)
    if constexpr (CTAS == 2 && !CONV) {
      // Pair tiles: the up to four boxes of a stage (one or two of A, one or two of B) are issued by four lanes in
      // ONE instruction, each lane with its own tensor map, destination and coordinates, instead of by one lane
      // in up to four instructions.  The producer's time between "stage free" and "loads issued" is what an empty
      // ring waits for: with both operands MN-major (the weight-gradient GEMMs, four boxes per stage) the
      // one-lane producer could not keep up with the MMAs, and this form made those launches 12-13 % faster.
      if (lane < 4) {
        const bool isA = lane < 2;
        const int j = lane & 1;
        const bool mn = isA ? (p.a_mn != 0) : (EPI != EPI_SWIGLU && p.b_mn != 0);
        const int nbox = !mn ? 1 : (isA ? BM / 64 : BNC / 64);
        const bool active = j < nbox;
        const CUtensorMap* tm = isA ? &tmA : &tmB;
        const uint32_t dst_off = (isA ? 0u : static_cast<uint32_t>(C::A_BYTES)) + static_cast<uint32_t>(j) * (64 * BK * 2);
        const uint32_t full0 = mapa_shared(bar_full, 0);
        const bool expects = (lane == 0 && cta_rank == 0);
        int s = 0;
        uint32_t ph = 0;
        bool ok = true;
        for (int tile = first_tile; tile < total && ok; tile += tile_step) {
          const Tile t = get_tile(p, tile, TN, TM, 64, order, row_base);
          const int gB = (p.sched == SCHED_GROUPED_M) ? t.g : 0;
          const int m0 = t.m0 + BM * static_cast<int>(cta_rank);
          const int bstep = (EPI != EPI_SWIGLU && p.N - t.n0 <= BN / 2) ? BNC / 2 : BNC;
          // this lane's box: the coordinate that does not move with k, and the group
          int fixed, grp;
          if (isA) {
            fixed = m0 + (mn ? 64 * j : 0);
            grp = 0;
          } else if constexpr (EPI == EPI_SWIGLU) {
            fixed = t.n0;
            grp = 2 * gB + static_cast<int>(cta_rank);
          } else {
            fixed = t.n0 + bstep * static_cast<int>(cta_rank) + (mn ? 64 * j : 0);
            grp = gB;
          }
          int kk = t.k0;
          for (int kb = 0; kb < t.nkb; ++kb, kk += BK) {
            if (!mbar_wait(bar_empty + 8 * s, ph ^ 1, abort_flag, ST_WAIT_PRODUCER)) {
              ok = false;
              break;
            }
            if (expects) mbar_arrive_expect_tx(bar_full + 8 * s, 2 * C::STAGE_BYTES);
            if (active)
              tma_load_3d_pair(smem_u32(smem + s * C::STAGE_BYTES) + dst_off, tm, full0 + 8 * s, mn ? fixed : kk,
                               mn ? kk : fixed, grp);
            if (++s == NSTAGE) {
              s = 0;
              ph ^= 1;
            }
          }
        }
      }
    } else if (lane == 0) {
      int s = 0;
      uint32_t ph = 0;
      bool ok = true;
      for (int tile = first_tile; tile < total && ok; tile += tile_step) {
        const Tile t = get_tile(p, tile, TN, TM, 64, order, row_base);
        const int gB = (p.sched == SCHED_GROUPED_M) ? t.g : 0;
        const int m0 = t.m0 + BM * static_cast<int>(cta_rank);
        // a last pair tile with at most BN/2 live columns runs as a 256 x BN/2 MMA: each CTA then
        // supplies BN/4 columns of B, the first ones of its (still BN/2 wide) staging tile
        const int bstep = (CTAS == 2 && EPI != EPI_SWIGLU && p.N - t.n0 <= BN / 2) ? BNC / 2 : BNC;
        for (int kb = 0; kb < t.nkb; ++kb) {
          if (!mbar_wait(bar_empty + 8 * s, ph ^ 1, abort_flag, ST_WAIT_PRODUCER)) {
            ok = false;
            break;
          }
          const uint32_t sa = smem_u32(smem + s * C::STAGE_BYTES);
          const uint32_t sb = sa + C::A_BYTES;
          const int kk = t.k0 + kb * BK;
          // coordinates of the B boxes (MN-major case) and of the A box (K-major case); a convolution operand
          // (see GemmParams::conv_taps) replaces the flat row by (position + shift, batch)
          int a_c0 = kk, a_c1 = m0, a_c2 = 0, b_n0 = t.n0, b_k = kk, b_g = gB;
          if (CONV && p.conv_taps > 0) {
            if (p.sched == SCHED_DENSE) {
              const int per_tap = p.conv_C / BK, tap = kb / per_tap;
              a_c2 = m0 / p.conv_S;
              a_c1 = m0 - a_c2 * p.conv_S + p.conv_sign * (tap - (p.conv_taps - 1));
              a_c0 = (kb - tap * per_tap) * BK;
            } else {
              const int tap = t.n0 / p.conv_C;
              b_n0 = t.n0 - tap * p.conv_C;
              b_g = kk / p.conv_S;
              b_k = kk - b_g * p.conv_S + tap - (p.conv_taps - 1);
            }
          }
          if constexpr (CTAS == 1) {
            const uint32_t full = bar_full + 8 * s;
            mbar_arrive_expect_tx(full, C::STAGE_BYTES);
            if (!p.a_mn) {
              tma_load_3d(sa, &tmA, full, a_c0, a_c1, a_c2);  // box {64 k, 128 rows}
            } else {
#pragma unroll
              for (int j = 0; j < BM / 64; ++j)  // boxes {64 mn, 64 k-rows}
                tma_load_3d(sa + j * (64 * BK * 2), &tmA, full, m0 + 64 * j, kk, 0);
            }
            if constexpr (EPI == EPI_SWIGLU) {
              // gate rows [n0, n0+BN/2) of W[e] then up rows of the same range: dims {H, I, 2E}
              tma_load_3d(sb, &tmB, full, kk, t.n0, 2 * gB);
              tma_load_3d(sb + (BN / 2) * BK * 2, &tmB, full, kk, t.n0, 2 * gB + 1);
            } else if (!p.b_mn) {
              tma_load_3d(sb, &tmB, full, kk, t.n0, gB);  // box {64 k, BN rows}
            } else {
#pragma unroll
              for (int j = 0; j < BN / 64; ++j)
                tma_load_3d(sb + j * (64 * BK * 2), &tmB, full, b_n0 + 64 * j, b_k, b_g);
            }
          } else {
            // the leader's barrier counts the bytes of both CTAs
            const uint32_t full = mapa_shared(bar_full + 8 * s, 0);
            if (cta_rank == 0) mbar_arrive_expect_tx(bar_full + 8 * s, 2 * C::STAGE_BYTES);
            if (!p.a_mn) {
              tma_load_3d_pair(sa, &tmA, full, a_c0, a_c1, a_c2);
            } else {
#pragma unroll
              for (int j = 0; j < BM / 64; ++j)
                tma_load_3d_pair(sa + j * (64 * BK * 2), &tmA, full, m0 + 64 * j, kk, 0);
            }
            if constexpr (EPI == EPI_SWIGLU) {
              // leader stages the gate rows, the peer the up rows of I-columns [n0, n0+128)
              tma_load_3d_pair(sb, &tmB, full, kk, t.n0, 2 * gB + static_cast<int>(cta_rank));
            } else if (!p.b_mn) {
              tma_load_3d_pair(sb, &tmB, full, kk, t.n0 + bstep * static_cast<int>(cta_rank), gB);
            } else {
#pragma unroll
              for (int j = 0; j < BNC / 64; ++j)
                tma_load_3d_pair(sb + j * (64 * BK * 2), &tmB, full,
                                 b_n0 + bstep * static_cast<int>(cta_rank) + 64 * j, b_k, b_g);
            }
          }
          if (++s == NSTAGE) {
            s = 0;
            ph ^= 1;
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer (leader CTA only)
    if (lane == 0 && cta_rank == 0) {
      const uint32_t idesc_full = umma_idesc_bf16(BN, p.a_mn, p.b_mn, TM);
      const uint32_t idesc_half = umma_idesc_bf16(BN / 2, p.a_mn, p.b_mn, TM);   // narrow last pair tile
      // K-major: rows are 128 B apart, 8-row groups 1024 B apart, 16 k-elements = 32 B.
      // MN-major: 64-wide MN blocks are 64*128 B apart (LBO), 8 k-rows 1024 B apart (SBO),
      //           16 k-rows = 2048 B.
      const uint32_t a_lbo = p.a_mn ? 64 * BK * 2 : 0, b_lbo = p.b_mn ? 64 * BK * 2 : 0;
      const uint32_t a_kstep = p.a_mn ? 2048 : 32, b_kstep = p.b_mn ? 2048 : 32;
      int s = 0, it = 0;
      uint32_t ph = 0;
      bool ok = true;
      for (int tile = first_tile; tile < total && ok; tile += tile_step, ++it) {
        const Tile t = get_tile(p, tile, TN, TM, 64, order, row_base);
        const int buf = it & 1;
        if (!mbar_wait(bar_tempty + 8 * buf, ((it >> 1) & 1) ^ 1, abort_flag, ST_WAIT_MMA_TMEM)) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + buf * BN;
        const uint32_t idesc =
            (CTAS == 2 && EPI != EPI_SWIGLU && p.N - t.n0 <= BN / 2) ? idesc_half : idesc_full;
        for (int kb = 0; kb < t.nkb; ++kb) {
          if (!mbar_wait(bar_full + 8 * s, ph, abort_flag, ST_WAIT_MMA_FULL)) {
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t sa = smem_u32(smem + s * C::STAGE_BYTES);
          const uint32_t sb = sa + C::A_BYTES;
#pragma unroll
          for (int k = 0; k < BK / 16; ++k) {
            const uint64_t da = umma_desc_sw128(sa + k * a_kstep, a_lbo, 1024);
            const uint64_t db = umma_desc_sw128(sb + k * b_kstep, b_lbo, 1024);
            if constexpr (CTAS == 2) umma_bf16_pair(d_tmem, da, db, idesc, (kb | k) != 0);
            else umma_bf16(d_tmem, da, db, idesc, (kb | k) != 0);
          }
          // frees the stage (in both CTAs) when these MMAs have read it
          if constexpr (CTAS == 2) umma_commit_pair(bar_empty + 8 * s);
          else umma_commit(bar_empty + 8 * s);
          if (++s == NSTAGE) {
            s = 0;
            ph ^= 1;
          }
        }
        if (!ok) break;
        if (t.nkb > 0) {
          if constexpr (CTAS == 2) umma_commit_pair(bar_tfull + 8 * buf);
          else umma_commit(bar_tfull + 8 * buf);
        } else {
          mbar_arrive(bar_tfull + 8 * buf);
          if constexpr (CTAS == 2) mbar_arrive_cluster(mapa_shared(bar_tfull + 8 * buf, 1));
        }
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue (8 warps per CTA)
    const int q = warp & 3;              // TMEM lane quarter this warp may read
    const int half = (warp - 2) >> 2;    // which half of the tile's columns this warp handles
    const uint32_t tempty_leader = (CTAS == 2) ? mapa_shared(bar_tempty, 0) : bar_tempty;
    uint32_t epi_phase = 0;   // parity of this warp's GLU-backward load barrier
    int it = 0;
    for (int tile = first_tile; tile < total; tile += tile_step, ++it) {
      const Tile t = get_tile(p, tile, TN, TM, 64, order, row_base);
      const int buf = it & 1;
      int act_code = 0;   // activation of this tile's expert (uniform over the tile)
      if constexpr (POLY && (EPI == EPI_SWIGLU || EPI == EPI_GLU_BWD)) act_code = p.act_codes[t.g];
      const int row0 = t.m0 + BM * static_cast<int>(cta_rank) + q * 32;   // first row of this warp
      const long long row = static_cast<long long>(row0) + lane;
      // GLU backward works on four 32-column sub-chunks per warp with two sets of (gate, up) boxes of
      // 32 rows x 32 columns (2 KB, 64-byte swizzle): a set is loaded by TMA, overwritten in place with
      // grad_gate / grad_up and stored by TMA while the other set is loading or being computed on.  The saved
      // gate/up values do not depend on the accumulator, so the first two loads go out before the MMAs of
      // the tile are waited for.
      const int glu_col0 = t.n0 + half * (BN / 2);
      uint8_t* ebuf = epi_smem + (warp - 2) * C::EPI_BYTES / kEpiWarps;   // [set][gate | up] boxes of 2 KB
      const uint32_t ebar = bar_epi + 16 * (warp - 2);                     // + 8 * set
      auto glu_load = [&](int sub) {   // tmD2 = saved gate_up seen as {I, rows, 2}, box {32, 32}
        const int set = sub & 1;
        if (lane == 0) {
          mbar_arrive_expect_tx(ebar + 8 * set, 2 * kGluBoxBytes);
          tma_load_3d(smem_u32(ebuf + set * 2 * kGluBoxBytes), &tmD2, ebar + 8 * set, glu_col0 + 32 * sub, row0, 0);
          tma_load_3d(smem_u32(ebuf + set * 2 * kGluBoxBytes + kGluBoxBytes), &tmD2, ebar + 8 * set,
                      glu_col0 + 32 * sub, row0, 1);
        }
      };
      uint8_t* bufG = ebuf;   // staging box of the other TMA-store epilogues
      if constexpr (TMA_EPI && EPI == EPI_GLU_BWD) {
        staging_free(lane);   // the previous tile's stores out of these boxes have been read
        if (glu_col0 < p.I) glu_load(0);
        if (glu_col0 + 32 < p.I) glu_load(1);
      }
      if (!mbar_wait(bar_tfull + 8 * buf, (it >> 1) & 1, abort_flag, ST_WAIT_EPILOGUE)) break;
      __syncwarp();
      tc_fence_after();
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + buf * BN;
      const bool have_acc = t.nkb > 0;

      if constexpr (TMA_EPI) {
        // results are packed to bf16, staged per warp as 32 rows x 64 columns and written by TMA
        // stores (which clip at the tensor's bounds, so no row or column masks are needed)
        uint8_t* sbuf = bufG;   // this warp's staging box
        const int grp = (p.sched == SCHED_GROUPED_K) ? t.g : 0;
        if constexpr (EPI == EPI_STORE || EPI == EPI_AXPBY || EPI == EPI_STORE_SYM) {
          constexpr int W = BN / 2;
          // push mode: this lane's output row goes to a slot of another GPU's (or this GPU's) receive buffer
          uint8_t* push_dst = nullptr;
          if (p.push_rank != nullptr) {
            const int rk = p.push_rank[row];
            if (rk >= 0)
              push_dst = reinterpret_cast<uint8_t*>(p.push_base[rk]) + static_cast<long long>(p.push_slot[row]) * p.N * 2;
          }
          const int ax_drow = (EPI == EPI_AXPBY) ? static_cast<int>(row) - p.poffs[t.g] : 0;   // row inside its group
#pragma unroll 1
          for (int c = half * W; c < (half + 1) * W; c += 64) {
            if (t.n0 + c >= p.N) break;
            uint32_t pk[32];
#pragma unroll
            for (int sub = 0; sub < 2; ++sub) {
              uint32_t r[32];
              if (have_acc) {
                tmem_ld32(taddr + c + 32 * sub, r);
                tmem_ld_wait();
              } else {
#pragma unroll
                for (int i = 0; i < 32; ++i) r[i] = 0u;
              }
              if constexpr (EPI == EPI_AXPBY) {
                // r = alpha * acc + beta * C[row, columns] (+ diag on the group's own diagonal); the lane reads the
                // 64 bytes of its row of C that lie under this sub-chunk
                const int col0 = t.n0 + c + 32 * sub;
                const uint4* src = reinterpret_cast<const uint4*>(reinterpret_cast<const __nv_bfloat16*>(p.aux) +
                                                                  row * p.N + col0);
#pragma unroll
                for (int v = 0; v < 4; ++v) {
                  const uint4 cv = src[v];
                  const uint32_t cw[4] = {cv.x, cv.y, cv.z, cv.w};
#pragma unroll
                  for (int h = 0; h < 4; ++h) {
                    const float2 cf = unpack_bf16x2(cw[h]);
                    const int i = 8 * v + 2 * h;
                    float v0 = p.ax_alpha * __uint_as_float(r[i]) + p.ax_beta * cf.x;
                    float v1 = p.ax_alpha * __uint_as_float(r[i + 1]) + p.ax_beta * cf.y;
                    if (col0 + i == ax_drow) v0 += p.ax_diag;
                    if (col0 + i + 1 == ax_drow) v1 += p.ax_diag;
                    r[i] = __float_as_uint(v0);
                    r[i + 1] = __float_as_uint(v1);
                  }
                }
              }
#pragma unroll
              for (int i = 0; i < 16; ++i)
                pk[16 * sub + i] = pack_bf16x2(__uint_as_float(r[2 * i]), __uint_as_float(r[2 * i + 1]));
            }
            if (p.push_rank != nullptr) {
              // each lane stages its own 128-byte row piece (unswizzled) and sends it with one bulk copy
              bulk_wait_read_all();   // this lane's previous copy has read the piece
              uint8_t* mine = sbuf + lane * 128;
#pragma unroll
              for (int j = 0; j < 8; ++j)
                *reinterpret_cast<uint4*>(mine + 16 * j) = make_uint4(pk[4 * j], pk[4 * j + 1], pk[4 * j + 2], pk[4 * j + 3]);
              fence_proxy_async_smem();
              if (push_dst != nullptr) {
                const int left = (p.N - (t.n0 + c)) * 2;
                bulk_store_1d(push_dst + static_cast<long long>(t.n0 + c) * 2, smem_u32(mine), left < 128 ? left : 128);
              }
              bulk_commit_group();
            } else {
              staging_free(lane);
              stage_row(sbuf, lane, pk);
              store_box(&tmD, sbuf, lane, t.n0 + c, row0, grp);
              if constexpr (EPI == EPI_AXPBY || EPI == EPI_STORE_SYM) if (p.sym_mirror) {
                // symmetric result: the chunk (32 rows x 64 columns) of a tile right of the diagonal tile is also
                // the transpose of a chunk nobody computes.  Stage it as 64 rows x 32 columns (unswizzled rows of
                // 64 bytes; lane l owns column l) and store it through the second map.
                const int lrow0 = row0 - t.g * p.sym_rows;          // this warp's first row inside its group
                if ((t.n0 + c) / B200MOE_TILE_M > lrow0 / B200MOE_TILE_M) {
                  staging_free(lane);                               // the store above has read the box
#pragma unroll
                  for (int m = 0; m < 32; ++m) {
                    *reinterpret_cast<uint16_t*>(sbuf + (2 * m) * 64 + lane * 2) = static_cast<uint16_t>(pk[m] & 0xffffu);
                    *reinterpret_cast<uint16_t*>(sbuf + (2 * m + 1) * 64 + lane * 2) = static_cast<uint16_t>(pk[m] >> 16);
                  }
                  store_box(&tmD2, sbuf, lane, lrow0, t.g * p.sym_rows + t.n0 + c, 0);
                }
              }
            }
          }
        } else if constexpr (EPI == EPI_SWIGLU) {
          // accumulator columns [0,BN/2) = gate, [BN/2,BN) = up for I-columns [n0, n0+BN/2)
          const int c = half * (BN / 4);
          if (t.n0 + c < p.I) {
            uint32_t og[32], ou[32], oh[32];
#pragma unroll
            for (int sub = 0; sub < 2; ++sub) {
              uint32_t g[32], u[32];
              tmem_ld32(taddr + c + 32 * sub, g);
              tmem_ld32(taddr + BN / 2 + c + 32 * sub, u);
              tmem_ld_wait();
#pragma unroll
              for (int i = 0; i < 16; ++i) {
                og[16 * sub + i] = pack_bf16x2(__uint_as_float(g[2 * i]), __uint_as_float(g[2 * i + 1]));
                ou[16 * sub + i] = pack_bf16x2(__uint_as_float(u[2 * i]), __uint_as_float(u[2 * i + 1]));
              }
              glu_fwd_pairs_by_code<POLY>(act_code, og + 16 * sub, ou + 16 * sub, oh + 16 * sub, 16);
            }
            staging_free(lane);
            stage_row(sbuf, lane, og);
            store_box(&tmD, sbuf, lane, t.n0 + c, row0, 0);    // gate half of gate_up
            staging_free(lane);
            stage_row(sbuf, lane, ou);
            store_box(&tmD, sbuf, lane, t.n0 + c, row0, 1);    // up half
            staging_free(lane);
            stage_row(sbuf, lane, oh);
            store_box(&tmD2, sbuf, lane, t.n0 + c, row0, 0);   // inter
          }
        } else {  // EPI_GLU_BWD: accumulator = grad_inter columns [n0, n0+BN); this warp: 128 of them
          constexpr int W = BN / 2;
#pragma unroll 1
          for (int sub = 0; sub < W / 32; ++sub) {
            const int col = glu_col0 + 32 * sub;
            if (col >= p.I) break;                       // warp-uniform
            const int set = sub & 1;
            uint8_t* bG = ebuf + set * 2 * kGluBoxBytes;
            uint8_t* bU = bG + kGluBoxBytes;
            uint32_t r[32];
            tmem_ld32(taddr + half * W + 32 * sub, r);
            if (!mbar_wait(ebar + 8 * set, (epi_phase >> set) & 1u, abort_flag, ST_WAIT_EPILOGUE)) break;
            epi_phase ^= 1u << set;
            uint4 g4[4], u4[4];
#pragma unroll
            for (int v = 0; v < 4; ++v) {              // this lane's row: 64 bytes, 64-byte swizzle
              const int off = lane * 64 + ((v ^ ((lane >> 1) & 3)) << 4);
              g4[v] = *reinterpret_cast<const uint4*>(bG + off);
              u4[v] = *reinterpret_cast<const uint4*>(bU + off);
            }
            tmem_ld_wait();
            uint32_t og[16], ou[16];
            glu_bwd32<POLY>(r, g4, u4, og, ou, act_code);
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
            // as soon as that store has read its boxes (a few hundred ns), they are reloaded with the sub-chunk
            // after the next one, which then has a whole sub-chunk of arithmetic to arrive
            if (sub + 2 < W / 32 && glu_col0 + 32 * (sub + 2) < p.I) {
              staging_free(lane);
              glu_load(sub + 2);
            }
          }
        }
      } else if constexpr (EPI == EPI_STORE || EPI == EPI_STORE_F32) {
        const bool row_ok = (p.sched == SCHED_GROUPED_M) || (row < p.M);
        const long long base = (p.sched == SCHED_GROUPED_K ? t.g * p.d_group_stride : 0) +
                               row * p.ldd + t.n0;
        constexpr int W = BN / 2;   // columns per warp
#pragma unroll 1
        for (int c0 = half * W; c0 < (half + 1) * W; c0 += 32) {
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
            if constexpr (EPI == EPI_STORE) {
              __nv_bfloat16* d = reinterpret_cast<__nv_bfloat16*>(p.D) + base + c0;
#pragma unroll
              for (int v = 0; v < 4; ++v)
                if (t.n0 + c0 + v * 8 < p.N) *reinterpret_cast<uint4*>(d + v * 8) = pack8(r + v * 8);
            } else {
              float* d = reinterpret_cast<float*>(p.D) + base + c0;
#pragma unroll
              for (int v = 0; v < 8; ++v)
                if (t.n0 + c0 + v * 4 < p.N)
                  *reinterpret_cast<uint4*>(d + v * 4) = make_uint4(r[v * 4 + 0], r[v * 4 + 1], r[v * 4 + 2], r[v * 4 + 3]);
            }
          }
        }
      } else if constexpr (EPI == EPI_SWIGLU) {
        // accumulator columns [0,BN/2) = gate, [BN/2,BN) = up for I-columns [n0, n0+BN/2)
        const int I = p.I;
        __nv_bfloat16* gu = reinterpret_cast<__nv_bfloat16*>(p.D) + row * (2LL * I);
        __nv_bfloat16* it_out = reinterpret_cast<__nv_bfloat16*>(p.aux) + row * static_cast<long long>(I);
        constexpr int W = BN / 4;   // I-columns per warp
#pragma unroll 1
        for (int c0 = half * W; c0 < (half + 1) * W; c0 += 32) {
          if (t.n0 + c0 >= I) break;
          uint32_t g[32], u[32];
          tmem_ld32(taddr + c0, g);
          tmem_ld32(taddr + BN / 2 + c0, u);
          tmem_ld_wait();
#pragma unroll
          for (int v = 0; v < 4; ++v) {
            const int col = t.n0 + c0 + v * 8;
            if (col < I) {
              uint32_t og[4], ou[4], oh[4];
#pragma unroll
              for (int h = 0; h < 4; ++h) {
                og[h] = pack_bf16x2(__uint_as_float(g[v * 8 + 2 * h]), __uint_as_float(g[v * 8 + 2 * h + 1]));
                ou[h] = pack_bf16x2(__uint_as_float(u[v * 8 + 2 * h]), __uint_as_float(u[v * 8 + 2 * h + 1]));
              }
              glu_fwd_pairs_by_code<POLY>(act_code, og, ou, oh, 4);
              *reinterpret_cast<uint4*>(gu + col) = make_uint4(og[0], og[1], og[2], og[3]);
              *reinterpret_cast<uint4*>(gu + I + col) = make_uint4(ou[0], ou[1], ou[2], ou[3]);
              *reinterpret_cast<uint4*>(it_out + col) = make_uint4(oh[0], oh[1], oh[2], oh[3]);
            }
          }
        }
      } else {  // EPI_GLU_BWD: accumulator = grad_inter columns [n0, n0+BN)
        const int I = p.I;
        const __nv_bfloat16* gu = reinterpret_cast<const __nv_bfloat16*>(p.aux) + row * (2LL * I);
        __nv_bfloat16* ggu = reinterpret_cast<__nv_bfloat16*>(p.D) + row * (2LL * I);
        constexpr int W = BN / 2;
        constexpr int NCH = W / 32;
        // the saved gate/up values of chunk c+1 are fetched while chunk c is computed
        uint4 gv[2][4], uv[2][4];
        auto fetch = [&](int c, int slot) {
#pragma unroll
          for (int v = 0; v < 4; ++v) {
            const int col = t.n0 + half * W + c * 32 + v * 8;
            if (col < I) {
              gv[slot][v] = __ldg(reinterpret_cast<const uint4*>(gu + col));
              uv[slot][v] = __ldg(reinterpret_cast<const uint4*>(gu + I + col));
            } else {
              gv[slot][v] = make_uint4(0u, 0u, 0u, 0u);
              uv[slot][v] = make_uint4(0u, 0u, 0u, 0u);
            }
          }
        };
        fetch(0, 0);
#pragma unroll
        for (int c = 0; c < NCH; ++c) {
          const int c0 = half * W + c * 32;
          if (t.n0 + c0 < I) {          // warp-uniform
            uint32_t r[32];
            tmem_ld32(taddr + c0, r);
            if (c + 1 < NCH) fetch(c + 1, (c + 1) & 1);
            tmem_ld_wait();
#pragma unroll
            for (int v = 0; v < 4; ++v) {
              const int col = t.n0 + c0 + v * 8;
              if (col < I) {
                const uint4 g4 = gv[c & 1][v], u4 = uv[c & 1][v];
                const uint32_t gw[4] = {g4.x, g4.y, g4.z, g4.w};
                const uint32_t uw[4] = {u4.x, u4.y, u4.z, u4.w};
                uint32_t og[4], ou[4];
                auto bwd8 = [&](auto code_tag) {
                  constexpr int CODE = decltype(code_tag)::value;
#pragma unroll
                  for (int h = 0; h < 4; ++h) {
                    const float2 gf = unpack_bf16x2(gw[h]);
                    const float2 uf = unpack_bf16x2(uw[h]);
                    // grad_inter is rounded to bf16 first: the reference materialises it in bf16
                    const float go0 = bf16_round(__uint_as_float(r[v * 8 + 2 * h]));
                    const float go1 = bf16_round(__uint_as_float(r[v * 8 + 2 * h + 1]));
                    float gg0, gu0, gg1, gu1;
                    glu_bwd_val<CODE>(gf.x, uf.x, go0, gg0, gu0);
                    glu_bwd_val<CODE>(gf.y, uf.y, go1, gg1, gu1);
                    og[h] = pack_bf16x2(gg0, gg1);
                    ou[h] = pack_bf16x2(gu0, gu1);
                  }
                };
                if (POLY && act_code == 1) bwd8(std::integral_constant<int, 1>{});
                else if (POLY && act_code == 5) bwd8(std::integral_constant<int, 5>{});
                else bwd8(std::integral_constant<int, 0>{});
                *reinterpret_cast<uint4*>(ggu + col) = make_uint4(og[0], og[1], og[2], og[3]);
                *reinterpret_cast<uint4*>(ggu + I + col) = make_uint4(ou[0], ou[1], ou[2], ou[3]);
              }
            }
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) {
        if constexpr (CTAS == 2) mbar_arrive_cluster(tempty_leader + 8 * buf);
        else mbar_arrive(bar_tempty + 8 * buf);
      }
    }
    if constexpr (TMA_EPI) {
      if (lane == 0 || p.push_rank != nullptr) bulk_wait_all();   // every bulk store of this warp (push mode: of this lane) has completed
    }
  }

  // ------------------------------------------------------------------ tear-down
  tc_fence_before();
  __syncthreads();
  if constexpr (CTAS == 2) {   // nobody leaves while the peer may still touch it
    __syncwarp();
    cluster_sync_all();
  }
  if (threadIdx.x == 0 && *abort_flag != 0 && p.status != nullptr) atomicCAS(p.status, 0, *abort_flag);
  if (warp == 1) {
    __syncwarp();
    tc_fence_after();
    if constexpr (CTAS == 2) tmem_dealloc_pair(tmem_base, C::TMEM_COLS);
    else tmem_dealloc(tmem_base, C::TMEM_COLS);
  }
}

// ---------------------------------------------------------------------------- host side
template <int BN, int EPI, int CTAS, bool POLY = false>
static int launch(const CUtensorMap& tmA, const CUtensorMap& tmB, const CUtensorMap& tmD, const CUtensorMap& tmD2,
                  const GemmParams& p, int max_tiles, cudaStream_t stream) {
  using C = Cfg<BN, CTAS, epi_warp_bytes<BN, EPI>()>;
  static std::once_flag once;
  static cudaError_t attr_err = cudaSuccess;
  std::call_once(once, [] {
    attr_err = cudaFuncSetAttribute(gemm_kernel<BN, EPI, CTAS, POLY>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                    C::SMEM_BYTES);
  });
  if (attr_err != cudaSuccess) return cuda_fail(attr_err, "cudaFuncSetAttribute(max dynamic smem)");
  int units = gemm_cta_budget() / CTAS;  // CTAs, or CTA pairs
  if (max_tiles > 0 && max_tiles < units) units = max_tiles;
  if (units < 1) units = 1;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(units * CTAS, 1, 1);
  cfg.blockDim = dim3(kThreads, 1, 1);
  cfg.dynamicSmemBytes = C::SMEM_BYTES;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = CTAS;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = (CTAS > 1) ? 1 : 0;
  B200_CUDA(cudaLaunchKernelEx(&cfg, gemm_kernel<BN, EPI, CTAS, POLY>, tmA, tmB, tmD, tmD2, p));
  return 0;
}

// Pair (2-CTA) tiles are used for the grouped schedules with 256-wide tiles.  Setting the
// environment variable B200MOE_FORCE_1CTA=1 keeps every launch on single-CTA tiles (A/B measurements).
static bool pairs_enabled() {
  static int v = -1;
  static std::once_flag once;
  std::call_once(once, [] {
    const char* e = getenv("B200MOE_FORCE_1CTA");
    v = (e != nullptr && e[0] == '1') ? 0 : 1;
  });
  return v == 1;
}

// Operand description used by the host-side dispatcher.
struct Operand {
  const void* ptr;
  int mn_major;         // 0: (rows, K) row-major;  1: (K, rows) row-major
  long long rows;       // M (for A) or N (for B)
  long long k;          // reduction extent visible in this tensor
  long long ld;         // elements between consecutive rows of the stored matrix
  long long groups;     // stacked matrices (experts), 1 if none
  long long group_stride;
};

static int encode_operand(CUtensorMap* tm, const Operand& o, int tile_rows) {
  if (!o.mn_major)  // dims {K, rows, groups}, box {64, tile_rows}
    return make_map(tm, o.ptr, o.k, o.rows, o.groups, o.ld, o.group_stride, BK, tile_rows);
  // dims {rows(mn), K, groups}, box {64 mn, 64 k}
  return make_map(tm, o.ptr, o.rows, o.k, o.groups, o.ld, o.group_stride, 64, BK);
}

static int pick_bn(long long n) {
  if (n <= 64) return 64;
  if (n % 256 == 0 || n > 1024) {
    // prefer the wide tile unless it wastes more than 1/8 of the last tile
    long long waste256 = ((n + 255) / 256) * 256 - n;
    if (waste256 * 8 <= n) return 256;
  }
  return 128;
}

// d1 / d2 describe the bf16 outputs as {columns, rows, groups} tensors for the TMA-store epilogue
// (d2 = the SwiGLU `inter` output); they are ignored by the kernels that store directly.
template <int EPI, bool POLY = false>
static int dispatch_bn(int bn, const Operand& A, const Operand& B, const Operand* d1, const Operand* d2,
                       GemmParams& p, int max_tiles, cudaStream_t stream) {
  const bool pair = (bn == 256) && (p.sched != SCHED_DENSE) && pairs_enabled();
  CUtensorMap tmA, tmB, tmD, tmD2;
  int rc = encode_operand(&tmA, A, BM);
  if (rc) return rc;
  // rows of B one TMA box brings in: half a tile for SwiGLU (gate and up halves) and for pairs
  const int b_rows = (EPI == EPI_SWIGLU || pair) ? bn / 2 : bn;
  rc = encode_operand(&tmB, B, b_rows);
  if (rc) return rc;
  tmD = tmA;
  tmD2 = tmA;
  if (bn == 256 && EPI != EPI_STORE_F32 && p.push_rank == nullptr) {
    if (d1 == nullptr) {
      set_error("internal: output description missing");
      return B200MOE_E_UNSUPPORTED;
    }
    if (EPI == EPI_GLU_BWD) {   // boxes {32 columns, 32 rows}, 64-byte swizzle, for the in-place epilogue
      if (d2 == nullptr) {
        set_error("internal: saved gate_up description missing");
        return B200MOE_E_UNSUPPORTED;
      }
      rc = make_map(&tmD, d1->ptr, d1->k, d1->rows, d1->groups, d1->ld, d1->group_stride, 32, 32, 2, 64);
      if (rc) return rc;
      rc = make_map(&tmD2, d2->ptr, d2->k, d2->rows, d2->groups, d2->ld, d2->group_stride, 32, 32, 2, 64);
      if (rc) return rc;
    } else {
      rc = encode_operand(&tmD, *d1, 32);   // box {64 columns, 32 rows}
      if (rc) return rc;
      if (d2 != nullptr) {
        rc = encode_operand(&tmD2, *d2, 32);
        if (rc) return rc;
      } else if (p.sym_mirror) {            // the same output through boxes {32 columns, 64 rows}, no swizzle
        rc = make_map(&tmD2, d1->ptr, d1->k, d1->rows, d1->groups, d1->ld, d1->group_stride, 32, 64, 2, 0);
        if (rc) return rc;
      }
    }
  }
  if (pair) return launch<256, EPI, 2, POLY>(tmA, tmB, tmD, tmD2, p, max_tiles > 0 ? (max_tiles + 1) / 2 : 0, stream);
  if constexpr (EPI == EPI_AXPBY || EPI == EPI_STORE_SYM) {   // built for the 256-wide TMA-store epilogue only
    if (bn == 256) return launch<256, EPI, 1>(tmA, tmB, tmD, tmD2, p, max_tiles, stream);
    set_error("tile width %d not built for this epilogue", bn);
    return B200MOE_E_UNSUPPORTED;
  } else
  switch (bn) {
    case 256: return launch<256, EPI, 1, POLY>(tmA, tmB, tmD, tmD2, p, max_tiles, stream);
    case 128: return launch<128, EPI, 1, POLY>(tmA, tmB, tmD, tmD2, p, max_tiles, stream);
    default:
      if constexpr (EPI == EPI_STORE || EPI == EPI_STORE_F32)
        return launch<64, EPI, 1, POLY>(tmA, tmB, tmD, tmD2, p, max_tiles, stream);
      set_error("tile width %d not built for this epilogue", bn);
      return B200MOE_E_UNSUPPORTED;
  }
}


}  // namespace b200moe

using namespace b200moe;

extern "C" {

int b200moe_gemm_nt(const void* A, const void* B, void* D, int64_t M, int64_t N, int64_t K, int32_t* status,
                    b200moe_stream_t stream) {
  B200_CHECK_ARG(A && B && D, B200MOE_E_NULL, "gemm_nt: null pointer");
  CHECK_DIM8(N); CHECK_DIM8(K); CHECK_I32(M); CHECK_I32(N); CHECK_I32(K);
  if (M == 0) return 0;
  B200_CHECK_ARG(aligned16(D), B200MOE_E_ALIGN, "gemm_nt: D not 16-byte aligned");
  Operand a{A, 0, M, K, K, 1, M * K};
  Operand b{B, 0, N, K, K, 1, N * K};
  GemmParams p{};
  p.sched = SCHED_DENSE; p.M = (int)M; p.N = (int)N; p.K = (int)K; p.num_groups = 1;
  p.D = D; p.ldd = N; p.status = status;
  const int bn = pick_bn(N);
  Operand d{D, 0, M, N, N, 1, M * N};
  return dispatch_bn<EPI_STORE>(bn, a, b, &d, nullptr, p, (int)(ceil_div(M, BM) * ceil_div(N, bn)), (cudaStream_t)stream);
}

int b200moe_gemm_nn(const void* A, const void* B, void* D, int64_t M, int64_t N, int64_t K, int32_t* status,
                    b200moe_stream_t stream) {
  B200_CHECK_ARG(A && B && D, B200MOE_E_NULL, "gemm_nn: null pointer");
  CHECK_DIM8(N); CHECK_DIM8(K); CHECK_I32(M); CHECK_I32(N); CHECK_I32(K);
  if (M == 0) return 0;
  B200_CHECK_ARG(aligned16(D), B200MOE_E_ALIGN, "gemm_nn: D not 16-byte aligned");
  Operand a{A, 0, M, K, K, 1, M * K};
  Operand b{B, 1, N, K, N, 1, N * K};   // stored (K, N): MN-major
  GemmParams p{};
  p.sched = SCHED_DENSE; p.b_mn = 1; p.M = (int)M; p.N = (int)N; p.K = (int)K; p.num_groups = 1;
  p.D = D; p.ldd = N; p.status = status;
  const int bn = pick_bn(N);
  Operand d{D, 0, M, N, N, 1, M * N};
  return dispatch_bn<EPI_STORE>(bn, a, b, &d, nullptr, p, (int)(ceil_div(M, BM) * ceil_div(N, bn)), (cudaStream_t)stream);
}

int b200moe_gemm_tn_splitk(const void* A, const void* B, float* P, int64_t M, int64_t N, int64_t K,
                           int64_t k_chunk, int32_t* status, b200moe_stream_t stream) {
  B200_CHECK_ARG(A && B && P, B200MOE_E_NULL, "gemm_tn_splitk: null pointer");
  CHECK_DIM8(M); CHECK_DIM8(N); CHECK_I32(M); CHECK_I32(N); CHECK_I32(K);
  B200_CHECK_ARG(k_chunk > 0 && k_chunk % 64 == 0, B200MOE_E_BAD_SHAPE,
                 "gemm_tn_splitk: k_chunk = %lld must be a positive multiple of 64", (long long)k_chunk);
  B200_CHECK_ARG(K > 0, B200MOE_E_BAD_SHAPE, "gemm_tn_splitk: K must be positive");
  B200_CHECK_ARG(aligned16(P), B200MOE_E_ALIGN, "gemm_tn_splitk: P not 16-byte aligned");
  const long long slices = ceil_div(K, k_chunk);
  Operand a{A, 1, M, K, M, 1, M * K};   // stored (K, M)
  Operand b{B, 1, N, K, N, 1, N * K};   // stored (K, N)
  GemmParams p{};
  p.sched = SCHED_GROUPED_K; p.a_mn = 1; p.b_mn = 1; p.M = (int)M; p.N = (int)N; p.K = (int)K;
  p.num_groups = (int)slices; p.k_chunk = (int)k_chunk; p.poffs = nullptr;
  p.D = P; p.ldd = N; p.d_group_stride = M * N; p.status = status;
  const int bn = pick_bn(N);
  return dispatch_bn<EPI_STORE_F32>(bn, a, b, nullptr, nullptr, p, (int)(slices * ceil_div(M, BM) * ceil_div(N, bn)),
                                    (cudaStream_t)stream);
}

static int check_conv(const char* who, int64_t B, int64_t S, int64_t H, int64_t E, int taps, int64_t s_mult,
                      int64_t c_mult64) {
  B200_CHECK_ARG(B > 0 && S > 0 && taps >= 1 && taps <= 64, B200MOE_E_BAD_SHAPE, "%s: B = %lld, S = %lld, taps = %d", who,
                 (long long)B, (long long)S, taps);
  B200_CHECK_ARG(S % s_mult == 0, B200MOE_E_BAD_SHAPE, "%s: S = %lld must be a multiple of %lld", who, (long long)S,
                 (long long)s_mult);
  B200_CHECK_ARG(c_mult64 % 64 == 0, B200MOE_E_BAD_SHAPE, "%s: the convolved channel count %lld must be a multiple of 64",
                 who, (long long)c_mult64);
  B200_CHECK_ARG(H % 8 == 0 && E % 8 == 0 && H > 0 && E > 0, B200MOE_E_BAD_SHAPE, "%s: H = %lld, E = %lld", who,
                 (long long)H, (long long)E);
  B200_CHECK_ARG(B * S < (1LL << 31) && taps * H < (1LL << 31) && taps * E < (1LL << 31), B200MOE_E_BAD_SHAPE,
                 "%s: extent beyond 2^31", who);
  return 0;
}

int b200moe_conv_gemm_fwd(const void* x, const void* wf, void* logits, int64_t B, int64_t S, int64_t H, int64_t E, int taps,
                          int32_t* status, b200moe_stream_t stream) {
  B200_CHECK_ARG(x && wf && logits, B200MOE_E_NULL, "conv_gemm_fwd: null pointer");
  int rc = check_conv("conv_gemm_fwd", B, S, H, E, taps, BM, H);
  if (rc) return rc;
  B200_CHECK_ARG(aligned16(logits), B200MOE_E_ALIGN, "conv_gemm_fwd: logits not 16-byte aligned");
  const int64_t M = B * S, K = taps * H;
  Operand a{x, 0, S, H, H, B, S * H};       // {H, S, B}: positions outside [0, S) read as zero
  Operand b{wf, 0, E, K, K, 1, E * K};
  GemmParams p{};
  p.sched = SCHED_DENSE; p.M = (int)M; p.N = (int)E; p.K = (int)K; p.num_groups = 1;
  p.D = logits; p.ldd = E; p.status = status;
  p.conv_taps = taps; p.conv_S = (int)S; p.conv_C = (int)H; p.conv_sign = 1;
  const int bn = pick_bn(E);
  Operand d{logits, 0, M, E, E, 1, M * E};
  return dispatch_bn<EPI_STORE, true>(bn, a, b, &d, nullptr, p, (int)(ceil_div(M, BM) * ceil_div(E, bn)), (cudaStream_t)stream);
}

int b200moe_conv_gemm_dx(const void* grad_logits, const void* wb, void* grad_x, int64_t B, int64_t S, int64_t H, int64_t E,
                         int taps, int32_t* status, b200moe_stream_t stream) {
  B200_CHECK_ARG(grad_logits && wb && grad_x, B200MOE_E_NULL, "conv_gemm_dx: null pointer");
  int rc = check_conv("conv_gemm_dx", B, S, H, E, taps, BM, E);
  if (rc) return rc;
  B200_CHECK_ARG(aligned16(grad_x), B200MOE_E_ALIGN, "conv_gemm_dx: grad_x not 16-byte aligned");
  const int64_t M = B * S, K = taps * E;
  Operand a{grad_logits, 0, S, E, E, B, S * E};   // {E, S, B}, read (taps - 1) - tap positions ahead
  Operand b{wb, 1, H, K, H, 1, H * K};            // stored (taps * E, H): MN-major
  GemmParams p{};
  p.sched = SCHED_DENSE; p.b_mn = 1; p.M = (int)M; p.N = (int)H; p.K = (int)K; p.num_groups = 1;
  p.D = grad_x; p.ldd = H; p.status = status;
  p.conv_taps = taps; p.conv_S = (int)S; p.conv_C = (int)E; p.conv_sign = -1;
  const int bn = pick_bn(H);
  Operand d{grad_x, 0, M, H, H, 1, M * H};
  return dispatch_bn<EPI_STORE, true>(bn, a, b, &d, nullptr, p, (int)(ceil_div(M, BM) * ceil_div(H, bn)), (cudaStream_t)stream);
}

int b200moe_conv_gemm_dw_splitk(const void* grad_logits, const void* x, float* P, int64_t B, int64_t S, int64_t H,
                                int64_t E, int taps, int64_t k_chunk, int32_t* status, b200moe_stream_t stream) {
  B200_CHECK_ARG(grad_logits && x && P, B200MOE_E_NULL, "conv_gemm_dw_splitk: null pointer");
  int rc = check_conv("conv_gemm_dw_splitk", B, S, H, E, taps, 64, H);
  if (rc) return rc;
  B200_CHECK_ARG(k_chunk > 0 && k_chunk % 64 == 0, B200MOE_E_BAD_SHAPE,
                 "conv_gemm_dw_splitk: k_chunk = %lld must be a positive multiple of 64", (long long)k_chunk);
  B200_CHECK_ARG(aligned16(P), B200MOE_E_ALIGN, "conv_gemm_dw_splitk: P not 16-byte aligned");
  const int64_t K = B * S, N = taps * H;
  const long long slices = ceil_div(K, k_chunk);
  Operand a{grad_logits, 1, E, K, E, 1, E * K};   // stored (B*S, E)
  Operand b{x, 1, H, S, H, B, S * H};             // {H, S, B}: the k rows of tap j are read j - (taps - 1) positions away
  GemmParams p{};
  p.sched = SCHED_GROUPED_K; p.a_mn = 1; p.b_mn = 1; p.M = (int)E; p.N = (int)N; p.K = (int)K;
  p.num_groups = (int)slices; p.k_chunk = (int)k_chunk; p.poffs = nullptr;
  p.D = P; p.ldd = N; p.d_group_stride = E * N; p.status = status;
  p.conv_taps = taps; p.conv_S = (int)S; p.conv_C = (int)H; p.conv_sign = 1;
  const int bn = H % 256 == 0 ? 256 : (H % 128 == 0 ? 128 : 64);   // a tile's columns belong to one tap
  return dispatch_bn<EPI_STORE_F32, true>(bn, a, b, nullptr, nullptr, p, (int)(slices * ceil_div(E, BM) * ceil_div(N, bn)),
                                    (cudaStream_t)stream);
}

// row window of a grouped-M launch: (0, 0) = every row, else tile-aligned 0 <= row_lo < row_hi <= rows_cap
static int check_row_window(const char* who, int64_t rows_cap, int64_t row_lo, int64_t row_hi) {
  if (row_lo == 0 && row_hi == 0) return 0;
  B200_CHECK_ARG(row_lo >= 0 && row_lo < row_hi && row_hi <= rows_cap && row_lo % B200MOE_TILE_M == 0 &&
                     row_hi % B200MOE_TILE_M == 0,
                 B200MOE_E_BAD_SHAPE, "%s: row window [%lld, %lld) must be tile-aligned and inside %lld rows", who,
                 (long long)row_lo, (long long)row_hi, (long long)rows_cap);
  return 0;
}

static int check_grouped(const char* who, const void* a, const void* b, const void* c, const int32_t* tile_expert,
                         const int32_t* poffs, int64_t rows_cap, int E, int64_t H, int64_t I) {
  B200_CHECK_ARG(a && b && c && poffs, B200MOE_E_NULL, "%s: null pointer", who);
  (void)tile_expert;
  B200_CHECK_ARG(E >= 1 && E <= 65535, B200MOE_E_BAD_SHAPE, "%s: E = %d out of range", who, E);
  B200_CHECK_ARG(rows_cap > 0 && rows_cap % B200MOE_TILE_M == 0 && rows_cap < (1LL << 31), B200MOE_E_BAD_SHAPE,
                 "%s: rows_cap = %lld must be a positive multiple of %d", who, (long long)rows_cap, B200MOE_TILE_M);
  B200_CHECK_ARG(H > 0 && H % 8 == 0 && I > 0 && I % 8 == 0, B200MOE_E_BAD_SHAPE,
                 "%s: H = %lld and I = %lld must be positive multiples of 8", who, (long long)H, (long long)I);
  B200_CHECK_ARG(2 * E * I < (1LL << 31) && E * H < (1LL << 31), B200MOE_E_BAD_SHAPE, "%s: weight stack too tall", who);
  return 0;
}

int b200moe_expert_gate_up_swiglu(const void* x_s, const void* gate_up_proj, const int32_t* tile_expert,
                                  const int32_t* poffs, int64_t rows_cap, int E, int64_t H, int64_t I,
                                  void* gate_up, void* inter, int32_t* status, b200moe_stream_t stream) {
  return b200moe_expert_gate_up_act(x_s, gate_up_proj, nullptr, tile_expert, poffs, rows_cap, 0, 0, E, H, I, gate_up,
                                    inter, status, stream);
}

int b200moe_expert_gate_up_act(const void* x_s, const void* gate_up_proj, const int32_t* act_codes,
                               const int32_t* tile_expert, const int32_t* poffs, int64_t rows_cap, int64_t row_lo,
                               int64_t row_hi, int E, int64_t H, int64_t I, void* gate_up, void* inter,
                               int32_t* status, b200moe_stream_t stream) {
  int rc = check_grouped("expert_gate_up_swiglu", x_s, gate_up_proj, gate_up, tile_expert, poffs, rows_cap, E, H, I);
  if (rc) return rc;
  rc = check_row_window("expert_gate_up_swiglu", rows_cap, row_lo, row_hi);
  if (rc) return rc;
  B200_CHECK_ARG(inter && tile_expert, B200MOE_E_NULL, "expert_gate_up_swiglu: null pointer");
  B200_CHECK_ARG(aligned16(gate_up) && aligned16(inter), B200MOE_E_ALIGN, "expert_gate_up_swiglu: outputs not aligned");
  Operand a{x_s, 0, rows_cap, H, H, 1, rows_cap * H};
  // W_gu (E, 2I, H) seen as dims {H, I, 2E}: group 2e = gate rows of expert e, 2e+1 = up rows
  Operand b{gate_up_proj, 0, I, H, H, 2LL * E, I * H};
  GemmParams p{};
  p.sched = SCHED_GROUPED_M; p.N = (int)I; p.K = (int)H; p.num_groups = E;
  p.tile_expert = tile_expert; p.poffs = poffs; p.D = gate_up; p.aux = inter; p.I = (int)I; p.status = status;
  p.row_lo = (int)row_lo; p.row_hi = (int)row_hi;
  const int bn = (I >= 128) ? 256 : 128;   // tile covers bn/2 intermediate columns
  Operand d1{gate_up, 0, rows_cap, I, 2 * I, 2, I};       // {I, rows, 2}: group 0 = gate half, 1 = up half
  Operand d2{inter, 0, rows_cap, I, I, 1, rows_cap * I};
  if (act_codes != nullptr) {
    p.act_codes = act_codes;
    return dispatch_bn<EPI_SWIGLU, true>(bn, a, b, &d1, &d2, p, 0, (cudaStream_t)stream);
  }
  return dispatch_bn<EPI_SWIGLU>(bn, a, b, &d1, &d2, p, 0, (cudaStream_t)stream);
}

int b200moe_expert_linear(const void* a, const void* w, const int32_t* tile_expert, const int32_t* poffs,
                          int64_t rows_cap, int E, int64_t N, int64_t K, void* out, int32_t* status,
                          b200moe_stream_t stream) {
  int rc = check_grouped("expert_linear", a, w, out, tile_expert, poffs, rows_cap, E, N, K);
  if (rc) return rc;
  B200_CHECK_ARG(tile_expert, B200MOE_E_NULL, "expert_linear: null pointer");
  B200_CHECK_ARG(aligned16(out), B200MOE_E_ALIGN, "expert_linear: output not aligned");
  Operand oa{a, 0, rows_cap, K, K, 1, rows_cap * K};
  Operand ob{w, 0, N, K, K, E, N * K};   // W (E, N, K): rows = output columns
  GemmParams p{};
  p.sched = SCHED_GROUPED_M; p.N = (int)N; p.K = (int)K; p.num_groups = E;
  p.tile_expert = tile_expert; p.poffs = poffs; p.D = out; p.ldd = N; p.status = status;
  Operand d{out, 0, rows_cap, N, N, 1, rows_cap * N};
  return dispatch_bn<EPI_STORE>(pick_bn(N) == 64 ? 128 : pick_bn(N), oa, ob, &d, nullptr, p, 0, (cudaStream_t)stream);
}

int b200moe_expert_gram(const void* x, const int32_t* tile_expert, const int32_t* poffs, int64_t rows_cap, int E,
                        int64_t K, int mirror, void* out, int32_t* status, b200moe_stream_t stream) {
  B200_CHECK_ARG(E >= 1 && rows_cap % E == 0, B200MOE_E_BAD_SHAPE, "expert_gram: %lld rows do not split into %d equal groups",
                 (long long)rows_cap, E);
  const int64_t R = rows_cap / E;
  int rc = check_grouped("expert_gram", x, x, out, tile_expert, poffs, rows_cap, E, R, K);
  if (rc) return rc;
  B200_CHECK_ARG(tile_expert, B200MOE_E_NULL, "expert_gram: null pointer");
  B200_CHECK_ARG(R % 256 == 0, B200MOE_E_BAD_SHAPE, "expert_gram: %lld rows per group must be a multiple of 256", (long long)R);
  B200_CHECK_ARG(aligned16(out), B200MOE_E_ALIGN, "expert_gram: output not aligned");
  Operand oa{x, 0, rows_cap, K, K, 1, rows_cap * K};
  Operand ob{x, 0, R, K, K, E, R * K};
  GemmParams p{};
  p.sched = SCHED_GROUPED_M; p.N = (int)R; p.K = (int)K; p.num_groups = E; p.sym_rows = (int)R; p.sym_mirror = mirror ? 1 : 0;
  p.tile_expert = tile_expert; p.poffs = poffs; p.D = out; p.ldd = R; p.status = status;
  Operand d{out, 0, rows_cap, R, R, 1, rows_cap * R};
  return dispatch_bn<EPI_STORE_SYM>(256, oa, ob, &d, nullptr, p, 0, (cudaStream_t)stream);
}

int b200moe_expert_linear_axpby(const void* a, const void* w, const void* c, float alpha, float beta, float diag,
                                int symmetric, const int32_t* tile_expert, const int32_t* poffs, int64_t rows_cap, int E,
                                int64_t N, int64_t K, void* out, int32_t* status, b200moe_stream_t stream) {
  int rc = check_grouped("expert_linear_axpby", a, w, out, tile_expert, poffs, rows_cap, E, N, K);
  if (rc) return rc;
  B200_CHECK_ARG(tile_expert && c, B200MOE_E_NULL, "expert_linear_axpby: null pointer");
  B200_CHECK_ARG(N % 256 == 0, B200MOE_E_BAD_SHAPE, "expert_linear_axpby: N = %lld must be a multiple of 256", (long long)N);
  B200_CHECK_ARG(aligned16(out) && aligned16(c), B200MOE_E_ALIGN, "expert_linear_axpby: pointers must be 16-byte aligned");
  Operand oa{a, 0, rows_cap, K, K, 1, rows_cap * K};
  Operand ob{w, 0, N, K, K, E, N * K};   // W (E, N, K): rows = output columns
  GemmParams p{};
  p.sched = SCHED_GROUPED_M; p.N = (int)N; p.K = (int)K; p.num_groups = E;
  p.tile_expert = tile_expert; p.poffs = poffs; p.D = out; p.ldd = N; p.status = status;
  p.aux = const_cast<void*>(c); p.ax_alpha = alpha; p.ax_beta = beta; p.ax_diag = diag;
  if (symmetric) {
    B200_CHECK_ARG(rows_cap == (int64_t)E * N, B200MOE_E_BAD_SHAPE,
                   "expert_linear_axpby: a symmetric result needs %d equal groups of N = %lld rows", E, (long long)N);
    p.sym_rows = (int)N;
    p.sym_mirror = symmetric > 1 ? 1 : 0;
  }
  Operand d{out, 0, rows_cap, N, N, 1, rows_cap * N};
  return dispatch_bn<EPI_AXPBY>(256, oa, ob, &d, nullptr, p, 0, (cudaStream_t)stream);
}

int b200moe_expert_linear_t(const void* a, const void* w, const int32_t* tile_expert, const int32_t* poffs,
                            int64_t rows_cap, int E, int64_t K, int64_t N, void* out, int32_t* status,
                            b200moe_stream_t stream) {
  int rc = check_grouped("expert_linear_t", a, w, out, tile_expert, poffs, rows_cap, E, N, K);
  if (rc) return rc;
  B200_CHECK_ARG(tile_expert, B200MOE_E_NULL, "expert_linear_t: null pointer");
  B200_CHECK_ARG(aligned16(out), B200MOE_E_ALIGN, "expert_linear_t: output not aligned");
  Operand oa{a, 0, rows_cap, K, K, 1, rows_cap * K};
  Operand ob{w, 1, N, K, N, E, K * N};   // W[e] stored (K, N): MN-major
  GemmParams p{};
  p.sched = SCHED_GROUPED_M; p.b_mn = 1; p.N = (int)N; p.K = (int)K; p.num_groups = E;
  p.tile_expert = tile_expert; p.poffs = poffs; p.D = out; p.ldd = N; p.status = status;
  Operand d{out, 0, rows_cap, N, N, 1, rows_cap * N};
  return dispatch_bn<EPI_STORE>(pick_bn(N) == 64 ? 128 : pick_bn(N), oa, ob, &d, nullptr, p, 0, (cudaStream_t)stream);
}

int b200moe_expert_linear_push(const void* a, const void* w, int w_kn, const int32_t* tile_expert, const int32_t* poffs,
                               int64_t rows_cap, int E, int64_t N, int64_t K, const int32_t* row_rank,
                               const int32_t* row_slot, const int64_t* peer_base, int32_t* status,
                               b200moe_stream_t stream) {
  int rc = check_grouped("expert_linear_push", a, w, peer_base, tile_expert, poffs, rows_cap, E, N, K);
  if (rc) return rc;
  B200_CHECK_ARG(tile_expert && row_rank && row_slot && peer_base, B200MOE_E_NULL, "expert_linear_push: null pointer");
  B200_CHECK_ARG(N % 64 == 0, B200MOE_E_BAD_SHAPE, "expert_linear_push: N = %lld must be a multiple of 64", (long long)N);
  Operand oa{a, 0, rows_cap, K, K, 1, rows_cap * K};
  Operand ob_nk{w, 0, N, K, K, E, N * K};   // W (E, N, K): rows = output columns
  Operand ob_kn{w, 1, N, K, N, E, K * N};   // W[e] stored (K, N): MN-major
  GemmParams p{};
  p.sched = SCHED_GROUPED_M; p.b_mn = w_kn ? 1 : 0; p.N = (int)N; p.K = (int)K; p.num_groups = E;
  p.tile_expert = tile_expert; p.poffs = poffs; p.D = nullptr; p.ldd = N; p.status = status;
  p.push_rank = row_rank; p.push_slot = row_slot; p.push_base = reinterpret_cast<const long long*>(peer_base);
  return dispatch_bn<EPI_STORE>(256, oa, w_kn ? ob_kn : ob_nk, nullptr, nullptr, p, 0, (cudaStream_t)stream);
}

int b200moe_expert_down(const void* inter, const void* down_proj, const int32_t* tile_expert, const int32_t* poffs,
                        int64_t rows_cap, int E, int64_t H, int64_t I, void* eo, int32_t* status,
                        b200moe_stream_t stream) {
  return b200moe_expert_linear(inter, down_proj, tile_expert, poffs, rows_cap, E, H, I, eo, status, stream);
}

int b200moe_expert_down_dgrad_glu(const void* grad_eo, const void* down_proj, const void* gate_up,
                                  const int32_t* tile_expert, const int32_t* poffs, int64_t rows_cap, int E,
                                  int64_t H, int64_t I, void* grad_gate_up, int32_t* status,
                                  b200moe_stream_t stream) {
  return b200moe_expert_down_dgrad_act(grad_eo, down_proj, gate_up, nullptr, tile_expert, poffs, rows_cap, 0, 0, E, H, I,
                                       grad_gate_up, status, stream);
}

int b200moe_expert_down_dgrad_act(const void* grad_eo, const void* down_proj, const void* gate_up,
                                  const int32_t* act_codes, const int32_t* tile_expert, const int32_t* poffs,
                                  int64_t rows_cap, int64_t row_lo, int64_t row_hi, int E, int64_t H, int64_t I,
                                  void* grad_gate_up, int32_t* status, b200moe_stream_t stream) {
  int rc = check_grouped("expert_down_dgrad_glu", grad_eo, down_proj, grad_gate_up, tile_expert, poffs, rows_cap, E, H, I);
  if (rc) return rc;
  rc = check_row_window("expert_down_dgrad_glu", rows_cap, row_lo, row_hi);
  if (rc) return rc;
  B200_CHECK_ARG(gate_up && tile_expert, B200MOE_E_NULL, "expert_down_dgrad_glu: null pointer");
  B200_CHECK_ARG(aligned16(grad_gate_up) && aligned16(gate_up), B200MOE_E_ALIGN, "expert_down_dgrad_glu: not aligned");
  Operand a{grad_eo, 0, rows_cap, H, H, 1, rows_cap * H};
  Operand b{down_proj, 1, I, H, I, E, H * I};   // W_d[e] stored (K=H, N=I): MN-major
  GemmParams p{};
  p.sched = SCHED_GROUPED_M; p.b_mn = 1; p.N = (int)I; p.K = (int)H; p.num_groups = E;
  p.tile_expert = tile_expert; p.poffs = poffs; p.D = grad_gate_up; p.aux = const_cast<void*>(gate_up);
  p.I = (int)I; p.status = status;
  p.row_lo = (int)row_lo; p.row_hi = (int)row_hi;
  const int bn = pick_bn(I) == 64 ? 128 : pick_bn(I);
  Operand d{grad_gate_up, 0, rows_cap, I, 2 * I, 2, I};   // {I, rows, 2}: grad_gate half, grad_up half
  Operand d2{gate_up, 0, rows_cap, I, 2 * I, 2, I};       // the saved forward gate_up, same view (input)
  if (act_codes != nullptr) {
    p.act_codes = act_codes;
    return dispatch_bn<EPI_GLU_BWD, true>(bn, a, b, &d, &d2, p, 0, (cudaStream_t)stream);
  }
  return dispatch_bn<EPI_GLU_BWD>(bn, a, b, &d, &d2, p, 0, (cudaStream_t)stream);
}

int b200moe_expert_gate_up_dgrad(const void* grad_gate_up, const void* gate_up_proj, const int32_t* tile_expert,
                                 const int32_t* poffs, int64_t rows_cap, int E, int64_t H, int64_t I,
                                 void* grad_x_s, int32_t* status, b200moe_stream_t stream) {
  return b200moe_expert_linear_t(grad_gate_up, gate_up_proj, tile_expert, poffs, rows_cap, E, 2 * I, H, grad_x_s,
                                 status, stream);
}

int b200moe_expert_wgrad(const void* A, const void* B, const int32_t* poffs, const int32_t* counts, int64_t rows_cap,
                         int E, int64_t Na, int64_t Nb, void* out, int32_t* status, b200moe_stream_t stream) {
  B200_CHECK_ARG(A && B && poffs && out, B200MOE_E_NULL, "expert_wgrad: null pointer");
  B200_CHECK_ARG(E >= 1, B200MOE_E_BAD_SHAPE, "expert_wgrad: E = %d", E);
  B200_CHECK_ARG(rows_cap > 0 && rows_cap % B200MOE_TILE_M == 0 && rows_cap < (1LL << 31), B200MOE_E_BAD_SHAPE,
                 "expert_wgrad: rows_cap = %lld must be a positive multiple of %d", (long long)rows_cap, B200MOE_TILE_M);
  CHECK_DIM8(Na); CHECK_DIM8(Nb); CHECK_I32(Na); CHECK_I32(Nb);
  B200_CHECK_ARG(aligned16(out), B200MOE_E_ALIGN, "expert_wgrad: output not aligned");
  Operand a{A, 1, Na, rows_cap, Na, 1, rows_cap * Na};
  Operand b{B, 1, Nb, rows_cap, Nb, 1, rows_cap * Nb};
  GemmParams p{};
  p.sched = SCHED_GROUPED_K; p.a_mn = 1; p.b_mn = 1; p.M = (int)Na; p.N = (int)Nb; p.K = (int)rows_cap;
  p.num_groups = E; p.poffs = poffs; p.counts = counts; p.D = out; p.ldd = Nb; p.d_group_stride = Na * Nb;
  p.status = status;
  const int bn = pick_bn(Nb);
  Operand d{out, 0, Na, Nb, Nb, E, Na * Nb};
  return dispatch_bn<EPI_STORE>(bn, a, b, &d, nullptr, p, (int)std::min<long long>(1 << 30, E * ceil_div(Na, BM) * ceil_div(Nb, bn)),
                                (cudaStream_t)stream);
}

}  // extern "C"
