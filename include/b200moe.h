/* libb200moe — C ABI of the B200 (sm_100a) MoE hot path.
 *
 * The reference (IsNoobgrammer/triton-kernel-fused) has no native interface: its boundary is a set
 * of Python callables (kernels/sm75/moe.py:838 `moe`, kernels/sm75/router.py:277 `fused_mlp_router`,
 * :292 `router_bias_update`).  This library sits underneath a Python package that keeps those
 * signatures; each entry point below replaces one launch site of the reference and cites it.
 *
 * Conventions
 *   - every pointer is a DEVICE pointer unless it says "host"; the library never allocates or frees
 *     device memory and never synchronises the device; all work is queued on `stream`;
 *   - bf16 matrices are row-major and contiguous unless a leading dimension is given;
 *   - return value: 0 on success, a negative B200MOE_E_* code otherwise (nothing was launched);
 *     b200moe_last_error_string() describes the last failure on the calling thread;
 *   - `status` is a caller-owned device int32, zero-initialised once.  Kernels write a non-zero
 *     code there when a bounded wait ran out or an index was out of range (see
 *     b200moe_status_string); the word is never cleared by the library;
 *   - "padded rows": routed rows live in an expert-contiguous layout in which expert e owns rows
 *     [poffs[e], poffs[e+1]) and every segment is a multiple of B200MOE_TILE_M rows; rows past the
 *     expert's count are zero rows.  Buffers are sized for the worst case b200moe_padded_rows_cap().
 */
#ifndef B200MOE_H_
#define B200MOE_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct CUstream_st* b200moe_stream_t; /* == cudaStream_t */

#define B200MOE_TILE_M 256
#define B200MOE_MAX_EXPERTS 256
#define B200MOE_MAX_TOPK 32

enum {
  B200MOE_OK = 0,
  B200MOE_E_BAD_SHAPE = -1,
  B200MOE_E_ALIGN = -2,
  B200MOE_E_UNSUPPORTED = -3,
  B200MOE_E_WS_TOO_SMALL = -4,
  B200MOE_E_CUDA = -5,
  B200MOE_E_NULL = -6
};

/* kinds of router input accepted by the top-k epilogue */
enum { B200MOE_LOGITS_BF16 = 0, B200MOE_LOGITS_F32 = 1, B200MOE_SCORES_F32 = 2 };

const char* b200moe_version(void);
const char* b200moe_last_error_string(void);
/* host: text for a value read back from a `status` word */
const char* b200moe_status_string(int status_word);
/* host: worst-case number of padded rows for M routed rows over E experts */
int64_t b200moe_padded_rows_cap(int64_t M, int E);

/* Failure-path self-test, no reference counterpart: one CTA waits (at most `limit_cycles` SM clocks,
 * 1e3..2e9) on a barrier that nothing completes; the wait gives up, `status` receives 6 and the kernel
 * returns normally.  Shows that a stalled pipeline ends in a status code, not in a hung GPU. */
int b200moe_selftest_bounded_wait(int32_t* status, int64_t limit_cycles, b200moe_stream_t stream);

/* host: keep `n` SMs free of the persistent GEMM kernels (process-wide, default 0) so that
 * communication kernels queued on another stream can run beside them.  No reference counterpart. */
int b200moe_set_reserved_sms(int n);
/* host: let b200moe_ep_combine_pull occupy at most `n` SMs (one 1024-thread CTA each; 0 = all SMs), the
 * counterpart of b200moe_set_reserved_sms when a pull runs beside a GEMM.  No reference counterpart. */
int b200moe_set_exchange_sms(int n);

/* ---- router --------------------------------------------------------------------------------- */
/* Replaces _router_epilogue_fwd_kernel (kernels/sm75/router.py:39-83, launcher :129-148):
 * sigmoid, +bias for selection only, k rounds of lowest-index argmax with knock-out, unbiased
 * weights, optional /(sum+1e-20), *scale; counts (nullable) are zeroed then accumulated.
 * input: (T,E) of `input_kind`; bias: (E) fp32 or NULL; idx: (T,k) int64; w: (T,k) fp32. */
int b200moe_router_topk_fwd(const void* input, int input_kind, const float* bias, int64_t T, int E,
                            int k, int norm_topk, float scale, int64_t* idx, float* w,
                            int32_t* counts, b200moe_stream_t stream);

/* Replaces _router_epilogue_bwd_kernel (kernels/sm75/router.py:86-126): grad_logits (T,E) bf16. */
int b200moe_router_topk_bwd(const void* logits, int input_kind, const int64_t* idx,
                            const float* grad_w, int64_t T, int E, int k, int norm_topk, float scale,
                            void* grad_logits, b200moe_stream_t stream);

/* Replaces router_bias_update (kernels/sm75/router.py:292-301): b += u*sign(mean(c)-c); no-op u<=0. */
int b200moe_router_bias_update(float* bias, const int32_t* counts, int E, float u,
                               b200moe_stream_t stream);

/* Conv-router front end (kernels/sm75/router.py:186-190 conv1d with padding K-1, :214-218 backward):
 * unfold: xu (B*S, K*H) with xu[(b,s), j*H+h] = x[b, s-(K-1)+j, h] or 0, so that the causal K-tap conv is one
 * GEMM against Wf (E, K*H), Wf[e, j*H+h] = W[e,h,j];  fold: grad_x[b,s,h] = sum_j grad_xu[(b,s+K-1-j), j*H+h]. */
int b200moe_conv_unfold(const void* x, int64_t B, int64_t S, int64_t H, int K, void* xu, b200moe_stream_t stream);
int b200moe_conv_fold(const void* grad_xu, int64_t B, int64_t S, int64_t H, int K, void* grad_x,
                      b200moe_stream_t stream);

/* The same convolution WITHOUT the unfolded copy (what the reference's one-launch conv router does,
 * kernels/sm120/router.py:34-85): the GEMM's TMA producer reads x through a {H, S, B} tensor map, one 64-channel box
 * per (tap, channel block), `tap - (K-1)` positions away from the tile's rows; positions before the sequence start
 * are out of the map's bounds and arrive as zeros (the causal padding).
 * fwd: logits (B*S, E) = conv(x (B,S,H), Wf (E, K*H));  needs S % 128 == 0 (a row tile stays inside one sequence)
 *      and H % 64 == 0.
 * dx:  grad_x (B*S, H) from grad_logits (B,S,E) and Wb (K*E, H), Wb[j*E+e, h] = W[e,h,j]; S % 128 == 0, E % 64 == 0.
 * dw_splitk: fp32 slices P[s] (E, K*H) of grad_Wf = grad_logits^T * unfold(x) over chunks of k_chunk rows (multiple
 *      of 64), to be summed by b200moe_splitk_reduce; S % 64 == 0, H % 64 == 0.
 * Other shapes take b200moe_conv_unfold / conv_fold with the plain GEMMs. */
int b200moe_conv_gemm_fwd(const void* x, const void* wf, void* logits, int64_t B, int64_t S, int64_t H, int64_t E,
                          int taps, int32_t* status, b200moe_stream_t stream);
int b200moe_conv_gemm_dx(const void* grad_logits, const void* wb, void* grad_x, int64_t B, int64_t S, int64_t H,
                         int64_t E, int taps, int32_t* status, b200moe_stream_t stream);
int b200moe_conv_gemm_dw_splitk(const void* grad_logits, const void* x, float* P, int64_t B, int64_t S, int64_t H,
                                int64_t E, int taps, int64_t k_chunk, int32_t* status, b200moe_stream_t stream);

/* ---- dense bf16 GEMMs on tcgen05 (router projections) ----------------------------------------
 * Replace the cuBLAS calls at kernels/sm75/router.py:235 (logits), :258 (dX), :259 (dW).
 * nt: D(M,N) = A(M,K) * B(N,K)^T      nn: D(M,N) = A(M,K) * B(K,N)
 * tn_splitk: P[s](M,N) fp32 = A(Kc_s,M)^T * B(Kc_s,N) over K-chunk s of `k_chunk` rows (multiple
 * of 64); P holds ceil(K/k_chunk) slices; splitk_reduce sums the slices into bf16 D(M,N).
 * All leading dimensions and N, K must be multiples of 8 elements; base pointers 16-byte aligned. */
int b200moe_gemm_nt(const void* A, const void* B, void* D, int64_t M, int64_t N, int64_t K,
                    int32_t* status, b200moe_stream_t stream);
int b200moe_gemm_nn(const void* A, const void* B, void* D, int64_t M, int64_t N, int64_t K,
                    int32_t* status, b200moe_stream_t stream);
int b200moe_gemm_tn_splitk(const void* A, const void* B, float* P, int64_t M, int64_t N, int64_t K,
                           int64_t k_chunk, int32_t* status, b200moe_stream_t stream);
int b200moe_splitk_reduce(const float* P, int64_t slices, int64_t elems, void* D,
                          b200moe_stream_t stream);

/* ---- permutation ---------------------------------------------------------------------------- */
size_t b200moe_permute_ws_bytes(int64_t M, int E);
/* Replaces _sort_by_expert + _build_schedule (kernels/sm75/moe.py:564-572, :535-543) with a stable
 * counting sort done on the device, no host sync.  idx: (T,k) int64.
 * Outputs: counts (E), offs (E+1) compact end-exclusive scan, poffs (E+1) padded scan,
 * slot_row (T*k) padded row of slot t*k+j, row_slot (cap) slot of each padded row or -1 (only rows
 * below poffs[E] are written), tile_expert (cap/B200MOE_TILE_M) expert of each row tile,
 * order (T*k, nullable) = the stable argsort of idx.flatten() (compact row -> slot),
 * slot_pos (T*k, nullable) = its inverse (slot -> compact row). ws: scratch, ws_bytes from above. */
int b200moe_permute_build(const int64_t* idx, int64_t T, int k, int E, int32_t* counts,
                          int32_t* offs, int32_t* poffs, int32_t* slot_row, int32_t* row_slot,
                          int32_t* tile_expert, int32_t* order, int32_t* slot_pos, void* ws,
                          size_t ws_bytes, int32_t* status, b200moe_stream_t stream);

/* No counterpart in the reference.  Same outputs as b200moe_permute_build, for callers that cannot
 * allocate device memory (a plugin inside a framework that owns all free memory, a latency-bound loop
 * where cudaMalloc's device-wide synchronisation is not allowed): the histogram scratch is a fixed
 * 1 MiB array inside the library, so ceil(T*k/512)*E*4 bytes must not exceed 1 MiB (e.g. T*k <= 2 097 152
 * at E = 64, 524 288 at E = 256); larger problems return B200MOE_E_WS_TOO_SMALL.  Allocates nothing.
 * The first call on each device looks the array's address up (cudaGetSymbolAddress, with that device
 * current); make that first call before any stream capture begins.  All calls on a device share the
 * one array: two calls whose kernels can overlap on the GPU (different streams) race on it. */
int b200moe_permute_build_static(const int64_t* idx, int64_t T, int k, int E, int32_t* counts,
                                 int32_t* offs, int32_t* poffs, int32_t* slot_row, int32_t* row_slot,
                                 int32_t* tile_expert, int32_t* order, int32_t* slot_pos,
                                 int32_t* status, b200moe_stream_t stream);

/* Replaces hidden.index_select(0, st) (kernels/sm75/moe.py:744, :589): x_s[r] = x[row_slot[r]/k],
 * zero rows where row_slot[r] < 0.  Only rows below *total_rows (device) are written. */
int b200moe_gather_rows(const void* x, const int32_t* row_slot, const int32_t* total_rows, int k,
                        int64_t H, int64_t rows_cap, void* x_s, b200moe_stream_t stream);

/* ---- grouped expert GEMMs (tcgen05, persistent, TMA-fed) -------------------------------------
 * All take the tables from b200moe_permute_build; `rows_cap` bounds the padded-row buffers. */
/* Replaces the gate/up GEMM + _glu_fwd (kernels/sm75/moe.py:590-591, :765-767), act code 0:
 * gate_up (rows,2I) bf16 = x_s * W_gu[e]^T (cols [0,I) gate, [I,2I) up); inter = silu(gate)*up. */
int b200moe_expert_gate_up_swiglu(const void* x_s, const void* gate_up_proj,
                                  const int32_t* tile_expert, const int32_t* poffs,
                                  int64_t rows_cap, int E, int64_t H, int64_t I, void* gate_up,
                                  void* inter, int32_t* status, b200moe_stream_t stream);
/* The same GEMM with a per-expert activation code (act_codes (E) int32: 0 SiLU, 1 ReLU^2, 5 SiTU = tanh(g)*sigmoid(g),
 * the parameter-free codes of _act_eager, kernels/sm75/moe.py:859-881, that need no row reduction) applied in the
 * epilogue in place of the separate _glu_fwd launch (kernels/sm75/moe.py:767); act_codes NULL = all SiLU.
 * [row_lo, row_hi): only the row tiles of these rows are computed (multiples of B200MOE_TILE_M inside rows_cap;
 * 0, 0 = every row): the expert-parallel layer runs the rows of one group of experts while the rows of the next
 * group are still arriving.  No reference counterpart for the window. */
int b200moe_expert_gate_up_act(const void* x_s, const void* gate_up_proj, const int32_t* act_codes,
                               const int32_t* tile_expert, const int32_t* poffs, int64_t rows_cap, int64_t row_lo,
                               int64_t row_hi, int E, int64_t H, int64_t I, void* gate_up, void* inter,
                               int32_t* status, b200moe_stream_t stream);
/* Generic grouped products over the padded rows (the two entry points after them are special cases):
 * linear:   out (rows,N) = a (rows,K) * W[e]^T, W (E,N,K)   -- kernels/sm75/moe.py:765,770 (x @ W[e].t())
 * linear_t: out (rows,N) = a (rows,K) * W[e],   W (E,K,N)   -- kernels/sm75/moe.py:807,822 (g @ W[e]) */
int b200moe_expert_linear(const void* a, const void* w, const int32_t* tile_expert, const int32_t* poffs,
                          int64_t rows_cap, int E, int64_t N, int64_t K, void* out, int32_t* status,
                          b200moe_stream_t stream);
int b200moe_expert_linear_t(const void* a, const void* w, const int32_t* tile_expert, const int32_t* poffs,
                            int64_t rows_cap, int E, int64_t K, int64_t N, void* out, int32_t* status,
                            b200moe_stream_t stream);
/* Fused GEMM + dispatch over peer memory: out row r = a[r] * W[e(r)] as b200moe_expert_linear (w_kn = 0,
 * W (E,N,K)) or b200moe_expert_linear_t (w_kn = 1, W (E,K,N)) computes it, but the row is not stored locally:
 * the epilogue sends it to peer_base[row_rank[r]] + row_slot[r] * N elements with one bulk copy per 128-byte
 * piece, tile by tile while the GEMM runs (rows with row_rank < 0 are dropped).  peer_base is a DEVICE array of
 * W buffer addresses (this GPU's own among them); N % 64 == 0.  No reference counterpart. */
int b200moe_expert_linear_push(const void* a, const void* w, int w_kn, const int32_t* tile_expert, const int32_t* poffs,
                               int64_t rows_cap, int E, int64_t N, int64_t K, const int32_t* row_rank,
                               const int32_t* row_slot, const int64_t* peer_base, int32_t* status,
                               b200moe_stream_t stream);
/* Replaces the down GEMM (kernels/sm75/moe.py:592, :770): eo (rows,H) = inter * W_d[e]^T. */
int b200moe_expert_down(const void* inter, const void* down_proj, const int32_t* tile_expert,
                        const int32_t* poffs, int64_t rows_cap, int E, int64_t H, int64_t I,
                        void* eo, int32_t* status, b200moe_stream_t stream);
/* Replaces grad_inter = grad_eo @ W_d[e] + _glu_bwd (kernels/sm75/moe.py:609,611, :807,818):
 * grad_gate_up (rows,2I) = [grad_gate | grad_up] from grad_inter and the saved gate_up. */
int b200moe_expert_down_dgrad_glu(const void* grad_eo, const void* down_proj, const void* gate_up,
                                  const int32_t* tile_expert, const int32_t* poffs,
                                  int64_t rows_cap, int E, int64_t H, int64_t I, void* grad_gate_up,
                                  int32_t* status, b200moe_stream_t stream);
/* The same with per-expert activation codes (see b200moe_expert_gate_up_act): the backward of _glu_bwd
 * (kernels/sm75/moe.py:187-232) for codes 0, 1 and 5 without parameters, fused in the epilogue; row window as for
 * b200moe_expert_gate_up_act. */
int b200moe_expert_down_dgrad_act(const void* grad_eo, const void* down_proj, const void* gate_up,
                                  const int32_t* act_codes, const int32_t* tile_expert, const int32_t* poffs,
                                  int64_t rows_cap, int64_t row_lo, int64_t row_hi, int E, int64_t H, int64_t I,
                                  void* grad_gate_up, int32_t* status, b200moe_stream_t stream);
/* Replaces grad_x_s = grad_gate_up @ W_gu[e] (kernels/sm75/moe.py:612, :822). */
int b200moe_expert_gate_up_dgrad(const void* grad_gate_up, const void* gate_up_proj,
                                 const int32_t* tile_expert, const int32_t* poffs,
                                 int64_t rows_cap, int E, int64_t H, int64_t I, void* grad_x_s,
                                 int32_t* status, b200moe_stream_t stream);
/* Replaces _grouped_wgrad / ge.t() @ it (kernels/sm75/moe.py:556-561, :808, :821):
 * out[e] (Na,Nb) bf16 = A[rows of e]^T * B[rows of e]; experts with no rows get zeros.
 * counts (E, nullable): live rows per expert; when given, the all-zero pad blocks are skipped. */
int b200moe_expert_wgrad(const void* A, const void* B, const int32_t* poffs, const int32_t* counts,
                         int64_t rows_cap, int E, int64_t Na, int64_t Nb, void* out, int32_t* status,
                         b200moe_stream_t stream);

/* ---- PolyGLU activations as row kernels (expert stacks that are not pure SiLU-GLU) -------------
 * Replace _glu_fwd / _glu_bwd (kernels/sm75/moe.py:363-434, kernels :163-232).  act_codes (E_total)
 * int32: 0 SiLU, 1 ReLU^2, 2 NormSiLU, 5 SiTU, 6 NormReLU^2, 7 NormSiTU (3 Identity / 4 Zero are expert
 * kinds, see special_rows); act_params (E_total,2) fp32 [alpha,gamma] for code 5 or NULL.  Rows below
 * *total_rows are processed; the code of a row is that of its tile's expert. */
int b200moe_glu_fwd_rows(const void* gate_up, const int32_t* tile_expert, const int32_t* act_codes,
                         const float* act_params, const int32_t* total_rows, int64_t rows_cap, int64_t I,
                         void* inter, b200moe_stream_t stream);
/* grad_gate_up (rows,2I) from grad_inter (rows,I) and the saved gate_up; row_da/row_dg (rows, nullable):
 * per-row gradient of alpha / gamma for code-5 rows. */
int b200moe_glu_bwd_rows(const void* grad_inter, const void* gate_up, const int32_t* tile_expert,
                         const int32_t* act_codes, const float* act_params, const int32_t* total_rows,
                         int64_t rows_cap, int64_t I, void* grad_gate_up, float* row_da, float* row_dg,
                         b200moe_stream_t stream);
/* out (E,2) = per-expert sums of row_da, row_dg (grad of act_params, kernels/sm75/moe.py:814-815). */
int b200moe_expert_row_sums(const float* row_da, const float* row_dg, const int32_t* poffs, int E, float* out,
                            b200moe_stream_t stream);
/* Identity / Zero experts (kernels/sm75/moe.py:761-764, :798-803): for the rows of experts
 * [first_special, num_experts): dst[row] = src[row] if the expert's code is 3, else 0. */
int b200moe_special_rows(const void* src, const int32_t* tile_expert, const int32_t* act_codes,
                         const int32_t* poffs, int first_special, int num_experts, int64_t H, int64_t rows_cap,
                         void* dst, b200moe_stream_t stream);

/* ---- MXFP8 (e4m3 elements, E8M0 scale per 32 elements along K) ---------------------------------
 * The reference has no MXFP8 path; these follow the OCP MX convention: scale exponent =
 * floor(log2(amax)) - 8, elements rounded to nearest even and saturated at +-448.
 * Scales are stored as 512-byte atoms per (128 rows x 128 k): byte (row%32)*16 + ((row%128)/32)*4 +
 * (k/32)%4, atoms ordered row-block major, k-chunk minor; b200moe_mxfp8_sf_bytes gives the size. */
size_t b200moe_mxfp8_sf_bytes(int64_t rows, int64_t K);
/* x (R,C) bf16 -> q (R,C) e4m3 + scales, blocks along C.  interleave_I > 0: x is a stack of (2I,C)
 * gate|up matrices and output rows are re-ordered in groups of 64 gate rows then 64 up rows. */
int b200moe_mxfp8_quant_rows(const void* x, int64_t R, int64_t C, int64_t interleave_I, void* q, void* sf,
                             b200moe_stream_t stream);
/* x (G,R,C) bf16 -> q (G,C,R) e4m3 + scales, blocks along R (R % 32 == 0, C even). */
int b200moe_mxfp8_quant_transpose(const void* x, int64_t G, int64_t R, int64_t C, void* q, void* sf,
                                  b200moe_stream_t stream);
/* Both quantisations of x (G,R,C) in one pass over DRAM: q_rows/sf_rows as b200moe_mxfp8_quant_rows gives for
 * x seen as (G*R, C) (interleave_I as there, with R = 2I), q_t/sf_t as b200moe_mxfp8_quant_transpose gives.
 * R % 32 == 0, C % 32 == 0. */
int b200moe_mxfp8_quant_both(const void* x, int64_t G, int64_t R, int64_t C, int64_t interleave_I, void* q_rows,
                             void* sf_rows, void* q_t, void* sf_t, b200moe_stream_t stream);
/* D (M,N) bf16 = dequant(A)(M,K) * dequant(B)(N,K)^T on tcgen05 block-scaled MMAs; K % 128 == 0. */
int b200moe_mxfp8_gemm_nt(const void* Aq, const void* Asf, const void* Bq, const void* Bsf, void* D,
                          int64_t M, int64_t N, int64_t K, int32_t* status, b200moe_stream_t stream);
/* Grouped expert GEMM over padded rows; B is an (E*N, K) stack (N % 128 == 0).  epilogue: 0 = bf16
 * store, 1 = SwiGLU (N = 2I, weight rows 64-interleaved, D = gate_up, aux = inter), 2 = GLU backward
 * (N = I, aux = saved gate_up, D = grad_gate_up).  Same roles as the bf16 entry points above.
 * q_out / q_sf (nullable, epilogues 1 and 2): the epilogue also writes its bf16 result quantised along the
 * row -- inter as (rows, I) codes, grad_gate_up as (rows, 2I) codes -- i.e. the A operand of the next GEMM,
 * bit-identical to b200moe_mxfp8_quant_rows on that result. */
int b200moe_mxfp8_expert_gemm(int epilogue, const void* Aq, const void* Asf, const void* Bq,
                              const void* Bsf, const int32_t* tile_expert, const int32_t* poffs,
                              int64_t rows_cap, int E, int64_t N, int64_t K, int64_t I, void* D, void* aux,
                              void* q_out, void* q_sf, int32_t* status, b200moe_stream_t stream);
/* Gather fused with the row quantiser: x_s[r] = x[row_slot[r]/k] (bf16, zero pad rows) plus its codes and
 * scales (H % 32 == 0); replaces b200moe_gather_rows + b200moe_mxfp8_quant_rows. */
int b200moe_mxfp8_gather_quant(const void* x, const int32_t* row_slot, const int32_t* total_rows, int k, int64_t H,
                               int64_t rows_cap, void* x_s, void* q, void* sf, b200moe_stream_t stream);
/* The gather fused with both quantisers: what b200moe_mxfp8_gather_quant's codes/scales and
 * b200moe_mxfp8_quant_transpose of its x_s would be, without writing x_s (rows_cap % 32 == 0, H % 32 == 0;
 * q_t is (H, rows_cap)). */
int b200moe_mxfp8_gather_quant_both(const void* x, const int32_t* row_slot, const int32_t* total_rows, int k, int64_t H,
                                    int64_t rows_cap, void* q_rows, void* sf_rows, void* q_t, void* sf_t,
                                    b200moe_stream_t stream);
/* Weight gradient: out[e] (Na,Nb) bf16 = At[:, rows of e] * Bt[:, rows of e]^T, At (Na, rows_cap) and
 * Bt (Nb, rows_cap) quantised along the token rows (b200moe_mxfp8_quant_transpose). */
int b200moe_mxfp8_expert_wgrad(const void* Atq, const void* Atsf, const void* Btq, const void* Btsf,
                               const int32_t* poffs, const int32_t* counts, int64_t rows_cap, int E,
                               int64_t Na, int64_t Nb, void* out, int32_t* status, b200moe_stream_t stream);

/* ---- combine -------------------------------------------------------------------------------- */
/* Replaces _combine_scatter_kernel / index_add_ (kernels/sm75/moe.py:673-682, :593-595):
 * out[t] = sum_j w[t,j] * rows[slot_row[t*k+j]], fp32 accumulate in slot order, bf16 store.
 * w == NULL means weight 1 (the grad_hidden un-permute, kernels/sm75/moe.py:614-615). */
int b200moe_combine(const void* rows, const float* w, const int32_t* slot_row, int64_t T, int k,
                    int64_t H, void* out, b200moe_stream_t stream);
/* Replaces _combine_bwd_kernel (kernels/sm75/moe.py:688-701): grad_eo[r] = go[tok]*w[slot],
 * grad_w[slot] = <go[tok], eo[r]> in fp32; zero rows where row_slot[r] < 0. */
int b200moe_combine_bwd(const void* grad_out, const void* eo, const float* w,
                        const int32_t* row_slot, const int32_t* total_rows, int k, int64_t H,
                        int64_t rows_cap, void* grad_eo, float* grad_w, b200moe_stream_t stream);

/* ---- expert-parallel exchange over peer memory (no reference counterpart: the reference has no
 * expert parallelism) ------------------------------------------------------------------------------
 * `*_peers` arguments are HOST arrays of W device pointers, entry r = the same buffer on rank r
 * (a symmetric allocation mapped into this process).  Kernels only read peer memory and never wait on
 * a peer; the caller separates the phases with cross-rank barriers.  W <= 16, E % W == 0.
 * ep_plan: counts_all (W,E) -> this rank's padded segments poffs_l (E/W+1), counts_l (E/W) live rows,
 * tile_expert_l, src_base (W,E/W) first row of each source rank's block, dest_base (E) first row of
 * THIS rank's block of expert e inside e's owner.  rows_cap > 0 (with a status word): the caller's buffers hold
 * rows_cap padded rows and were sized without reading the row count back to the host; if ANY rank's padded rows
 * exceed it (every rank evaluates the same count matrix and decides alike) the status word gets 8 and the tables are
 * written so that the step computes nothing: empty segments, source blocks at a negative row (which the pull kernels
 * skip).  rows_cap = 0: no check. */
int b200moe_ep_plan(const int32_t* counts_all, int W, int rank, int E, int32_t* poffs_l, int32_t* counts_l,
                    int32_t* tile_expert_l, int32_t* src_base, int32_t* dest_base, int64_t rows_cap, int32_t* status,
                    b200moe_stream_t stream);
/* ep_local_rows: host_words[0] = the number of routed rows that arrive on this rank (sum over the sources of
 * counts_all (W,E) for the local experts); host_words[1 + j], j < E/W = the row at which local expert j ends in the
 * padded layout (poffs_l[j + 1] of b200moe_ep_plan).  `host_words`: 1 + E/W words of PINNED HOST memory
 * (cudaHostAlloc / cudaHostRegister; the call fails with B200MOE_E_CUDA and launches nothing otherwise).  The host
 * sizes its buffers, and splits the local experts into groups of about equal rows, after waiting for an event
 * recorded behind this call; no device-to-host copy is involved, so the read does not queue behind transfers that
 * occupy the copy engines.  No reference counterpart. */
int b200moe_ep_local_rows(const int32_t* counts_all, int W, int rank, int E, int32_t* host_words,
                          b200moe_stream_t stream);
/* ep_publish: this rank's routing tables -- idx (M) int64, slot_pos (M) int32, w (M) fp32 routing weights, offs
 * (E+1) int32 -- stored into slot `rank` of the replica arrays of EVERY rank (tab_*_peers[r] = base of rank r's
 * replica array, laid out [W][slot_stride] resp. [W][offs_stride] elements, both strides multiples of 4 so that
 * every replica starts 16-byte aligned; plain peer stores, the local rank included).  After the next
 * cross-rank ordering point every rank holds all W tables locally, and b200moe_ep_gather_pull /
 * b200moe_ep_combine_bwd_pull are given pointers into these replicas as their idx / slot_pos / offs / w tables, so
 * that only payload rows are read from peers.  No reference counterpart. */
int b200moe_ep_publish(const int64_t* idx, const int32_t* slot_pos, const float* w, const int32_t* offs, int64_t M, int E,
                       int W, int rank, int64_t slot_stride, int offs_stride, const void* const* tab_idx_peers, const void* const* tab_spos_peers,
                       const void* const* tab_w_peers, const void* const* tab_offs_peers, b200moe_stream_t stream);
/* Cross-rank barrier of the exchange (no reference counterpart).  flags_peers: HOST array of W device pointers,
 * entry r = rank r's flag array of W uint32 words (symmetric memory, zero before the first barrier).  The kernel
 * stores `generation` into word `rank` of every peer's array (release) and waits until all W words of its own
 * array have reached `generation` (acquire); the caller passes 1, 2, 3, ... on successive barriers, the same
 * sequence on every rank.  The wait gives up after `limit_cycles` SM clocks (1e3..4e10): `status` then receives 7
 * and the kernel returns normally -- a peer that never arrives costs a status code, not a hung GPU.  Writes
 * queued on `stream` before the barrier (peer stores included) are visible to every rank's kernels queued
 * after it. */
int b200moe_ep_barrier(const void* const* flags_peers, int W, int rank, uint32_t generation, int64_t limit_cycles,
                       int32_t* status, b200moe_stream_t stream);
/* owner side, forward.  For every source rank s and token t the kernel reads slot j of the token from the
 * source's routing tables (idx_peers int64 (T,k), spos_peers = slot_pos int32 (T,k), offs_peers int32 (E+1)) and,
 * for each expert that lives on this rank, writes x_peers[s][t] to row
 * src_base[s][e_local] + slot_pos - offs[e]; the token row is read from the peer ONCE however many of its
 * experts live here.  Pad rows are zeroed.  T is the token count of every rank.  row_rank / row_slot (nullable,
 * both or none): for every row the home rank and the slot t*k+j it came from (-1 / 0 for pad rows), i.e. where
 * b200moe_expert_linear_push sends that row's result.  [e_lo, e_hi): the local experts whose rows this launch fills
 * (0, E/W = all), so that the rows of one group of experts can arrive while the GEMMs of another group run;
 * max_sms > 0 limits the launch to that many SMs' worth of CTAs (a launch beside a persistent GEMM that leaves
 * them free, see b200moe_set_reserved_sms), 0 = all SMs. */
int b200moe_ep_gather_pull(const void* const* x_peers, const void* const* idx_peers, const void* const* spos_peers,
                           const void* const* offs_peers, const int32_t* counts_l, const int32_t* poffs_l,
                           const int32_t* src_base, int W, int rank, int E, int e_lo, int e_hi, int max_sms, int64_t T,
                           int k, int64_t H, void* x_s, int32_t* row_rank, int32_t* row_slot, b200moe_stream_t stream);
/* home side: out[t] = sum_j w[t,j] * rows_peers[owner][dest_base[e] + slot_pos[s] - offs[e]] (w NULL = 1),
 * summed in slot order; the rows arrive by bulk copies into a shared-memory ring (one CTA per SM, on at most
 * the SMs b200moe_set_exchange_sms allows).  When gw_peers / grad_w are given, grad_w[s] is fetched from the
 * owner's per-row dot products.  `status` (nullable) receives a wait code if a bounded wait gives up. */
int b200moe_ep_combine_pull(const void* const* rows_peers, const float* w, const int64_t* idx,
                            const int32_t* slot_pos, const int32_t* offs, const int32_t* dest_base, int W, int E,
                            int64_t T, int k, int64_t H, void* out, const void* const* gw_peers, float* grad_w,
                            int32_t* status, b200moe_stream_t stream);
/* owner side, backward, same traversal: grad_eo[row] = w_peers[s][t,j] * go_peers[s][t] (grad_out read once per
 * token and owner); gw_rows[row] = <go, eo[row]> (eo and gw_rows both NULL: no dot products); pad rows zero.
 * e_lo, e_hi, max_sms as for b200moe_ep_gather_pull. */
int b200moe_ep_combine_bwd_pull(const void* const* go_peers, const void* const* w_peers,
                                const void* const* idx_peers, const void* const* spos_peers,
                                const void* const* offs_peers, const void* eo, const int32_t* counts_l,
                                const int32_t* poffs_l, const int32_t* src_base, int W, int rank, int E, int e_lo,
                                int e_hi, int max_sms, int64_t T, int k, int64_t H, void* grad_eo, float* gw_rows,
                                b200moe_stream_t stream);

/* out[t*k+j] = <grad_out[t], rows[t*k+j]> (fp32): the gradient of the routing weights at the home rank when the
 * expert outputs of its tokens were pushed to it in slot order.  No reference counterpart as a kernel (the
 * reference computes this inside _combine_bwd_kernel, kernels/sm75/moe.py:688-701). */
int b200moe_slot_dots(const void* grad_out, const void* rows, int64_t T, int k, int64_t H, float* out,
                      b200moe_stream_t stream);

/* ---- Expert-stack optimizer step (Muon), the consumer of the layer's weight gradients.
 * Replaces the body of FusedMuon.step for stacks (E, r, c) of matrices (kernels/sm75/muon.py:366-434, the
 * capturable form :300-315) and newton_schulz (:62-89).  The three matrix products of each Newton-Schulz iteration
 * are b200moe_expert_linear / b200moe_expert_linear_t calls on a stack whose E row segments have `Rp` rows each
 * (a multiple of B200MOE_TILE_M, rows past the matrix are zero); these entry points are everything around them.
 * r and c are multiples of 8; bf16 unless stated. */

/* buf = mu*buf + g; u = nesterov ? g + mu*buf : buf (kernels/sm75/muon.py:389-390).  grad: n elements, fp32 if
 * grad_f32 else bf16, rounded to bf16 first as the reference's staging copy does (:386-388); mom (in/out), u: bf16. */
int b200moe_muon_momentum(const void* grad, int grad_f32, void* mom, void* u, int64_t n, float mu, int nesterov,
                          b200moe_stream_t stream);

/* rowss[row] = sum_j x[row,j]^2, fp32 accumulation (torch.linalg.vector_norm(..., dtype=float32),
 * kernels/sm75/muon.py:78, kernels/muon/muon_scaling.py:110). */
int b200moe_muon_row_sumsq(const void* x, int64_t rows, int64_t cols, float* rowss, b200moe_stream_t stream);

/* out[row,:] = bf16(x[row,:] * (tgt / max(sqrt(rowss[row]), eps))); rowss_out[row] = sum of squares of the rounded
 * row.  The row prescale of scale_mode "aurora" with K = 1, beta = 0 (kernels/muon/muon_scaling.py:107-111). */
int b200moe_muon_prescale_rows(const void* x, const float* rowss, int64_t rows, int64_t cols, float tgt, float eps,
                               void* out, float* rowss_out, b200moe_stream_t stream);
/* Row scaling with a given multiplier (the combined per-row multiplier of the reference's `aurora_ema` prescale,
 * kernels/muon/muon_scaling.py:141-142): out[row,:] = bf16(x[row,:] * mult[row]), rowss_out[row] = sum of squares of
 * the rounded row.  x, out (rows, cols) bf16; mult, rowss_out (rows) fp32. */
int b200moe_muon_scale_rows(const void* x, const float* mult, int64_t rows, int64_t cols, void* out, float* rowss_out,
                            b200moe_stream_t stream);
/* Weight update of the per-row scale modes (`normuon`, `aurora_ema_v2`: kernels/muon/muon_scaling.py:166-195 and the
 * scatter at kernels/sm75/muon.py:381,431-434): p[row,:] = decay * p[row,:] + alpha * bf16(x[row,:] * mult[row]);
 * x (rows, cols) bf16 in the parameters' own layout, p bf16 or fp32 (p_f32). */
int b200moe_muon_update_rows(const void* x, const float* mult, int64_t rows, int64_t cols, float decay, float alpha, void* p,
                             int p_f32, b200moe_stream_t stream);

/* Frobenius normalisation into the iteration's layout (kernels/sm75/muon.py:78-82): norms[e] =
 * bf16(max(sqrt(sum_i rowss[e*r+i]), eps)); transposed == 0: xp (E, Rp, c), xp[e,i,:] = x[e,i,:] / norms[e];
 * transposed != 0 (use it when r > c): xp (E, Rp, r), xp[e,j,i] = x[e,i,j] / norms[e].  Rows of xp past the matrix
 * are written as zeros.  norms: E floats of caller-owned scratch. */
int b200moe_muon_normalise_pack(const void* x, const float* rowss, int E, int64_t r, int64_t c, int64_t Rp,
                                int transposed, float eps, float* norms, void* xp, b200moe_stream_t stream);

/* Gram matrices of a stack: out[e] (R,R) = x[e] x[e]^T for E equal groups of R = rows_cap / E rows (R a multiple of
 * 256), x (rows_cap,K).  The result is symmetric, so only the tiles that reach the upper triangle of each group are
 * computed; with mirror != 0 the epilogue stores every chunk right of the diagonal tile a second time, transposed,
 * so the whole matrix is written, with mirror == 0 b200moe_mirror_upper completes it.  torch.bmm(X, X.transpose(1, 2)),
 * kernels/sm75/muon.py:84 (the reference's sm_120 fork has a symmetric-product kernel for the same purpose,
 * kernels/sm120/newton_schulz_symmul.py:50). */
int b200moe_expert_gram(const void* x, const int32_t* tile_expert, const int32_t* poffs, int64_t rows_cap, int E,
                        int64_t K, int mirror, void* out, int32_t* status, b200moe_stream_t stream);

/* a[e,i,j] = a[e,j,i] for every 64 x 64 block strictly below the block diagonal of E matrices of order n (a multiple
 * of 64), in place: the second half of a symmetric product.  No reference counterpart as a kernel. */
int b200moe_mirror_upper(void* a, int E, int64_t n, b200moe_stream_t stream);

/* out (rows,N) = bf16(alpha * (a (rows,K) @ W[e]^T) + beta * c + diag * I_e): b200moe_expert_linear with the
 * reference's baddbmm epilogue (kernels/sm75/muon.py:85: b*A + c*(A@A)) and an identity term on each group's own
 * diagonal (column == row - poffs[e]) folded into the GEMM's store.  c: (rows,N) bf16, read-only, must not alias out.
 * N a multiple of 256.  With a = c = the Gram matrices A, W = A, alpha = c, beta = b, diag = a it produces the whole
 * left factor (b A + c A A + a I) of one Newton-Schulz iteration.  symmetric != 0 (E equal groups of N rows, a
 * result known to be symmetric): only the tiles reaching the upper triangle are computed, as in b200moe_expert_gram;
 * symmetric == 2 also stores the transposed chunks from the epilogue (the whole matrix is written). */
int b200moe_expert_linear_axpby(const void* a, const void* w, const void* c, float alpha, float beta, float diag,
                                int symmetric, const int32_t* tile_expert, const int32_t* poffs, int64_t rows_cap, int E, int64_t N,
                                int64_t K, void* out, int32_t* status, b200moe_stream_t stream);

/* out = bf16(alpha*x + beta*y + diag*I), n elements seen as a stack of ld x ld matrices (ld = 0: no identity term);
 * out may alias x or y.  The axpy halves of the reference's baddbmm calls (kernels/sm75/muon.py:85-86): with
 * alpha = b, beta = c, diag = a it builds (b A + c A A) + a I, whose product with X is a X + (b A + c A A) X. */
int b200moe_axpby_bf16(const void* x, float alpha, const void* y, float beta, float diag, int64_t ld, void* out,
                       int64_t n, b200moe_stream_t stream);

/* p = round(round(p*decay) + alpha * bf16(gain*o)), o[e,i,j] = xp[e,i,j] (xp (E,Rp,c)) or xp[e,j,i] (transposed,
 * xp (E,Rp,r)); p (E,r,c) fp32 if p_f32 else bf16.  Decoupled weight decay + update (kernels/sm75/muon.py:381,
 * 431-434); gain is the aurora gain (kernels/muon/muon_scaling.py:112), 1 for scale_mode "polar". */
int b200moe_muon_apply(const void* xp, int E, int64_t r, int64_t c, int64_t Rp, int transposed, float gain, float decay,
                       float alpha, void* p, int p_f32, b200moe_stream_t stream);

#ifdef __cplusplus
}
#endif
#endif /* B200MOE_H_ */
