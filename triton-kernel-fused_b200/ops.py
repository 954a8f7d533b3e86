"""Thin Python callers of the C ABI, one per entry point; they allocate outputs with torch and
queue the kernels on the current CUDA stream.  No computation happens in Python."""
from __future__ import annotations

from dataclasses import dataclass

import torch

from . import _lib as L

LOGITS_BF16, LOGITS_F32, SCORES_F32 = 0, 1, 2
TILE_M = 256   # B200MOE_TILE_M: expert segments are padded to this many rows

# Optional observer used by the benchmark: hook(name, kernel_launches, start_event, end_event) is
# called for every op below with CUDA events recorded on the launching stream around it.
_hook = None


def set_hook(hook):
    global _hook
    _hook = hook


def _op(name, launches=1):
    def deco(fn):
        def wrapped(*a, **kw):
            if _hook is None:
                return fn(*a, **kw)
            e0 = torch.cuda.Event(enable_timing=True)
            e1 = torch.cuda.Event(enable_timing=True)
            e0.record()
            r = fn(*a, **kw)
            e1.record()
            _hook(name, launches, e0, e1)
            return r
        wrapped.__name__ = fn.__name__
        wrapped.__doc__ = fn.__doc__
        return wrapped
    return deco


def _kind(t: torch.Tensor, scores: bool) -> int:
    if scores:
        L.require(t.dtype == torch.float32, "scores must be float32")
        return SCORES_F32
    if t.dtype == torch.bfloat16:
        return LOGITS_BF16
    L.require(t.dtype == torch.float32, f"logits must be bfloat16 or float32, got {t.dtype}")
    return LOGITS_F32


@_op("router_topk_fwd", 1)
def router_topk_fwd(logits, bias, top_k, norm_topk=True, scale=1.0, want_counts=True, scores=False):
    """(N,E) logits (or fp32 scores) -> idx int64 (N,k), w fp32 (N,k), counts int32 (E,) or None."""
    L.require(logits.is_cuda and logits.dim() == 2 and logits.is_contiguous(), "logits must be a contiguous CUDA (N,E) tensor")
    N, E = logits.shape
    if bias is not None:
        L.require(bias.is_cuda and bias.dtype == torch.float32 and bias.numel() == E and bias.is_contiguous(),
                  "bias must be a contiguous float32 CUDA tensor of E elements")
    dev = logits.device
    idx = torch.empty(N, top_k, dtype=torch.int64, device=dev)
    w = torch.empty(N, top_k, dtype=torch.float32, device=dev)
    counts = torch.empty(E, dtype=torch.int32, device=dev) if want_counts else None
    L.check(L.lib().b200moe_router_topk_fwd(L.ptr(logits), _kind(logits, scores), L.ptr(bias), N, E, int(top_k),
                                            int(bool(norm_topk)), float(scale), L.ptr(idx), L.ptr(w),
                                            L.ptr(counts), L.stream_of(logits)))
    return idx, w, counts


@_op("router_topk_bwd", 1)
def router_topk_bwd(logits, idx, grad_w, norm_topk=True, scale=1.0):
    N, E = logits.shape
    k = idx.shape[1]
    gw = grad_w.contiguous().float()
    gl = torch.empty(N, E, dtype=torch.bfloat16, device=logits.device)
    L.check(L.lib().b200moe_router_topk_bwd(L.ptr(logits), _kind(logits, False), L.ptr(idx), L.ptr(gw), N, E, k,
                                            int(bool(norm_topk)), float(scale), L.ptr(gl), L.stream_of(logits)))
    return gl


@_op("router_bias_update", 1)
def router_bias_update(bias, counts, u):
    L.require(bias.is_cuda and bias.dtype == torch.float32 and bias.is_contiguous(), "bias must be contiguous float32 CUDA")
    L.require(counts.is_cuda and counts.dtype == torch.int32 and counts.is_contiguous(), "counts must be contiguous int32 CUDA")
    L.check(L.lib().b200moe_router_bias_update(L.ptr(bias), L.ptr(counts), bias.numel(), float(u), L.stream_of(bias)))


@_op("gemm_nt", 1)
def gemm_nt(a, b):
    """a (M,K) @ b (N,K)^T -> (M,N) bf16."""
    L.require_cuda_bf16("a", a); L.require_cuda_bf16("b", b)
    L.require(a.is_contiguous() and b.is_contiguous() and a.shape[1] == b.shape[1], "gemm_nt: need contiguous (M,K),(N,K)")
    M, K = a.shape
    N = b.shape[0]
    d = torch.empty(M, N, dtype=torch.bfloat16, device=a.device)
    L.check(L.lib().b200moe_gemm_nt(L.ptr(a), L.ptr(b), L.ptr(d), M, N, K, L.ptr(L.status_word(a.device)), L.stream_of(a)))
    return d


@_op("gemm_nn", 1)
def gemm_nn(a, b):
    """a (M,K) @ b (K,N) -> (M,N) bf16."""
    L.require_cuda_bf16("a", a); L.require_cuda_bf16("b", b)
    L.require(a.is_contiguous() and b.is_contiguous() and a.shape[1] == b.shape[0], "gemm_nn: need contiguous (M,K),(K,N)")
    M, K = a.shape
    N = b.shape[1]
    d = torch.empty(M, N, dtype=torch.bfloat16, device=a.device)
    L.check(L.lib().b200moe_gemm_nn(L.ptr(a), L.ptr(b), L.ptr(d), M, N, K, L.ptr(L.status_word(a.device)), L.stream_of(a)))
    return d


@_op("gemm_tn", 2)
def gemm_tn(a, b, target_ctas=296):
    """a (K,M)^T @ b (K,N) -> (M,N) bf16 through fp32 split-K slices."""
    L.require_cuda_bf16("a", a); L.require_cuda_bf16("b", b)
    L.require(a.is_contiguous() and b.is_contiguous() and a.shape[0] == b.shape[0], "gemm_tn: need contiguous (K,M),(K,N)")
    K, M = a.shape
    N = b.shape[1]
    tiles = ((M + 127) // 128) * ((N + 255) // 256)
    slices = max(1, min(target_ctas // max(tiles, 1), (K + 63) // 64))
    k_chunk = (((K + slices - 1) // slices) + 63) // 64 * 64
    slices = (K + k_chunk - 1) // k_chunk
    part = torch.empty(slices, M, N, dtype=torch.float32, device=a.device)
    d = torch.empty(M, N, dtype=torch.bfloat16, device=a.device)
    L.check(L.lib().b200moe_gemm_tn_splitk(L.ptr(a), L.ptr(b), L.ptr(part), M, N, K, k_chunk,
                                           L.ptr(L.status_word(a.device)), L.stream_of(a)))
    L.check(L.lib().b200moe_splitk_reduce(L.ptr(part), slices, M * N, L.ptr(d), L.stream_of(a)))
    return d


@dataclass
class Permutation:
    """Device tables of one routing decision (see include/b200moe.h, b200moe_permute_build)."""
    T: int
    k: int
    E: int
    cap: int                  # rows of every padded buffer
    counts: torch.Tensor      # (E,) int32
    offs: torch.Tensor        # (E+1,) int32 compact offsets
    poffs: torch.Tensor       # (E+1,) int32 padded offsets
    slot_row: torch.Tensor    # (T*k,) int32
    row_slot: torch.Tensor    # (cap,) int32, valid below poffs[E]
    tile_expert: torch.Tensor # (cap/TILE_M,) int32
    order: torch.Tensor | None      # (T*k,) int32 compact row -> slot (stable argsort of idx.flatten())
    slot_pos: torch.Tensor | None   # (T*k,) int32 slot -> compact row

    @property
    def total_rows(self):     # device scalar view
        return self.poffs[self.E:]


@_op("permute_build", 3)
def permute_build(idx, E, want_order=False) -> Permutation:
    L.require(idx.is_cuda and idx.dtype == torch.int64 and idx.dim() == 2, "top_k_indices must be a CUDA int64 (N,k) tensor")
    idx = idx.contiguous()
    T, k = idx.shape
    dev = idx.device
    M = T * k
    cap = L.padded_rows_cap(M, E)
    i32 = dict(dtype=torch.int32, device=dev)
    counts = torch.empty(E, **i32)
    offs = torch.empty(E + 1, **i32)
    poffs = torch.empty(E + 1, **i32)
    slot_row = torch.empty(M, **i32)
    row_slot = torch.empty(cap, **i32)
    tile_expert = torch.empty(cap // TILE_M, **i32)
    order = torch.empty(M, **i32) if want_order else None
    slot_pos = torch.empty(M, **i32) if want_order else None
    ws_bytes = int(L.lib().b200moe_permute_ws_bytes(M, E))
    ws = torch.empty(max(ws_bytes, 4), dtype=torch.uint8, device=dev)
    L.check(L.lib().b200moe_permute_build(L.ptr(idx), T, k, E, L.ptr(counts), L.ptr(offs), L.ptr(poffs),
                                          L.ptr(slot_row), L.ptr(row_slot), L.ptr(tile_expert), L.ptr(order),
                                          L.ptr(slot_pos), L.ptr(ws), ws_bytes, L.ptr(L.status_word(dev)), L.stream_of(idx)))
    return Permutation(T, k, E, cap, counts, offs, poffs, slot_row, row_slot, tile_expert, order, slot_pos)


@_op("gather_rows", 1)
def gather_rows_raw(x, row_slot, total_rows, k, rows_cap):
    """out[r] = x[row_slot[r] // k] for r < *total_rows (device scalar), zero rows where row_slot < 0."""
    L.require_cuda_bf16("x", x)
    H = x.shape[1]
    out = torch.empty(max(rows_cap, 1), H, dtype=torch.bfloat16, device=x.device)
    L.check(L.lib().b200moe_gather_rows(L.ptr(x), L.ptr(row_slot), L.ptr(total_rows), k, H, rows_cap,
                                        L.ptr(out), L.stream_of(x)))
    return out


def gather_rows(x, perm: Permutation):
    """Rows of x in the padded expert-contiguous layout of `perm`."""
    return gather_rows_raw(x, perm.row_slot, perm.total_rows, perm.k, perm.cap)


def gather_compact(x, perm: Permutation):
    """Rows of x in the compact expert-sorted order of `perm` (needs want_order=True)."""
    return gather_rows_raw(x, perm.order, perm.offs[perm.E:], perm.k, perm.T * perm.k)


@_op("expert_gate_up_swiglu", 1)
def expert_gate_up_swiglu(x_s, gate_up_proj, perm: Permutation, act_codes=None, out=None, rows=(0, 0)):
    """act_codes: (E,) int32 device tensor of per-expert codes 0 / 1 / 5 applied in the epilogue (None = all SiLU).
    out: (gate_up, inter) buffers of perm.cap rows to write into; rows = (lo, hi): only these rows (tile-aligned)."""
    E, twoI, H = gate_up_proj.shape
    I = twoI // 2
    if out is None:
        gate_up = torch.empty(perm.cap, twoI, dtype=torch.bfloat16, device=x_s.device)
        inter = torch.empty(perm.cap, I, dtype=torch.bfloat16, device=x_s.device)
    else:
        gate_up, inter = out
    L.check(L.lib().b200moe_expert_gate_up_act(L.ptr(x_s), L.ptr(gate_up_proj), L.ptr(act_codes), L.ptr(perm.tile_expert),
                                               L.ptr(perm.poffs), perm.cap, rows[0], rows[1], E, H, I, L.ptr(gate_up),
                                               L.ptr(inter),
                                               L.ptr(L.status_word(x_s.device)), L.stream_of(x_s)))
    return gate_up, inter


@_op("expert_down", 1)
def expert_down(inter, down_proj, perm: Permutation, out=None):
    E, H, I = down_proj.shape
    eo = torch.empty(perm.cap, H, dtype=torch.bfloat16, device=inter.device) if out is None else out
    L.check(L.lib().b200moe_expert_down(L.ptr(inter), L.ptr(down_proj), L.ptr(perm.tile_expert), L.ptr(perm.poffs),
                                        perm.cap, E, H, I, L.ptr(eo), L.ptr(L.status_word(inter.device)),
                                        L.stream_of(inter)))
    return eo


@_op("expert_down_dgrad_glu", 1)
def expert_down_dgrad_glu(grad_eo, down_proj, gate_up, perm: Permutation, act_codes=None, out=None, rows=(0, 0)):
    E, H, I = down_proj.shape
    ggu = torch.empty(perm.cap, 2 * I, dtype=torch.bfloat16, device=grad_eo.device) if out is None else out
    L.check(L.lib().b200moe_expert_down_dgrad_act(L.ptr(grad_eo), L.ptr(down_proj), L.ptr(gate_up), L.ptr(act_codes),
                                                  L.ptr(perm.tile_expert), L.ptr(perm.poffs), perm.cap, rows[0], rows[1],
                                                  E, H, I,
                                                  L.ptr(ggu), L.ptr(L.status_word(grad_eo.device)),
                                                  L.stream_of(grad_eo)))
    return ggu


@_op("expert_gate_up_dgrad", 1)
def expert_gate_up_dgrad(grad_gate_up, gate_up_proj, perm: Permutation, out=None):
    E, twoI, H = gate_up_proj.shape
    gx = torch.empty(perm.cap, H, dtype=torch.bfloat16, device=grad_gate_up.device) if out is None else out
    L.check(L.lib().b200moe_expert_gate_up_dgrad(L.ptr(grad_gate_up), L.ptr(gate_up_proj), L.ptr(perm.tile_expert),
                                                 L.ptr(perm.poffs), perm.cap, E, H, twoI // 2, L.ptr(gx),
                                                 L.ptr(L.status_word(gx.device)), L.stream_of(gx)))
    return gx


@_op("expert_wgrad", 1)
def expert_wgrad(a, b, perm: Permutation):
    """out[e] (Na,Nb) = a[rows of e]^T @ b[rows of e]; zero for experts without rows."""
    Na, Nb = a.shape[1], b.shape[1]
    out = torch.empty(perm.E, Na, Nb, dtype=torch.bfloat16, device=a.device)
    L.check(L.lib().b200moe_expert_wgrad(L.ptr(a), L.ptr(b), L.ptr(perm.poffs), L.ptr(perm.counts), perm.cap, perm.E, Na, Nb,
                                         L.ptr(out),
                                         L.ptr(L.status_word(a.device)), L.stream_of(a)))
    return out


@_op("combine", 1)
def combine_raw(rows, w, slot_table, T, k):
    """out[t] = sum_j w[t,j] * rows[slot_table[t*k+j]] (w None = 1), fp32 accumulate, bf16 out."""
    H = rows.shape[1]
    out = torch.empty(max(T, 1), H, dtype=torch.bfloat16, device=rows.device)[:T]
    L.check(L.lib().b200moe_combine(L.ptr(rows), L.ptr(w), L.ptr(slot_table), T, k, H, L.ptr(out),
                                    L.stream_of(rows)))
    return out


def combine(rows, w, perm: Permutation):
    return combine_raw(rows, w, perm.slot_row, perm.T, perm.k)


@_op("combine_bwd", 1)
def combine_bwd_raw(grad_out, eo, w, row_slot, total_rows, k, rows_cap):
    H = eo.shape[1]
    grad_eo = torch.empty_like(eo)
    grad_w = torch.empty(w.shape, dtype=torch.float32, device=eo.device)
    L.check(L.lib().b200moe_combine_bwd(L.ptr(grad_out), L.ptr(eo), L.ptr(w), L.ptr(row_slot), L.ptr(total_rows), k,
                                        H, rows_cap, L.ptr(grad_eo), L.ptr(grad_w), L.stream_of(eo)))
    return grad_eo, grad_w


def combine_bwd(grad_out, eo, w, perm: Permutation):
    return combine_bwd_raw(grad_out, eo, w, perm.row_slot, perm.total_rows, perm.k, perm.cap)


# ----------------------------------------------------------------------------- MXFP8
EPI_STORE, EPI_SWIGLU, EPI_GLU_BWD = 0, 1, 2


def _sf_empty(rows, K, device):
    return torch.empty(int(L.lib().b200moe_mxfp8_sf_bytes(rows, K)), dtype=torch.uint8, device=device)


@_op("mxfp8_quant_rows", 1)
def mxfp8_quant_rows(x, interleave_I=0):
    """x (R,C) bf16 -> (q uint8 (R,C) e4m3 codes, scale atoms), one E8M0 scale per 32 elements along C."""
    L.require_cuda_bf16("x", x)
    L.require(x.dim() == 2 and x.is_contiguous(), "mxfp8_quant_rows: need a contiguous (R,C) tensor")
    R, C = x.shape
    q = torch.empty(R, C, dtype=torch.uint8, device=x.device)
    sf = _sf_empty(R, C, x.device)
    L.check(L.lib().b200moe_mxfp8_quant_rows(L.ptr(x), R, C, int(interleave_I), L.ptr(q), L.ptr(sf), L.stream_of(x)))
    return q, sf


@_op("mxfp8_quant_transpose", 1)
def mxfp8_quant_transpose(x):
    """x (G,R,C) or (R,C) bf16 -> (q uint8 (G,C,R) / (C,R), scale atoms), scales along R."""
    L.require_cuda_bf16("x", x)
    x3 = x if x.dim() == 3 else x.unsqueeze(0)
    L.require(x3.is_contiguous(), "mxfp8_quant_transpose: need a contiguous tensor")
    G, R, C = x3.shape
    q = torch.empty(G, C, R, dtype=torch.uint8, device=x.device)
    sf = _sf_empty(G * C, R, x.device)
    L.check(L.lib().b200moe_mxfp8_quant_transpose(L.ptr(x3), G, R, C, L.ptr(q), L.ptr(sf), L.stream_of(x)))
    return (q if x.dim() == 3 else q[0]), sf


@_op("mxfp8_quant_both", 1)
def mxfp8_quant_both(x, interleave_I=0):
    """x (G,R,C) or (R,C) bf16 -> (q_rows (G*R,C), sf_rows, q_t (G,C,R) / (C,R), sf_t): the results of
    `mxfp8_quant_rows` and `mxfp8_quant_transpose` from one pass over x."""
    L.require_cuda_bf16("x", x)
    x3 = x if x.dim() == 3 else x.unsqueeze(0)
    L.require(x3.is_contiguous(), "mxfp8_quant_both: need a contiguous tensor")
    G, R, C = x3.shape
    q = torch.empty(G * R, C, dtype=torch.uint8, device=x.device)
    sf = _sf_empty(G * R, C, x.device)
    qt = torch.empty(G, C, R, dtype=torch.uint8, device=x.device)
    sft = _sf_empty(G * C, R, x.device)
    L.check(L.lib().b200moe_mxfp8_quant_both(L.ptr(x3), G, R, C, int(interleave_I), L.ptr(q), L.ptr(sf), L.ptr(qt),
                                             L.ptr(sft), L.stream_of(x)))
    return q, sf, (qt if x.dim() == 3 else qt[0]), sft


@_op("mxfp8_gemm_nt", 1)
def mxfp8_gemm_nt(aq, asf, bq, bsf):
    """dequant(aq)(M,K) @ dequant(bq)(N,K)^T -> (M,N) bf16."""
    M, K = aq.shape
    N = bq.shape[0]
    d = torch.empty(M, N, dtype=torch.bfloat16, device=aq.device)
    L.check(L.lib().b200moe_mxfp8_gemm_nt(L.ptr(aq), L.ptr(asf), L.ptr(bq), L.ptr(bsf), L.ptr(d), M, N, K,
                                          L.ptr(L.status_word(aq.device)), L.stream_of(aq)))
    return d


@_op("mxfp8_expert_gemm", 1)
def mxfp8_expert_gemm(epilogue, aq, asf, bq, bsf, perm: Permutation, N, K, I, d, aux=None, quantise_result=False):
    """quantise_result (SwiGLU / GLU-backward epilogues): also return (codes, scale atoms) of the result
    quantised along its rows, produced inside the epilogue."""
    q = qsf = None
    if quantise_result:
        width = I if epilogue == EPI_SWIGLU else 2 * I
        q = torch.empty(perm.cap, width, dtype=torch.uint8, device=d.device)
        qsf = _sf_empty(perm.cap, width, d.device)
    L.check(L.lib().b200moe_mxfp8_expert_gemm(int(epilogue), L.ptr(aq), L.ptr(asf), L.ptr(bq), L.ptr(bsf),
                                              L.ptr(perm.tile_expert), L.ptr(perm.poffs), perm.cap, perm.E, N, K, I,
                                              L.ptr(d), L.ptr(aux), L.ptr(q), L.ptr(qsf),
                                              L.ptr(L.status_word(d.device)), L.stream_of(d)))
    return (d, q, qsf) if quantise_result else d


@_op("mxfp8_gather_quant_both", 1)
def mxfp8_gather_quant_both(x, perm: Permutation):
    """Codes + scales of the gathered rows x[row_slot/k] quantised along H (rows, H) and along the rows (H, rows),
    pad rows as zeros; the gathered bf16 matrix is not materialised."""
    L.require_cuda_bf16("x", x)
    H = x.shape[1]
    q = torch.empty(perm.cap, H, dtype=torch.uint8, device=x.device)
    sf = _sf_empty(perm.cap, H, x.device)
    qt = torch.empty(H, perm.cap, dtype=torch.uint8, device=x.device)
    sft = _sf_empty(H, perm.cap, x.device)
    L.check(L.lib().b200moe_mxfp8_gather_quant_both(L.ptr(x), L.ptr(perm.row_slot), L.ptr(perm.total_rows), perm.k, H,
                                                    perm.cap, L.ptr(q), L.ptr(sf), L.ptr(qt), L.ptr(sft), L.stream_of(x)))
    return q, sf, qt, sft


@_op("mxfp8_gather_quant", 1)
def mxfp8_gather_quant(x, perm: Permutation):
    """Gather into the padded layout and quantise along the rows in one pass: (x_s bf16, codes, scale atoms)."""
    L.require_cuda_bf16("hidden", x)
    H = x.shape[1]
    x_s = torch.empty(perm.cap, H, dtype=torch.bfloat16, device=x.device)
    q = torch.empty(perm.cap, H, dtype=torch.uint8, device=x.device)
    sf = _sf_empty(perm.cap, H, x.device)
    L.check(L.lib().b200moe_mxfp8_gather_quant(L.ptr(x), L.ptr(perm.row_slot), L.ptr(perm.total_rows), perm.k, H,
                                               perm.cap, L.ptr(x_s), L.ptr(q), L.ptr(sf), L.stream_of(x)))
    return x_s, q, sf


@_op("mxfp8_expert_wgrad", 1)
def mxfp8_expert_wgrad(atq, atsf, btq, btsf, perm: Permutation):
    """out[e] (Na,Nb) = At[:, rows of e] @ Bt[:, rows of e]^T from transposed-quantised operands."""
    Na, Nb = atq.shape[0], btq.shape[0]
    out = torch.empty(perm.E, Na, Nb, dtype=torch.bfloat16, device=atq.device)
    L.check(L.lib().b200moe_mxfp8_expert_wgrad(L.ptr(atq), L.ptr(atsf), L.ptr(btq), L.ptr(btsf), L.ptr(perm.poffs),
                                               L.ptr(perm.counts), perm.cap, perm.E, Na, Nb, L.ptr(out),
                                               L.ptr(L.status_word(out.device)), L.stream_of(out)))
    return out


# ----------------------------------------------------------------------------- PolyGLU (generic path)
@_op("expert_linear", 1)
def expert_linear(a, w, perm: Permutation, out=None):
    """out (rows,N) = a (rows,K) @ W[e]^T with W (E,N,K), E = perm.E."""
    E, N, K = w.shape
    out = torch.empty(perm.cap, N, dtype=torch.bfloat16, device=a.device) if out is None else out
    L.check(L.lib().b200moe_expert_linear(L.ptr(a), L.ptr(w), L.ptr(perm.tile_expert), L.ptr(perm.poffs), perm.cap,
                                          perm.E, N, K, L.ptr(out), L.ptr(L.status_word(a.device)), L.stream_of(a)))
    return out


@_op("expert_linear_axpby", 1)
def expert_linear_axpby(a, w, c, alpha, beta, diag, perm: Permutation, out, symmetric=0):
    """out (rows,N) = alpha * (a (rows,K) @ W[e]^T) + beta * c + diag on each group's own diagonal; W (E,N,K).
    symmetric: 1 = the result is known to be symmetric per group and only its upper tiles are computed and written
    (mirror_upper completes it), 2 = the epilogue also writes the transposed chunks (complete result)."""
    E, N, K = w.shape
    L.check(L.lib().b200moe_expert_linear_axpby(L.ptr(a), L.ptr(w), L.ptr(c), float(alpha), float(beta), float(diag),
                                                int(symmetric), L.ptr(perm.tile_expert), L.ptr(perm.poffs),
                                                perm.cap, perm.E, N, K, L.ptr(out), L.ptr(L.status_word(a.device)),
                                                L.stream_of(a)))
    return out


@_op("expert_gram", 1)
def expert_gram(x, perm: Permutation, out, mirror=True):
    """out[e] = x[e] x[e]^T for equal groups of rows, computed over the tiles that reach the upper triangle; the
    epilogue writes the transposed chunks too (mirror=False: only the computed tiles are written)."""
    K = x.shape[-1]
    L.check(L.lib().b200moe_expert_gram(L.ptr(x), L.ptr(perm.tile_expert), L.ptr(perm.poffs), perm.cap, perm.E, K,
                                        1 if mirror else 0, L.ptr(out), L.ptr(L.status_word(x.device)), L.stream_of(x)))
    return out


@_op("mirror_upper", 1)
def mirror_upper(a, E, n):
    """In place a[e,i,j] = a[e,j,i] below the 64-block diagonal of E matrices of order n."""
    L.check(L.lib().b200moe_mirror_upper(L.ptr(a), E, n, L.stream_of(a)))
    return a


@_op("expert_linear_push", 1)
def expert_linear_push(a, w, perm: Permutation, row_rank, row_slot, peer_base, w_kn=False):
    """Row r of a (rows,K) @ W[e(r)]^T (W (E,N,K); w_kn: a @ W[e(r)], W (E,K,N)) is sent to
    peer_base[row_rank[r]] + row_slot[r] * N elements instead of being stored; rows with row_rank < 0 are dropped.
    peer_base: int64 device tensor of buffer addresses."""
    E = w.shape[0]
    K, N = (w.shape[1], w.shape[2]) if w_kn else (w.shape[2], w.shape[1])
    L.check(L.lib().b200moe_expert_linear_push(L.ptr(a), L.ptr(w), 1 if w_kn else 0, L.ptr(perm.tile_expert),
                                               L.ptr(perm.poffs), perm.cap, E, N, K, L.ptr(row_rank), L.ptr(row_slot),
                                               L.ptr(peer_base), L.ptr(L.status_word(a.device)), L.stream_of(a)))


@_op("expert_linear_t", 1)
def expert_linear_t(a, w, perm: Permutation, out=None):
    """out (rows,N) = a (rows,K) @ W[e] with W (E,K,N), E = perm.E."""
    E, K, N = w.shape
    out = torch.empty(perm.cap, N, dtype=torch.bfloat16, device=a.device) if out is None else out
    L.check(L.lib().b200moe_expert_linear_t(L.ptr(a), L.ptr(w), L.ptr(perm.tile_expert), L.ptr(perm.poffs), perm.cap,
                                            perm.E, K, N, L.ptr(out), L.ptr(L.status_word(a.device)), L.stream_of(a)))
    return out


@_op("glu_fwd_rows", 1)
def glu_fwd_rows(gate_up, act_codes, act_params, perm: Permutation):
    I = gate_up.shape[1] // 2
    inter = torch.empty(perm.cap, I, dtype=torch.bfloat16, device=gate_up.device)
    L.check(L.lib().b200moe_glu_fwd_rows(L.ptr(gate_up), L.ptr(perm.tile_expert), L.ptr(act_codes), L.ptr(act_params),
                                         L.ptr(perm.total_rows), perm.cap, I, L.ptr(inter), L.stream_of(gate_up)))
    return inter


@_op("glu_bwd_rows", 1)
def glu_bwd_rows(grad_inter, gate_up, act_codes, act_params, perm: Permutation, want_param_grads=False):
    I = gate_up.shape[1] // 2
    dev = gate_up.device
    ggu = torch.empty_like(gate_up)
    row_da = torch.empty(perm.cap, dtype=torch.float32, device=dev) if want_param_grads else None
    row_dg = torch.empty(perm.cap, dtype=torch.float32, device=dev) if want_param_grads else None
    L.check(L.lib().b200moe_glu_bwd_rows(L.ptr(grad_inter), L.ptr(gate_up), L.ptr(perm.tile_expert), L.ptr(act_codes),
                                         L.ptr(act_params), L.ptr(perm.total_rows), perm.cap, I, L.ptr(ggu),
                                         L.ptr(row_da), L.ptr(row_dg), L.stream_of(gate_up)))
    return ggu, row_da, row_dg


@_op("expert_row_sums", 1)
def expert_row_sums(row_da, row_dg, perm: Permutation, out):
    """out[:perm.E] (E,2) = per-expert sums of the per-row alpha / gamma gradients."""
    L.check(L.lib().b200moe_expert_row_sums(L.ptr(row_da), L.ptr(row_dg), L.ptr(perm.poffs), perm.E, L.ptr(out),
                                            L.stream_of(out)))
    return out


@_op("special_rows", 1)
def special_rows(src, dst, act_codes, perm: Permutation, first_special):
    """Rows of the Identity / Zero experts [first_special, perm.E): dst = src or 0."""
    H = src.shape[1]
    L.check(L.lib().b200moe_special_rows(L.ptr(src), L.ptr(perm.tile_expert), L.ptr(act_codes), L.ptr(perm.poffs),
                                         int(first_special), perm.E, H, perm.cap, L.ptr(dst), L.stream_of(src)))
    return dst


# ----------------------------------------------------------------------------- conv router front end
@_op("conv_unfold", 1)
def conv_unfold(x, K):
    """x (B,S,H) bf16 -> (B*S, K*H): row (b,s) holds x[b, s-(K-1) .. s] (zeros before the sequence start)."""
    L.require_cuda_bf16("x", x)
    B, S, H = x.shape
    xu = torch.empty(B * S, K * H, dtype=torch.bfloat16, device=x.device)
    L.check(L.lib().b200moe_conv_unfold(L.ptr(x), B, S, H, int(K), L.ptr(xu), L.stream_of(x)))
    return xu


@_op("conv_fold", 1)
def conv_fold(grad_xu, B, S, H, K):
    gx = torch.empty(B, S, H, dtype=torch.bfloat16, device=grad_xu.device)
    L.check(L.lib().b200moe_conv_fold(L.ptr(grad_xu), B, S, H, int(K), L.ptr(gx), L.stream_of(grad_xu)))
    return gx


def conv_direct_ok(S, H):
    """Shapes the no-copy convolution GEMMs take (forward and weight gradient): row tiles inside one sequence,
    64-channel k-blocks inside one tap."""
    return S % 128 == 0 and H % 64 == 0


@_op("conv_gemm_fwd", 1)
def conv_gemm_fwd(x, wf, K):
    """logits (B*S, E) of the causal K-tap convolution of x (B,S,H) with Wf (E, K*H), x read in place."""
    L.require_cuda_bf16("x", x); L.require_cuda_bf16("wf", wf)
    B, S, H = x.shape
    E = wf.shape[0]
    logits = torch.empty(B * S, E, dtype=torch.bfloat16, device=x.device)
    L.check(L.lib().b200moe_conv_gemm_fwd(L.ptr(x), L.ptr(wf), L.ptr(logits), B, S, H, E, int(K),
                                          L.ptr(L.status_word(x.device)), L.stream_of(x)))
    return logits


@_op("conv_gemm_dx", 1)
def conv_gemm_dx(grad_logits, wb, B, S, K):
    """grad_x (B,S,H) from grad_logits (B*S, E) and Wb (K*E, H), Wb[j*E+e, h] = W[e,h,j]."""
    E, H = grad_logits.shape[1], wb.shape[1]
    gx = torch.empty(B, S, H, dtype=torch.bfloat16, device=grad_logits.device)
    L.check(L.lib().b200moe_conv_gemm_dx(L.ptr(grad_logits), L.ptr(wb), L.ptr(gx), B, S, H, E, int(K),
                                         L.ptr(L.status_word(gx.device)), L.stream_of(gx)))
    return gx


@_op("conv_gemm_dw", 2)
def conv_gemm_dw(grad_logits, x, K, target_ctas=296):
    """grad_Wf (E, K*H) = grad_logits (B*S, E)^T @ unfold(x), through fp32 split-K slices, x read in place."""
    B, S, H = x.shape
    E = grad_logits.shape[1]
    rows, N = B * S, K * H
    bn = 256 if H % 256 == 0 else (128 if H % 128 == 0 else 64)
    tiles = ((E + 127) // 128) * (N // bn)
    slices = max(1, min(target_ctas // max(tiles, 1), (rows + 63) // 64))
    k_chunk = (((rows + slices - 1) // slices) + 63) // 64 * 64
    slices = (rows + k_chunk - 1) // k_chunk
    part = torch.empty(slices, E, N, dtype=torch.float32, device=x.device)
    d = torch.empty(E, N, dtype=torch.bfloat16, device=x.device)
    L.check(L.lib().b200moe_conv_gemm_dw_splitk(L.ptr(grad_logits), L.ptr(x), L.ptr(part), B, S, H, E, int(K), k_chunk,
                                                L.ptr(L.status_word(x.device)), L.stream_of(x)))
    L.check(L.lib().b200moe_splitk_reduce(L.ptr(part), slices, E * N, L.ptr(d), L.stream_of(x)))
    return d
