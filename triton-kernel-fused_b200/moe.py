"""Expert pipeline of the MoE block behind the reference's callables.

Mirrors kernels/sm75/moe.py: `moe` (:838), `moe_grouped` (:621), `moe_per_expert` (:829) keep their
signatures and return the (N,H) combined output; all three run the one sm_100a path
(device-side counting sort -> gather -> grouped tcgen05 GEMMs with fused SwiGLU -> weighted
gather-combine), with a hand-written backward (dgrad + wgrad grouped GEMMs, fused GLU backward).
"""
from __future__ import annotations

import torch

from . import _lib as L
from . import ops

__all__ = ["moe", "moe_grouped", "moe_per_expert", "GROUPED_MIN_TOKENS"]

GROUPED_MIN_TOKENS = 4096   # kept for API compatibility (kernels/sm75/moe.py:78); one path here


def _amp_cast(*ts):
    """Under CUDA autocast cast float tensors to the autocast dtype (kernels/sm75/moe.py:97-104)."""
    if torch.is_autocast_enabled("cuda"):
        dt = torch.get_autocast_dtype("cuda")
        return tuple(t.to(dt) if t.is_floating_point() else t for t in ts)
    return ts


class _GroupedMoE(torch.autograd.Function):
    """Forward saves x_s, gate_up, inter, eo and the permutation tables, as the reference's grouped
    Function does (kernels/sm75/moe.py:576-599); backward follows :602-618."""

    @staticmethod
    def forward(ctx, hidden, idx, wt, gate_up_proj, down_proj, act_codes):
        hidden, gate_up_proj, down_proj = _amp_cast(hidden, gate_up_proj, down_proj)
        L.require(hidden.dim() == 2, "hidden must be (N,H)")
        for name, t in (("hidden", hidden), ("gate_up_proj", gate_up_proj), ("down_proj", down_proj)):
            L.require_cuda_bf16(name, t)
        N, H = hidden.shape
        E, twoI, H2 = gate_up_proj.shape
        I = twoI // 2
        L.require(H2 == H and tuple(down_proj.shape) == (E, H, I) and twoI == 2 * I,
                  f"weight shapes must be (E,2I,H) and (E,H,I); got {tuple(gate_up_proj.shape)}, {tuple(down_proj.shape)}")
        L.require(act_codes.numel() == E, "act_codes must have one code per expert")
        L.require(tuple(idx.shape) == tuple(wt.shape) and idx.shape[0] == N, "indices/weights must be (N,k)")
        hidden = hidden.contiguous()
        gate_up_proj = gate_up_proj.contiguous()
        down_proj = down_proj.contiguous()
        w32 = wt.detach().float().contiguous()

        # a stack that mixes the parameter-free codes 0 / 1 / 5 keeps the fused epilogues: the code of a tile's
        # expert picks the activation there; an all-SiLU stack runs the SiLU-only instantiations
        codes, _ = _code_info(act_codes)
        codes_dev = None
        if any(c != 0 for c in codes):
            codes_dev = act_codes.to(device=hidden.device, dtype=torch.int32).contiguous()

        perm = ops.permute_build(idx, E)
        x_s = ops.gather_rows(hidden, perm)
        gate_up, inter = ops.expert_gate_up_swiglu(x_s, gate_up_proj, perm, codes_dev)
        eo = ops.expert_down(inter, down_proj, perm)
        out = ops.combine(eo, w32, perm)

        ctx.perm = perm
        ctx.wt_dtype = wt.dtype
        ctx.codes_dev = codes_dev
        ctx.save_for_backward(x_s, gate_up, inter, eo, w32, gate_up_proj, down_proj)
        return out

    @staticmethod
    def backward(ctx, grad_out):
        x_s, gate_up, inter, eo, w32, gate_up_proj, down_proj = ctx.saved_tensors
        perm = ctx.perm
        need_x, _, need_w, need_gu, need_dn, _ = ctx.needs_input_grad
        grad_out = grad_out.contiguous()
        if grad_out.dtype != torch.bfloat16:
            grad_out = grad_out.to(torch.bfloat16)
        grad_eo, grad_w = ops.combine_bwd(grad_out, eo, w32, perm)
        grad_hidden = grad_gate_up_proj = grad_down_proj = None
        if need_x or need_gu:
            grad_gu = ops.expert_down_dgrad_glu(grad_eo, down_proj, gate_up, perm, ctx.codes_dev)
            if need_gu:
                grad_gate_up_proj = ops.expert_wgrad(grad_gu, x_s, perm)
            if need_x:
                grad_x_s = ops.expert_gate_up_dgrad(grad_gu, gate_up_proj, perm)
                grad_hidden = ops.combine(grad_x_s, None, perm)
        if need_dn:
            grad_down_proj = ops.expert_wgrad(grad_eo, inter, perm)
        grad_wt = grad_w.to(ctx.wt_dtype) if need_w else None
        return grad_hidden, None, grad_wt, grad_gate_up_proj, grad_down_proj, None


GLU_CODES = (0, 1, 2, 5, 6, 7)     # weight-carrying experts (kernels/sm75/moe.py:1-31)
FUSED_CODES = (0, 1, 5)            # applied inside the GEMM epilogues (no row reduction, no parameters)
SPECIAL_CODES = (3, 4)             # Identity, Zero: expert kinds without weights, listed after the GLU experts


def _code_info(act_codes: torch.Tensor):
    """(codes tuple, number of GLU experts), read from the device once per tensor lifetime: act_codes
    is static model config (the reference reads it with .tolist() on every call, moe.py:741)."""
    info = getattr(act_codes, "_code_info_cache", None)
    if info is None:
        codes = tuple(int(c) for c in act_codes.tolist())
        for c in codes:
            if c not in GLU_CODES + SPECIAL_CODES:
                raise ValueError(f"unknown act code {c}; supported: 0 SiLU, 1 ReLU^2, 2 NormSiLU, 3 Identity, "
                                 "4 Zero, 5 SiTU, 6 NormReLU^2, 7 NormSiTU")
        n_glu = sum(1 for c in codes if c in GLU_CODES)
        if any(c in SPECIAL_CODES for c in codes[:n_glu]):
            raise ValueError("GLU act codes must precede the Identity/Zero experts in act_codes")
        info = (codes, n_glu)
        try:
            act_codes._code_info_cache = info
        except Exception:
            pass
    return info


class _PolyGLUMoE(torch.autograd.Function):
    """Generic path for stacks that are not pure SiLU-GLU: the same sort / GEMMs / combine, with the
    activation as row kernels between the GEMMs (Norm codes need a row reduction over d_ff) and the
    Identity / Zero experts handled on their rows.  Mirrors _PerExpertMoE (kernels/sm75/moe.py:724-826)."""

    @staticmethod
    def forward(ctx, hidden, idx, wt, gate_up_proj, down_proj, act_codes, act_params):
        hidden, gate_up_proj, down_proj = _amp_cast(hidden, gate_up_proj, down_proj)
        for name, t in (("hidden", hidden), ("gate_up_proj", gate_up_proj), ("down_proj", down_proj)):
            L.require_cuda_bf16(name, t)
        codes, n_glu = _code_info(act_codes)
        E_total = len(codes)
        N, H = hidden.shape
        E, twoI, H2 = gate_up_proj.shape
        I = twoI // 2
        L.require(E == n_glu, f"gate_up_proj holds {E} experts but act_codes lists {n_glu} GLU experts")
        L.require(H2 == H and tuple(down_proj.shape) == (E, H, I), "weight shapes must be (E,2I,H) and (E,H,I)")
        L.require(tuple(idx.shape) == tuple(wt.shape) and idx.shape[0] == N, "indices/weights must be (N,k)")
        hidden, gate_up_proj, down_proj = hidden.contiguous(), gate_up_proj.contiguous(), down_proj.contiguous()
        w32 = wt.detach().float().contiguous()
        codes_dev = act_codes.to(device=hidden.device, dtype=torch.int32).contiguous()
        ap32 = None
        if act_params is not None:
            L.require(tuple(act_params.shape) == (E_total, 2), "act_params must be (E,2) [alpha, gamma]")
            ap32 = act_params.detach().float().contiguous()

        import dataclasses
        perm = ops.permute_build(idx, E_total)
        perm_glu = dataclasses.replace(perm, E=n_glu)          # GEMMs and row kernels see the GLU rows only
        x_s = ops.gather_rows(hidden, perm)
        gate_up = ops.expert_linear(x_s, gate_up_proj, perm_glu)
        inter = ops.glu_fwd_rows(gate_up, codes_dev, ap32, perm_glu)
        eo = ops.expert_linear(inter, down_proj, perm_glu)
        if n_glu < E_total:
            ops.special_rows(x_s, eo, codes_dev, perm, n_glu)
        out = ops.combine(eo, w32, perm)

        ctx.perm, ctx.perm_glu, ctx.n_glu, ctx.E_total = perm, perm_glu, n_glu, E_total
        ctx.wt_dtype = wt.dtype
        ctx.has_params = ap32 is not None
        ctx.save_for_backward(x_s, gate_up, inter, eo, w32, gate_up_proj, down_proj, codes_dev,
                              ap32 if ap32 is not None else torch.empty(0, device=hidden.device))
        return out

    @staticmethod
    def backward(ctx, grad_out):
        x_s, gate_up, inter, eo, w32, gate_up_proj, down_proj, codes_dev, ap32 = ctx.saved_tensors
        ap32 = ap32 if ctx.has_params else None
        perm, perm_glu, n_glu = ctx.perm, ctx.perm_glu, ctx.n_glu
        need_x, _, need_w, need_gu, need_dn, _, need_ap = ctx.needs_input_grad
        want_ap = bool(ctx.has_params and need_ap)
        grad_out = grad_out.contiguous().to(torch.bfloat16)
        grad_eo, grad_w = ops.combine_bwd(grad_out, eo, w32, perm)
        grad_inter = ops.expert_linear_t(grad_eo, down_proj, perm_glu)
        grad_gu, row_da, row_dg = ops.glu_bwd_rows(grad_inter, gate_up, codes_dev, ap32, perm_glu, want_ap)
        grad_down_proj = ops.expert_wgrad(grad_eo, inter, perm_glu) if need_dn else None
        grad_gate_up_proj = ops.expert_wgrad(grad_gu, x_s, perm_glu) if need_gu else None
        grad_hidden = None
        if need_x:
            grad_x_s = ops.expert_linear_t(grad_gu, gate_up_proj, perm_glu)
            if n_glu < ctx.E_total:
                ops.special_rows(grad_eo, grad_x_s, codes_dev, perm, n_glu)
            grad_hidden = ops.combine(grad_x_s, None, perm)
        grad_ap = None
        if want_ap:
            grad_ap = torch.zeros(ctx.E_total, 2, dtype=torch.float32, device=x_s.device)
            ops.expert_row_sums(row_da, row_dg, perm_glu, grad_ap)
        grad_wt = grad_w.to(ctx.wt_dtype) if need_w else None
        return grad_hidden, None, grad_wt, grad_gate_up_proj, grad_down_proj, None, grad_ap


def _empty_result(hidden, top_k_weights, *params):
    """No tokens: an empty (0,H) result that still hangs on every differentiable input, so that a backward pass
    gives zero gradients of the right shapes (what the reference's eager loop does with zero rows)."""
    out = _amp_cast(hidden)[0]
    out = out + top_k_weights.to(out.dtype).sum(dim=-1, keepdim=True)
    for p in params:
        if p is not None:
            out = out + 0.0 * p.sum().to(out.dtype)
    return out


_BF16_COPIES = {}     # id(parameter) -> (weak reference, version, bf16 copy)


def _bf16_copy(t):
    """bf16 copy of an fp16 / fp32 expert stack, kept until the tensor changes (its autograd version counter moves
    on every in-place update, e.g. an optimizer step) or is freed.  Callers with fp32 master weights would otherwise
    pay a full copy of both stacks on every call.  Tensors that need a gradient are cast afresh, so that autograd
    carries the gradient back through the cast."""
    if t.requires_grad and torch.is_grad_enabled():
        return t.to(torch.bfloat16)
    import weakref
    key = id(t)
    hit = _BF16_COPIES.get(key)
    if hit is not None and hit[0]() is t and hit[1] == t._version:
        return hit[2]
    c = t.detach().to(torch.bfloat16)
    _BF16_COPIES[key] = (weakref.ref(t, lambda _r, k=key: _BF16_COPIES.pop(k, None)), t._version, c)
    return c


def moe(hidden, top_k_indices, top_k_weights, gate_up_proj, down_proj, act_codes, act_params=None):
    """hidden (N,H) bf16 (fp16 / fp32: computed in bf16), indices (N,k) int64, weights (N,k) float, gate_up_proj (E_glu,2I,H),
    down_proj (E_glu,H,I), act_codes (E,) int32, act_params (E,2) fp32 [alpha,gamma] for code 5 or None
    -> (N,H).  Same contract as the reference's `moe` (kernels/sm75/moe.py:838-855); differentiable
    w.r.t. hidden, weights, both projections and act_params.  A stack of SiLU / ReLU^2 / parameter-free SiTU experts
    (codes 0, 1, 5, no act_params, no Identity / Zero experts) runs with the activation fused into the GEMM epilogues;
    any other stack (Norm codes, learnable SiTU, special experts) runs the PolyGLU row kernels."""
    codes, n_glu = _code_info(act_codes)
    if hidden.shape[0] == 0:
        return _empty_result(hidden, top_k_weights, gate_up_proj, down_proj, act_params)
    if hidden.dtype in (torch.float16, torch.float32) and not torch.is_autocast_enabled("cuda"):
        # The reference computes in hidden's dtype.  The kernels here are bf16 (fp32 accumulation): fp16 / fp32 callers
        # get the bf16 computation, the result in their dtype and, through the casts, gradients in the dtypes of
        # their tensors.  Accuracy is that of the bf16 path (2e-2 relative L2 against fp32).
        bf = torch.bfloat16
        out = moe(hidden.to(bf), top_k_indices, top_k_weights, _bf16_copy(gate_up_proj), _bf16_copy(down_proj),
                  act_codes, act_params)
        return out.to(hidden.dtype)
    if act_params is None and n_glu == len(codes) and all(c in FUSED_CODES for c in codes):
        return _GroupedMoE.apply(hidden, top_k_indices, top_k_weights, gate_up_proj, down_proj, act_codes)
    return _PolyGLUMoE.apply(hidden, top_k_indices, top_k_weights, gate_up_proj, down_proj, act_codes, act_params)


def moe_grouped(hidden, top_k_indices, top_k_weights, gate_up_proj, down_proj, act_codes):
    """Same signature as kernels/sm75/moe.py:621 (which has no act_params: code 5 runs parameter-free)."""
    return moe(hidden, top_k_indices, top_k_weights, gate_up_proj, down_proj, act_codes)


def moe_per_expert(hidden, top_k_indices, top_k_weights, gate_up_proj, down_proj, act_codes, act_params=None):
    """Same signature as kernels/sm75/moe.py:829; runs the one grouped path."""
    return moe(hidden, top_k_indices, top_k_weights, gate_up_proj, down_proj, act_codes, act_params)
