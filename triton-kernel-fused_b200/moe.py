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


def _code_max(act_codes: torch.Tensor) -> int:
    """Largest activation code (negative codes count as unsupported), one host sync per tensor
    lifetime: act_codes is static model config (kernels/sm75/moe.py:84-94)."""
    m = getattr(act_codes, "_code_max_cache", None)
    if m is None:
        m = int(act_codes.abs().max()) if act_codes.numel() else 0
        try:
            act_codes._code_max_cache = m
        except Exception:
            pass
    return m


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

        perm = ops.permute_build(idx, E)
        x_s = ops.gather_rows(hidden, perm)
        gate_up, inter = ops.expert_gate_up_swiglu(x_s, gate_up_proj, perm)
        eo = ops.expert_down(inter, down_proj, perm)
        out = ops.combine(eo, w32, perm)

        ctx.perm = perm
        ctx.wt_dtype = wt.dtype
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
            grad_gu = ops.expert_down_dgrad_glu(grad_eo, down_proj, gate_up, perm)
            if need_gu:
                grad_gate_up_proj = ops.expert_wgrad(grad_gu, x_s, perm)
            if need_x:
                grad_x_s = ops.expert_gate_up_dgrad(grad_gu, gate_up_proj, perm)
                grad_hidden = ops.combine(grad_x_s, None, perm)
        if need_dn:
            grad_down_proj = ops.expert_wgrad(grad_eo, inter, perm)
        grad_wt = grad_w.to(ctx.wt_dtype) if need_w else None
        return grad_hidden, None, grad_wt, grad_gate_up_proj, grad_down_proj, None


def _check_codes(act_codes, act_params):
    if act_params is not None:
        raise ValueError("act_params (learnable SiTU, code 5) is not built in this library; only act code 0 (SwiGLU)")
    if _code_max(act_codes) != 0:
        raise ValueError("only act code 0 (SiLU-GLU) is built in this library; codes 1-7 are unsupported")


def moe(hidden, top_k_indices, top_k_weights, gate_up_proj, down_proj, act_codes, act_params=None):
    """hidden (N,H) bf16, indices (N,k) int64, weights (N,k) float, gate_up_proj (E,2I,H),
    down_proj (E,H,I), act_codes (E,) int32 (all 0) -> (N,H).  Same contract as the reference's
    `moe` (kernels/sm75/moe.py:838-855); differentiable w.r.t. hidden, weights and both projections."""
    _check_codes(act_codes, act_params)
    return _GroupedMoE.apply(hidden, top_k_indices, top_k_weights, gate_up_proj, down_proj, act_codes)


def moe_grouped(hidden, top_k_indices, top_k_weights, gate_up_proj, down_proj, act_codes):
    """Same signature as kernels/sm75/moe.py:621."""
    return moe(hidden, top_k_indices, top_k_weights, gate_up_proj, down_proj, act_codes)


def moe_per_expert(hidden, top_k_indices, top_k_weights, gate_up_proj, down_proj, act_codes, act_params=None):
    """Same signature as kernels/sm75/moe.py:829; runs the one grouped path."""
    return moe(hidden, top_k_indices, top_k_weights, gate_up_proj, down_proj, act_codes, act_params)
