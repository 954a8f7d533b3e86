"""Sigmoid-gate linear router behind the reference's callables (kernels/sm75/router.py).

`fused_mlp_router` (:277-289), `FusedMLPRouter` (:221-260) and `router_bias_update` (:292-301) keep
their signatures.  Logits are a tcgen05 GEMM (fp32 accumulate, stored in x's dtype as the reference
does), followed by the warp-level top-k epilogue kernel; backward is the epilogue Jacobian kernel
plus two tcgen05 GEMMs (dX, and dW as a split-K reduction over the tokens).
"""
from __future__ import annotations

import torch

from . import _lib as L
from . import ops

__all__ = ["fused_mlp_router", "FusedMLPRouter", "fused_router", "FusedConvRouter", "router_bias_update"]


class FusedMLPRouter(torch.autograd.Function):
    """Returns (idx (N,k) int64, weights (N,k) fp32 final, counts (E,) int32); only `weights` is
    differentiable (kernels/sm75/router.py:229-242)."""

    @staticmethod
    def forward(ctx, x, weight, bias, top_k, num_experts, norm_topk=True, scale=1.0):
        if torch.is_autocast_enabled("cuda"):
            dt = torch.get_autocast_dtype("cuda")
            x, weight = x.to(dt), weight.to(dt)
        L.require_cuda_bf16("x", x)
        L.require_cuda_bf16("gate_weight", weight)
        L.require(weight.dim() == 2 and weight.shape[1] == x.shape[-1], "gate_weight must be (E,H)")
        L.require(num_experts is None or int(num_experts) == weight.shape[0], "num_experts must equal gate_weight.shape[0]")
        xf = x.reshape(-1, x.shape[-1]).contiguous()
        weight = weight.contiguous()
        logits = ops.gemm_nt(xf, weight)
        bias32 = None
        if bias is not None:
            bias32 = bias.detach().float().contiguous()
        idx, w, counts = ops.router_topk_fwd(logits, bias32, top_k, norm_topk and top_k > 1, scale)
        ctx.xshape = x.shape
        ctx.save_for_backward(xf, weight, logits, idx)
        ctx.norm, ctx.scale = bool(norm_topk and top_k > 1), float(scale)
        ctx.mark_non_differentiable(idx, counts)
        return idx, w, counts

    @staticmethod
    def backward(ctx, grad_idx, grad_weights, grad_counts):
        xf, weight, logits, idx = ctx.saved_tensors
        gl = ops.router_topk_bwd(logits, idx, grad_weights, ctx.norm, ctx.scale)
        grad_x = ops.gemm_nn(gl, weight).view(ctx.xshape) if ctx.needs_input_grad[0] else None
        grad_w = ops.gemm_tn(gl, xf) if ctx.needs_input_grad[1] else None
        return grad_x, grad_w, None, None, None, None, None


def _empty_routing(x, weight, top_k):
    """No tokens: empty picks and weights (the weights still hang on x and the gate weight), zero counts."""
    n = x.numel() // max(x.shape[-1], 1)
    idx = torch.zeros(n, top_k, dtype=torch.int64, device=x.device)
    w = (x.reshape(n, x.shape[-1])[:, :1].float() + 0.0 * weight.float().sum()).expand(n, top_k)
    counts = torch.zeros(weight.shape[0], dtype=torch.int32, device=x.device)
    return idx, w, counts


def fused_mlp_router(x, gate_weight, bias, top_k, num_experts, norm_topk_prob=True,
                     routed_scaling_factor=1.0, return_counts=False):
    """x (B,S,H) or (N,H), gate_weight (E,H), bias (E,) fp32 or None -> (idx, weights[, counts]);
    (B,S,k) shapes for 3-D x (kernels/sm75/router.py:277-289)."""
    if x.numel() == 0:
        idx, w, counts = _empty_routing(x, gate_weight, top_k)
    else:
        idx, w, counts = FusedMLPRouter.apply(x, gate_weight, bias, top_k, num_experts, norm_topk_prob,
                                              routed_scaling_factor)
    if x.ndim == 3:
        B, S, _ = x.shape
        idx = idx.view(B, S, top_k)
        w = w.view(B, S, top_k)
    return (idx, w, counts) if return_counts else (idx, w)


class FusedConvRouter(torch.autograd.Function):
    """Causal-conv router (kernels/sm75/router.py:172-218, FusedConvRouterCuDNN): logits[b,s,e] =
    sum_{j,h} x[b, s-(K-1)+j, h] * W[e,h,j], then the same sigmoid / bias / top-k epilogue.  The conv is one
    tcgen05 GEMM whose TMA producer reads x in place, tap by tap, through a (H, S, B) tensor map (S a multiple of
    128, H of 64; as kernels/sm120/router.py:34-85 does in one launch), or over an unfolded copy of x for other
    shapes; backward = epilogue Jacobian, dX GEMM (the same way over grad_logits when E is a multiple of 64, else
    plain GEMM + fold), split-K dW GEMM."""

    @staticmethod
    def forward(ctx, x, weight, bias, top_k, num_experts, norm_topk=True, scale=1.0):
        if torch.is_autocast_enabled("cuda"):
            dt = torch.get_autocast_dtype("cuda")
            x, weight = x.to(dt), weight.to(dt)
        L.require_cuda_bf16("x", x)
        L.require_cuda_bf16("conv_weight", weight)
        L.require(x.dim() == 3 and weight.dim() == 3 and weight.shape[1] == x.shape[2], "need x (B,S,H) and conv_weight (E,H,K)")
        B, S, H = x.shape
        E, _, K = weight.shape
        L.require(num_experts is None or int(num_experts) == E, "num_experts must equal conv_weight.shape[0]")
        x = x.contiguous()
        wf = weight.permute(0, 2, 1).reshape(E, K * H).contiguous()      # Wf[e, j*H+h] = W[e,h,j]
        ctx.direct = ops.conv_direct_ok(S, H)
        if ctx.direct:
            xu = x                                                        # read in place by the GEMMs
            logits = ops.conv_gemm_fwd(x, wf, K)
        else:
            xu = ops.conv_unfold(x, K)
            logits = ops.gemm_nt(xu, wf)
        bias32 = bias.detach().float().contiguous() if bias is not None else None
        idx, w, counts = ops.router_topk_fwd(logits, bias32, top_k, norm_topk and top_k > 1, scale)
        ctx.shape = (B, S, H, E, K)
        ctx.save_for_backward(xu, wf, weight, logits, idx)
        ctx.norm, ctx.scale = bool(norm_topk and top_k > 1), float(scale)
        ctx.mark_non_differentiable(idx, counts)
        return idx, w, counts

    @staticmethod
    def backward(ctx, grad_idx, grad_weights, grad_counts):
        xu, wf, weight, logits, idx = ctx.saved_tensors
        B, S, H, E, K = ctx.shape
        gl = ops.router_topk_bwd(logits, idx, grad_weights, ctx.norm, ctx.scale)
        grad_x = None
        if ctx.needs_input_grad[0]:
            if ctx.direct and E % 64 == 0:
                wb = weight.permute(2, 0, 1).reshape(K * E, H).contiguous()   # Wb[j*E+e, h] = W[e,h,j]
                grad_x = ops.conv_gemm_dx(gl, wb, B, S, K)
            else:
                grad_x = ops.conv_fold(ops.gemm_nn(gl, wf), B, S, H, K)
        grad_w = None
        if ctx.needs_input_grad[1]:
            gwf = ops.conv_gemm_dw(gl, xu, K) if ctx.direct else ops.gemm_tn(gl, xu)
            grad_w = gwf.view(E, K, H).permute(0, 2, 1).contiguous()
        return grad_x, grad_w, None, None, None, None, None


def fused_router(x, conv_weight, bias, top_k, num_experts, norm_topk_prob=True, routed_scaling_factor=1.0,
                 return_counts=False):
    """Whole conv router: x (B,S,H), conv_weight (E,H,K) from nn.Conv1d(H,E,K), bias (E,) fp32 or None ->
    (idx (B,S,k) int64, weights (B,S,k) fp32[, counts (E,) int32]); kernels/sm75/router.py:263-274."""
    B, S, _ = x.shape
    if x.numel() == 0:
        idx, w, counts = _empty_routing(x, conv_weight, top_k)
    else:
        idx, w, counts = FusedConvRouter.apply(x, conv_weight, bias, top_k, num_experts, norm_topk_prob,
                                               routed_scaling_factor)
    idx = idx.view(B, S, top_k)
    w = w.view(B, S, top_k)
    return (idx, w, counts) if return_counts else (idx, w)


@torch.no_grad()
def router_bias_update(bias, counts, u):
    """b += u*sign(mean_load - load), in place; `counts` must already be the global load (the caller
    all-reduces it across ranks first); no-op when u <= 0 (kernels/sm75/router.py:292-301)."""
    if u <= 0:
        return
    ops.router_bias_update(bias, counts.to(torch.int32).contiguous(), u)
