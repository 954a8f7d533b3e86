"""MXFP8 expert pipeline: the same block as `moe`, with every expert GEMM (forward, dgrad, wgrad)
run on tcgen05 block-scaled MMAs over e4m3 operands with E8M0 block-32 scales.

The reference has no MXFP8 path; the signature mirrors `moe` (kernels/sm75/moe.py:838) and the
numerics follow the OCP MX convention (see include/b200moe.h).  Master weights stay bf16; their quantised
copies are kept until the weights change (autograd version counter: an optimizer step invalidates them, the
micro-batches of a gradient-accumulation step and inference calls reuse them; `WEIGHT_CACHE = False` turns it
off); each GEMM quantises its operands along its own reduction dimension
(row-wise for forward/dgrad activations, transposed copies for weights in dgrad and for both
operands of the wgrads).  Needs d_model % 128 == 0 and d_ff % 128 == 0.
"""
from __future__ import annotations

import os

import torch

from . import _lib as L
from . import ops
from .moe import _amp_cast, _code_info, _empty_result

__all__ = ["moe_mxfp8", "FUSE_QUANT_EPILOGUE"]

# B200MOE_MXFP8_FUSE_QUANT=1: where only the row-wise quantisation of a SwiGLU / GLU-backward result is
# needed (no weight gradient wants its transposed copy), the GEMM epilogue writes it (bit-identical to the
# row quantiser) instead of a separate pass.  Off by default: it measured 2 % slower on the full step,
# because the pair kernel's single-buffered accumulator exposes every cycle added to the epilogue.
FUSE_QUANT_EPILOGUE = os.environ.get("B200MOE_MXFP8_FUSE_QUANT", "0") == "1"

# Quantised copies of the expert stacks are reused while the stacks are unchanged (B200MOE_MXFP8_WEIGHT_CACHE=0: off).
# They cost one byte per weight and direction: 2 x the bf16 stack's bytes when both directions are kept.
WEIGHT_CACHE = os.environ.get("B200MOE_MXFP8_WEIGHT_CACHE", "1") == "1"
_QUANTISED = {}      # id(stack) -> (weak reference, version, data pointer, has the transposed copy, tensors)


def _quantised_weights(stack, rows_fn, both_fn, both):
    """(q, sf) or (q, sf, qt, sft) of an expert stack, from the cache when the stack is the same tensor, at the same
    address, with the same autograd version as when the copies were made (every in-place update moves the version)."""
    if not WEIGHT_CACHE:
        return both_fn() if both else rows_fn()
    import weakref
    key = id(stack)
    hit = _QUANTISED.get(key)
    if hit is not None and hit[0]() is stack and hit[1] == stack._version and hit[2] == stack.data_ptr() and (hit[3] or not both):
        return hit[4] if both or not hit[3] else hit[4][:2]
    res = both_fn() if both else rows_fn()
    _QUANTISED[key] = (weakref.ref(stack, lambda _r, k=key: _QUANTISED.pop(k, None)), stack._version, stack.data_ptr(),
                       both, res)
    return res


class _MoEMxfp8(torch.autograd.Function):
    @staticmethod
    def forward(ctx, hidden, idx, wt, gate_up_proj, down_proj, act_codes):
        hidden, gate_up_proj, down_proj = _amp_cast(hidden, gate_up_proj, down_proj)
        for name, t in (("hidden", hidden), ("gate_up_proj", gate_up_proj), ("down_proj", down_proj)):
            L.require_cuda_bf16(name, t)
        N, H = hidden.shape
        E, twoI, H2 = gate_up_proj.shape
        I = twoI // 2
        L.require(H2 == H and tuple(down_proj.shape) == (E, H, I), "weight shapes must be (E,2I,H) and (E,H,I)")
        L.require(H % 128 == 0 and I % 128 == 0, f"MXFP8 path needs d_model and d_ff multiples of 128 (got {H}, {I})")
        hidden = hidden.contiguous()
        gate_up_proj = gate_up_proj.contiguous()
        down_proj = down_proj.contiguous()
        w32 = wt.detach().float().contiguous()
        dev = hidden.device

        need_x, _, _, need_gu, need_dn, _ = ctx.needs_input_grad
        perm = ops.permute_build(idx, E)
        # the gather is the quantising producer; when the gate/up weight gradient is wanted it also writes the
        # copy quantised along the token rows, and the gathered bf16 rows are never materialised
        xt = xtsf = None
        if need_gu:
            xq, xsf, xt, xtsf = ops.mxfp8_gather_quant_both(hidden, perm)
        else:
            _, xq, xsf = ops.mxfp8_gather_quant(hidden, perm)
        # tensors that the backward needs quantised along their other dimension are quantised both ways in
        # one pass over DRAM, and the transposed copy is what the backward keeps
        wgt = wgtsf = wtq = wtsf = it = itsf = None
        res = _quantised_weights(gate_up_proj, lambda: ops.mxfp8_quant_rows(gate_up_proj.view(E * twoI, H), interleave_I=I),
                                 lambda: ops.mxfp8_quant_both(gate_up_proj, interleave_I=I), need_x)   # + (E, H, 2I)
        if need_x:
            wq, wsf, wgt, wgtsf = res
        else:
            wq, wsf = res
        gate_up = torch.empty(perm.cap, twoI, dtype=torch.bfloat16, device=dev)
        inter = torch.empty(perm.cap, I, dtype=torch.bfloat16, device=dev)
        fuse = FUSE_QUANT_EPILOGUE and not need_dn
        res = ops.mxfp8_expert_gemm(ops.EPI_SWIGLU, xq, xsf, wq, wsf, perm, twoI, H, I, gate_up, inter,
                                    quantise_result=fuse)
        if fuse:    # the SwiGLU epilogue also emitted `inter` quantised for the down GEMM
            _, iq, isf = res
        elif need_dn:
            iq, isf, it, itsf = ops.mxfp8_quant_both(inter)                                 # + (I, rows)
        else:
            iq, isf = ops.mxfp8_quant_rows(inter)
        res = _quantised_weights(down_proj, lambda: ops.mxfp8_quant_rows(down_proj.view(E * H, I)),
                                 lambda: ops.mxfp8_quant_both(down_proj), need_x or need_gu)           # + (E, I, H)
        if need_x or need_gu:
            dq, dsf, wtq, wtsf = res
        else:
            dq, dsf = res
        eo = torch.empty(perm.cap, H, dtype=torch.bfloat16, device=dev)
        ops.mxfp8_expert_gemm(ops.EPI_STORE, iq, isf, dq, dsf, perm, H, I, I, eo)
        out = ops.combine(eo, w32, perm)

        ctx.perm = perm
        ctx.wt_dtype = wt.dtype
        ctx.dims = (E, H, I)
        ctx.quantised = (wgt, wgtsf, wtq, wtsf, it, itsf, xt, xtsf)   # uint8 copies for the backward (not differentiable)
        ctx.save_for_backward(gate_up, eo, w32)
        return out

    @staticmethod
    def backward(ctx, grad_out):
        gate_up, eo, w32 = ctx.saved_tensors
        wgt, wgtsf, wtq, wtsf, it, itsf, xt, xtsf = ctx.quantised
        perm = ctx.perm
        E, H, I = ctx.dims
        twoI = 2 * I
        dev = eo.device
        need_x, _, need_w, need_gu, need_dn, _ = ctx.needs_input_grad
        grad_out = grad_out.contiguous().to(torch.bfloat16)
        grad_eo, grad_w = ops.combine_bwd(grad_out, eo, w32, perm)
        grad_hidden = grad_gate_up_proj = grad_down_proj = None
        gq = gsf = gt = gtsf = None
        if need_dn and (need_x or need_gu):
            gq, gsf, gt, gtsf = ops.mxfp8_quant_both(grad_eo)             # K = H, and (H, rows)
        elif need_dn:
            gt, gtsf = ops.mxfp8_quant_transpose(grad_eo)
        elif need_x or need_gu:
            gq, gsf = ops.mxfp8_quant_rows(grad_eo)
        if need_x or need_gu:
            grad_gu = torch.empty(perm.cap, twoI, dtype=torch.bfloat16, device=dev)
            fuse = FUSE_QUANT_EPILOGUE and need_x and not need_gu
            res = ops.mxfp8_expert_gemm(ops.EPI_GLU_BWD, gq, gsf, wtq, wtsf, perm, I, H, I, grad_gu, gate_up,
                                        quantise_result=fuse)
            ggq = ggsf = at = atsf = None
            if fuse:   # the GLU-backward epilogue also emitted grad_gate_up quantised along 2I
                _, ggq, ggsf = res
            elif need_x and need_gu:
                ggq, ggsf, at, atsf = ops.mxfp8_quant_both(grad_gu)       # K = 2I, and (2I, rows)
            elif need_x:
                ggq, ggsf = ops.mxfp8_quant_rows(grad_gu)
            else:
                at, atsf = ops.mxfp8_quant_transpose(grad_gu)
            if need_gu:
                grad_gate_up_proj = ops.mxfp8_expert_wgrad(at, atsf, xt, xtsf, perm)   # xt: (H, rows) from the forward
            if need_x:
                grad_x_s = torch.empty(perm.cap, H, dtype=torch.bfloat16, device=dev)
                ops.mxfp8_expert_gemm(ops.EPI_STORE, ggq, ggsf, wgt, wgtsf, perm, H, twoI, I, grad_x_s)
                grad_hidden = ops.combine(grad_x_s, None, perm)
        if need_dn:
            grad_down_proj = ops.mxfp8_expert_wgrad(gt, gtsf, it, itsf, perm)
        grad_wt = grad_w.to(ctx.wt_dtype) if need_w else None
        return grad_hidden, None, grad_wt, grad_gate_up_proj, grad_down_proj, None


def moe_mxfp8(hidden, top_k_indices, top_k_weights, gate_up_proj, down_proj, act_codes, act_params=None):
    """Same contract as `moe`; expert GEMMs in MXFP8 (e4m3 + E8M0 block-32 scales), bf16 in and out."""
    codes, n_glu = _code_info(act_codes)
    if act_params is not None or n_glu != len(codes) or any(c != 0 for c in codes):
        raise ValueError("the MXFP8 path is built for pure SiLU-GLU stacks (act code 0) only")
    if hidden.shape[0] == 0:
        return _empty_result(hidden, top_k_weights, gate_up_proj, down_proj)
    return _MoEMxfp8.apply(hidden, top_k_indices, top_k_weights, gate_up_proj, down_proj, act_codes)
