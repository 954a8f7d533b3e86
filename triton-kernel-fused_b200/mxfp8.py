"""MXFP8 expert pipeline: the same block as `moe`, with every expert GEMM (forward, dgrad, wgrad)
run on tcgen05 block-scaled MMAs over e4m3 operands with E8M0 block-32 scales.

The reference has no MXFP8 path; the signature mirrors `moe` (kernels/sm75/moe.py:838) and the
numerics follow the OCP MX convention (see include/b200moe.h).  Master weights stay bf16 and are
quantised on every call; each GEMM quantises its operands along its own reduction dimension
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
        if need_x:
            wq, wsf, wgt, wgtsf = ops.mxfp8_quant_both(gate_up_proj, interleave_I=I)       # + (E, H, 2I)
        else:
            wq, wsf = ops.mxfp8_quant_rows(gate_up_proj.view(E * twoI, H), interleave_I=I)
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
        if need_x or need_gu:
            dq, dsf, wtq, wtsf = ops.mxfp8_quant_both(down_proj)                            # + (E, I, H)
        else:
            dq, dsf = ops.mxfp8_quant_rows(down_proj.view(E * H, I))
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
