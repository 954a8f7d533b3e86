"""CPU oracle for the MXFP8 path: quantise -> dequantise restatement of the OCP MX format
(e4m3 elements, one E8M0 power-of-two scale per block of 32 elements along the GEMM's K).

TEST INFRASTRUCTURE ONLY.  PARITY UNPINNED: the reference (IsNoobgrammer/triton-kernel-fused) has
no MXFP8 / FP8 code at all (no e4m3, e8m0 or scaled-mm anywhere in its tree), so there is no
reference output to pin this file against; it restates the published MX convention:
    exponent = floor(log2(amax)) - 8,  scale byte = exponent + 127 clamped to [0, 254],
    element  = round-to-nearest-even(x / 2^exponent) saturated to +-448.
The exponent is computed with integer arithmetic (frexp), never through a float8 cast of the scale.
"""
from __future__ import annotations

import torch

E4M3_MAX = 448.0


def quantise(x: torch.Tensor):
    """x (..., K) float, K % 32 == 0 -> (codes uint8 (..., K), scale bytes uint8 (..., K/32))."""
    x = x.float()
    K = x.shape[-1]
    xb = x.reshape(*x.shape[:-1], K // 32, 32)
    amax = xb.abs().amax(-1)
    _, ex = torch.frexp(amax)                       # amax = m * 2^ex, m in [0.5, 1)
    sb = (ex - 1 - 8 + 127).clamp(0, 254)
    sb = torch.where((amax == 0) | (amax < 2.0 ** -126), torch.zeros_like(sb), sb)
    inv = torch.pow(2.0, (127 - sb).float())
    y = (xb * inv[..., None]).clamp(-E4M3_MAX, E4M3_MAX)
    codes = y.to(torch.float8_e4m3fn).view(torch.uint8).reshape(x.shape)
    return codes, sb.to(torch.uint8)


def dequantise(codes: torch.Tensor, sb: torch.Tensor) -> torch.Tensor:
    K = codes.shape[-1]
    v = codes.view(torch.float8_e4m3fn).float().reshape(*codes.shape[:-1], K // 32, 32)
    return (v * torch.pow(2.0, sb.float() - 127.0)[..., None]).reshape(codes.shape)


def qdq(x: torch.Tensor) -> torch.Tensor:
    """Quantise then dequantise along the last dimension."""
    return dequantise(*quantise(x))


def sf_atoms(sb: torch.Tensor) -> torch.Tensor:
    """Scale bytes (R, K/32) -> the 512-byte-atom layout the kernels use: atom (row//128, kb//4),
    byte (row%32)*16 + ((row%128)//32)*4 + kb%4; rows and k-blocks padded with zeros."""
    R, KB = sb.shape
    RB, KC = (R + 127) // 128, (KB + 3) // 4
    pad = torch.zeros(RB * 128, KC * 4, dtype=torch.uint8)
    pad[:R, :KB] = sb
    a = pad.view(RB, 4, 32, KC, 4)               # rb, quarter, row%32, kc, kb%4
    return a.permute(0, 3, 2, 1, 4).contiguous().view(-1)   # rb, kc, row%32, quarter, kb%4


class _MxMatmul(torch.autograd.Function):
    """out = qdq_K(a) @ qdq_K(b)^T with a (M,K), b (N,K); every GEMM of the backward quantises its
    own operands along its own reduction dimension (the MX training recipe)."""

    @staticmethod
    def forward(ctx, a, b):
        ctx.save_for_backward(a, b)
        return qdq(a) @ qdq(b).t()

    @staticmethod
    def backward(ctx, g):
        a, b = ctx.saved_tensors
        ga = qdq(g) @ qdq(b.t().contiguous()).t()                       # reduce over N
        gb = qdq(g.t().contiguous()) @ qdq(a.t().contiguous()).t()      # reduce over M
        return ga, gb


def mx_matmul_nt(a, b):
    return _MxMatmul.apply(a, b)


def moe_experts_mxfp8(hidden, top_k_indices, top_k_weights, gate_up_proj, down_proj):
    """The expert pipeline of oracle.moe_oracle.moe_experts with every GEMM replaced by its
    quantise->dequantise version (fp32 everywhere else)."""
    from . import moe_oracle as O
    N, H = hidden.shape
    E, twoI, _ = gate_up_proj.shape
    I = twoI // 2
    order, st, counts, offs = O.sort_by_expert_stable(top_k_indices, E)
    sw = top_k_weights.flatten()[order]
    out = torch.zeros(N, H, dtype=torch.float32, device=hidden.device)   # runs on whichever device holds the inputs
    w_gu, w_dn = gate_up_proj.unbind(0), down_proj.unbind(0)
    for e in range(E):
        s, en = int(offs[e]), int(offs[e + 1])
        if en == s:
            continue
        m = en - s
        pad = (-m) % 32                              # the kernels reduce over zero-padded token rows
        rows = st[s:en]
        x_e = torch.cat([hidden[rows], hidden.new_zeros(pad, H)])
        gu = mx_matmul_nt(x_e, w_gu[e])
        inter = O.swiglu(gu, I)
        eo = mx_matmul_nt(inter, w_dn[e])[:m]
        out = out.index_add(0, rows, eo * sw[s:en].unsqueeze(-1))
    return out
