"""CPU restatement of the reference's expert-stack optimizer step (Muon).  TEST INFRASTRUCTURE ONLY: nothing
in the package imports this file; tests, the smoke check and the CPU leg of the benchmark may.

Follows kernels/sm75/muon.py (`newton_schulz` :62-89, `FusedMuon.step` :366-434 and its capturable body
`_compute` :300-315) and kernels/muon/muon_scaling.py (`scalar_scale` :79-83, `aurora_update` :92-120,
`aurora_ema_update` :123-143, `aurora_ema_v2_update` :146-163, `apply_perrow` :166-195).  Plain PyTorch on the CPU, any iteration dtype (the reference iterates in fp16 on
Turing and bf16 on Blackwell, kernels/sm120/muon.py; fp32 is its numerically safe setting).

Pinned: tests/golden/make_golden_muon.py runs the reference's own `newton_schulz` and `FusedMuon` on the CPU
and stores their results; tests/test_muon_oracle.py compares this file with them.
"""
from __future__ import annotations

import torch

# Default schedule of the reference: 8 Keller-Jordan quintic steps + 2 polish steps (kernels/sm75/muon.py:50).
DSV4_COEFFS = ((3.4445, -4.7750, 2.0315),) * 8 + ((2.0, -1.5, 0.5),) * 2
RMS_TARGET = 0.2          # kernels/muon/muon_scaling.py:33
ROW_EPS = 1e-8            # PERROW_EPS, kernels/muon/muon_scaling.py:36


def newton_schulz(G: torch.Tensor, coeffs=DSV4_COEFFS, ns_dtype=torch.float32, eps: float = 1e-7) -> torch.Tensor:
    """Drive the singular values of every matrix of G ((r,c) or (E,r,c)) towards 1 (kernels/sm75/muon.py:62-89):
    fp32 Frobenius norm per matrix, clamp at eps, work on the wide orientation, divide in ns_dtype, then for each
    (a,b,c): A = X X^T; B = b A + c A A; X = a X + B X; transpose back, return in G's dtype."""
    X = G[None] if G.dim() == 2 else G
    nrm = X.flatten(1).float().pow(2).sum(1).sqrt().clamp_min(eps).view(-1, 1, 1)
    tall = X.shape[1] > X.shape[2]
    if tall:
        X = X.transpose(1, 2)
    X = X.to(ns_dtype) / nrm.to(ns_dtype)
    for a, b, c in coeffs:
        A = X @ X.transpose(1, 2)
        B = (b * A.float() + c * (A @ A).float()).to(ns_dtype) if ns_dtype != torch.float32 else b * A + c * (A @ A)
        X = (a * X.float() + (B @ X).float()).to(ns_dtype) if ns_dtype != torch.float32 else a * X + B @ X
    if tall:
        X = X.transpose(1, 2)
    X = X[0] if G.dim() == 2 else X
    return X.to(G.dtype)


def polar_scale(rows: int, cols: int) -> float:
    """scale_mode "polar": 0.2 * sqrt(max(rows, cols)) (kernels/muon/muon_scaling.py:79-83)."""
    return RMS_TARGET * max(rows, cols) ** 0.5


def aurora_update(M: torch.Tensor, coeffs=DSV4_COEFFS, ns_dtype=torch.float32) -> torch.Tensor:
    """scale_mode "aurora" with K = 1, beta = 0 (kernels/muon/muon_scaling.py:101-112): rows divided by their fp32
    L2 norm (clamped at 1e-8) and multiplied by sqrt(min(r,c)/r), one orthogonalisation, times the polar gain."""
    rows, cols = M.shape[-2], M.shape[-1]
    tgt = (min(rows, cols) / rows) ** 0.5
    rn = M.float().pow(2).sum(-1).sqrt().clamp_min(ROW_EPS)
    pre = (M.float() * (tgt / rn).unsqueeze(-1)).to(M.dtype)
    X = newton_schulz(pre, coeffs, ns_dtype)
    return (X.float() * polar_scale(rows, cols)).to(M.dtype)


PERROW_BETA2 = 0.95       # kernels/muon/muon_scaling.py:35


def aurora_update_k(M: torch.Tensor, K: int, coeffs=DSV4_COEFFS, ns_dtype=torch.float32) -> torch.Tensor:
    """scale_mode "aurora" with K passes and beta = 0, the general branch of `aurora_update`
    (kernels/muon/muon_scaling.py:113-120): Frobenius-normalise, then K times {divide rows by their L2 norm, times
    sqrt(min(r,c)/r), orthogonalise}; times the polar gain.  K = 1 equals `aurora_update` above."""
    rows, cols = M.shape[-2], M.shape[-1]
    tgt = (min(rows, cols) / rows) ** 0.5
    X = M.float()
    fro = X.flatten(-2, -1).norm(dim=-1).clamp_min(ROW_EPS)
    X = X / fro.view(-1, 1, 1)
    for _ in range(K):
        r = X.norm(dim=-1).clamp_min(ROW_EPS)
        X = newton_schulz((tgt * (X / r.unsqueeze(-1))).to(M.dtype), coeffs, ns_dtype).float()
    return (polar_scale(rows, cols) * X).to(M.dtype)


def aurora_ema_update(M, v_ema, coeffs=DSV4_COEFFS, ns_dtype=torch.float32, beta2=PERROW_BETA2):
    """scale_mode "aurora_ema" (kernels/muon/muon_scaling.py:123-143): rows prescaled by the EMA of their normalised
    mean square (v_ema (n, rows) fp32, updated in place) before ONE orthogonalisation."""
    rows, cols = M.shape[-2], M.shape[-1]
    tgt = (min(rows, cols) / rows) ** 0.5
    rn = M.float().pow(2).sum(-1).sqrt()
    fro = rn.pow(2).sum(-1).sqrt().clamp_min(ROW_EPS)
    row_ms = (rn / fro.unsqueeze(-1)).square() / cols
    v_ema.mul_(beta2).add_(row_ms, alpha=1.0 - beta2)
    D = v_ema.sqrt().clamp_min(ROW_EPS)
    X = newton_schulz((M.float() * (tgt / (fro.unsqueeze(-1) * D)).unsqueeze(-1)).to(M.dtype), coeffs, ns_dtype)
    return (X.float() * polar_scale(rows, cols)).to(M.dtype)


def apply_perrow(O, v, beta2=PERROW_BETA2):
    """scale_mode "normuon" (kernels/muon/muon_scaling.py:166-195): rows of the orthogonalised update divided by the
    root of the EMA of their mean square (v (n, rows) fp32, in place), each matrix rescaled to Frobenius norm
    0.2 * sqrt(rows * cols)."""
    rows, cols = O.shape[-2], O.shape[-1]
    rn = O.float().pow(2).sum(-1).sqrt()
    v.mul_(beta2).add_(rn.square() / cols, alpha=1.0 - beta2)
    inv = 1.0 / (v.sqrt() + ROW_EPS)
    fro = (rn * inv).pow(2).sum(-1).sqrt().clamp_min(1e-12)
    mult = inv * (RMS_TARGET * (rows * cols) ** 0.5 / fro).unsqueeze(-1)
    return (O.float() * mult.unsqueeze(-1)).to(O.dtype)


def aurora_ema_v2_update(M, v_ema, K=1, coeffs=DSV4_COEFFS, ns_dtype=torch.float32, beta2=PERROW_BETA2):
    """scale_mode "aurora_ema_v2" (kernels/muon/muon_scaling.py:146-163): the aurora update, then the per-row EMA
    rescale after the orthogonalisation, each matrix renormalised to the RMS target."""
    rows, cols = M.shape[-2], M.shape[-1]
    O = aurora_update_k(M, K, coeffs, ns_dtype).float()
    row_sq = O.mul(O).mean(dim=-1)
    v_ema.mul_(beta2).add_(row_sq, alpha=1.0 - beta2)
    Ohat = O / v_ema.sqrt().add(ROW_EPS).unsqueeze(-1)
    fro = Ohat.flatten(-2).norm(dim=-1).clamp_min(1e-12)
    return (Ohat * (RMS_TARGET * (rows * cols) ** 0.5 / fro).view(-1, 1, 1)).to(M.dtype)


def muon_step(p: torch.Tensor, grad: torch.Tensor, mom: torch.Tensor, lr: float, momentum: float = 0.95,
              nesterov: bool = True, weight_decay: float = 0.0, coeffs=DSV4_COEFFS, ns_dtype=torch.float32,
              scale_mode: str = "aurora", aurora_k: int = 1, scale_v: torch.Tensor | None = None):
    """One step on one stack, in place on p and mom (kernels/sm75/muon.py:381-434).  mom has dtype ns_dtype and the
    shape of p seen as (n, r, c); the gradient is first copied into ns_dtype (:386-388).  scale_v: the (n, r) fp32
    EMA state of the per-row modes ("normuon", "aurora_ema", "aurora_ema_v2"), updated in place."""
    r, c = p.shape[-2], p.shape[-1]
    if weight_decay != 0:
        p.mul_(1.0 - lr * weight_decay)
    g = grad.reshape(-1, r, c).to(ns_dtype)
    mom.mul_(momentum).add_(g)
    u = g.add(mom, alpha=momentum) if nesterov else mom
    if scale_mode == "polar":
        out, alpha = newton_schulz(u, coeffs, ns_dtype), -lr * polar_scale(r, c)
    elif scale_mode == "aurora":
        out = aurora_update(u, coeffs, ns_dtype) if aurora_k == 1 else aurora_update_k(u, aurora_k, coeffs, ns_dtype)
        alpha = -lr
    elif scale_mode == "aurora_ema":
        out, alpha = aurora_ema_update(u, scale_v, coeffs, ns_dtype), -lr
    elif scale_mode == "aurora_ema_v2":
        out, alpha = aurora_ema_v2_update(u, scale_v, aurora_k, coeffs, ns_dtype), -lr
    elif scale_mode == "normuon":
        out, alpha = apply_perrow(newton_schulz(u, coeffs, ns_dtype), scale_v), -lr
    else:
        raise ValueError(f"unknown scale_mode {scale_mode!r}")
    p.add_(out.reshape(p.shape).to(p.dtype), alpha=alpha)
    return p


def rel_l2(a: torch.Tensor, b: torch.Tensor) -> float:
    return float((a.double() - b.double()).norm() / b.double().norm().clamp_min(1e-30))
