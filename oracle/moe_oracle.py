"""CPU oracle for the MoE block: sigmoid+bias top-k router, expert sort, SwiGLU experts, combine.

TEST INFRASTRUCTURE ONLY.  Nothing in the product package may import this module; it is used by
the tests, by the smoke check and by the CPU-baseline leg of the benchmark as the checker.

Every function restates, in plain PyTorch on the CPU, what one piece of the reference
(IsNoobgrammer/triton-kernel-fused) computes, and cites the reference lines it follows.
Parity pin: `tests/golden/make_golden.py` runs the reference's own `moe_eager` and
`_sort_by_expert` (they import and run on CPU) and stores their outputs; `tests/test_oracle.py`
checks this module against those stored outputs.  The router functions are pinned on the
reference's own fused kernels: `tests/golden/make_golden_router.py` runs `_epilogue_fwd`,
`_router_epilogue_bwd_kernel`, `_count_experts`, `FusedMLPRouter`, `FusedConvRouterCuDNN` and
`router_bias_update` of kernels/sm75/router.py under the Triton interpreter on CPU tensors
(tie-free logits and logits full of exact ties), and `tests/test_router_golden.py` holds
`router_epilogue_fwd/bwd`, `mlp_router_fwd/bwd`, `conv_router_logits` and `router_bias_update`
to those outputs (picks and counts bit-exact, weights 1e-6, gradients 1e-5).
"""
from __future__ import annotations

import torch
import torch.nn.functional as F

NEG_KNOCKOUT = -1e30   # kernels/sm75/router.py:64,75


# ----------------------------------------------------------------------------- router
def sigmoid_scores(logits: torch.Tensor) -> torch.Tensor:
    """fp32 scores = 1/(1+exp(-logit))  (kernels/sm75/router.py:57-59)."""
    x = logits.float()
    return 1.0 / (1.0 + torch.exp(-x))


def topk_from_scores(scores: torch.Tensor, bias, top_k: int, norm_topk: bool = True,
                     scale: float = 1.0):
    """Selection from fp32 scores (N,E): sel = scores + bias picks, lowest index wins ties, picks
    are emitted in descending-sel order, weights are the UNBIASED scores at the picks, divided by
    (sum + 1e-20) when norm_topk and top_k > 1, then multiplied by scale.
    Follows kernels/sm75/router.py:60-79 (iterative argmax with -1e30 knock-out).
    Returns idx int64 (N,k), w fp32 (N,k), counts int32 (E,)."""
    scores = scores.float()
    N, E = scores.shape
    sel = scores.clone()
    if bias is not None:
        sel = sel + bias.float()[None, :]
    idx = torch.empty(N, top_k, dtype=torch.int64)
    w = torch.empty(N, top_k, dtype=torch.float32)
    rows = torch.arange(N)
    for k in range(top_k):
        mx = sel.max(dim=1, keepdim=True).values
        # lowest index among the maxima (tl.argmax tie rule, router.py:68)
        am = (sel == mx).to(torch.int8).argmax(dim=1)
        idx[:, k] = am
        w[:, k] = scores[rows, am]
        sel[rows, am] = NEG_KNOCKOUT
    if norm_topk and top_k > 1:
        t = torch.zeros(N, dtype=torch.float32)
        for k in range(top_k):          # fixed left-to-right fp32 summation order
            t = t + w[:, k]
        t = t + 1e-20
        w = w / t[:, None]
    w = w * float(scale)
    counts = torch.bincount(idx.flatten(), minlength=E).to(torch.int32)
    return idx, w, counts


def router_epilogue_fwd(logits, bias, top_k, norm_topk=True, scale=1.0):
    """logits (N,E) any float dtype -> (idx, w, counts); kernels/sm75/router.py:39-83."""
    return topk_from_scores(sigmoid_scores(logits), bias, top_k, norm_topk, scale)


def router_epilogue_bwd(logits, idx, grad_w, norm_topk=True, scale=1.0, out_dtype=None):
    """grad_logits (N,E) from grad of the final weights; kernels/sm75/router.py:86-126.
    With norm: graw_j = scale/T * (G_j - <G,w>/T), T = sum_k w_k + 1e-20 (w = raw picked scores);
    without: graw_j = scale*G_j.  Scattered to the picked columns, times s(1-s)."""
    s = sigmoid_scores(logits)
    N, E = s.shape
    k = idx.shape[1]
    G = grad_w.float()
    wk = s.gather(1, idx)
    if norm_topk and k > 1:
        t = wk.sum(1) + 1e-20
        dot = (G * wk).sum(1)
        graw = (float(scale) / t)[:, None] * (G - (dot / t)[:, None])
    else:
        graw = G * float(scale)
    gscore = torch.zeros(N, E, dtype=torch.float32)
    gscore.scatter_add_(1, idx, graw)
    gout = gscore * (s * (1.0 - s))
    return gout.to(out_dtype if out_dtype is not None else logits.dtype)


def mlp_router_fwd(x, gate_weight, bias, top_k, norm_topk=True, scale=1.0):
    """Linear router forward (kernels/sm75/router.py:229-242): logits are produced in x's dtype
    (fp32 accumulate, one rounding) and the epilogue reads those rounded logits."""
    xf = x.reshape(-1, x.shape[-1])
    logits = (xf.float() @ gate_weight.float().t()).to(x.dtype)
    idx, w, counts = router_epilogue_fwd(logits, bias, top_k, norm_topk, scale)
    return idx, w, counts, logits


def mlp_router_bwd(x, gate_weight, logits, idx, grad_w, norm_topk=True, scale=1.0):
    """kernels/sm75/router.py:245-260: grad_logits in x dtype, then dX = gl@W, dW = gl^T@xf."""
    xf = x.reshape(-1, x.shape[-1])
    gl = router_epilogue_bwd(logits, idx, grad_w, norm_topk, scale, out_dtype=x.dtype)
    grad_x = (gl.float() @ gate_weight.float()).to(x.dtype).view(x.shape)
    grad_wt = (gl.float().t() @ xf.float()).to(gate_weight.dtype)
    return grad_x, grad_wt, gl


def router_bias_update(bias, counts, u):
    """b += u*sign(mean(c) - c), in place, no-op when u <= 0 (kernels/sm75/router.py:292-301)."""
    if u <= 0:
        return bias
    tpe = counts.float()
    bias.add_(u * (tpe.mean() - tpe).sign())
    return bias


def eager_router_topk(x, gate_weight, bias, top_k):
    """The eager statement of the same router (.autoresearch/train_grok_moe.py:72-77):
    sigmoid -> +bias -> torch.topk -> gather -> /(sum+1e-20).  Differs from the fused rule only
    in tie order and pick order; used to cross-check the restatement on tie-free inputs."""
    scores = torch.sigmoid((x.float() @ gate_weight.float().t()))
    sel = scores + (bias.float() if bias is not None else 0.0)
    _, idx = torch.topk(sel, top_k, dim=-1)
    w = scores.gather(-1, idx)
    w = w / (w.sum(-1, keepdim=True) + 1e-20)
    return idx, w


# ----------------------------------------------------------------------------- permutation
def sort_by_expert_stable(idx: torch.Tensor, E: int):
    """Canonical permutation: slots (t*k+j) sorted by expert, ties by slot index (stable).
    The reference uses an unstable sort (kernels/sm75/moe.py:564-572), so its within-expert row
    order is unspecified; counts and bounds are the exact comparison, segments compare as sets.
    Returns order int64 (M,), st (token of each sorted row), counts int32 (E,), offs int32 (E+1,)."""
    N, k = idx.shape
    flat = idx.flatten()
    _, order = torch.sort(flat, stable=True)
    st = order // k
    counts = torch.bincount(flat, minlength=E).to(torch.int32)
    offs = torch.zeros(E + 1, dtype=torch.int32)
    offs[1:] = torch.cumsum(counts, 0)
    return order, st, counts, offs


def padded_layout(counts: torch.Tensor, tile: int = 256):
    """Tile-padded expert segments used by the CUDA path: expert e owns padded rows
    [poffs[e], poffs[e+1]) with poffs[e+1]-poffs[e] = ceil(counts[e]/tile)*tile.  Zero-count
    experts own zero rows (the reference emits zero tiles for them, kernels/sm75/moe.py:535-543)."""
    c = counts.to(torch.int64)
    padded = ((c + tile - 1) // tile) * tile
    poffs = torch.zeros(c.numel() + 1, dtype=torch.int32)
    poffs[1:] = torch.cumsum(padded, 0)
    return poffs


def permutation_tables(idx: torch.Tensor, E: int, tile: int = 256):
    """All tables the CUDA permute kernels emit, computed on the CPU:
    slot_row (M,) padded row of slot t*k+j; row_slot (poffs[E],) slot of each padded row or -1;
    tile_expert (poffs[E]/tile,) expert of each row tile."""
    order, st, counts, offs = sort_by_expert_stable(idx, E)
    poffs = padded_layout(counts, tile)
    M = idx.numel()
    flat = idx.flatten()
    pos = torch.empty(M, dtype=torch.int64)
    pos[order] = torch.arange(M)
    rank = pos - offs[:-1].to(torch.int64)[flat]
    slot_row = (poffs[:-1].to(torch.int64)[flat] + rank).to(torch.int32)
    total = int(poffs[-1])
    row_slot = torch.full((total,), -1, dtype=torch.int32)
    row_slot[slot_row.long()] = torch.arange(M, dtype=torch.int32)
    tile_expert = torch.repeat_interleave(
        torch.arange(E, dtype=torch.int32), ((poffs[1:] - poffs[:-1]) // tile).long())
    return dict(order=order, counts=counts, offs=offs, poffs=poffs, slot_row=slot_row,
                row_slot=row_slot, tile_expert=tile_expert)


# ----------------------------------------------------------------------------- experts
def swiglu(gate_up: torch.Tensor, I: int) -> torch.Tensor:
    """act code 0: silu(gate)*up with gate = cols [0,I), up = cols [I,2I)
    (kernels/sm75/moe.py:859-861,906-907)."""
    return F.silu(gate_up[:, :I]) * gate_up[:, I:]


def moe_experts(hidden, top_k_indices, top_k_weights, gate_up_proj, down_proj):
    """SwiGLU MoE experts with weighted fp32 combine; restates moe_eager
    (kernels/sm75/moe.py:884-909) for act code 0 through the sorted formulation, so it is
    differentiable by autograd and costs one pass per expert over that expert's rows only."""
    N, H = hidden.shape
    E, twoI, _ = gate_up_proj.shape
    I = twoI // 2
    k = top_k_indices.shape[1]
    order, st, counts, offs = sort_by_expert_stable(top_k_indices, E)
    sw = top_k_weights.flatten()[order]
    out = torch.zeros(N, H, dtype=torch.float32)
    # unbind once: the backward of a per-expert select would allocate a full (E,.,.) zero tensor per
    # expert; this only changes how autograd accumulates, not any value
    w_gu, w_dn = gate_up_proj.unbind(0), down_proj.unbind(0)
    for e in range(E):
        s, en = int(offs[e]), int(offs[e + 1])
        if en == s:
            continue
        rows = st[s:en]
        gu = hidden[rows] @ w_gu[e].t()
        inter = swiglu(gu, I)
        eo = inter @ w_dn[e].t()
        out = out.index_add(0, rows, (eo * sw[s:en].unsqueeze(-1).to(eo.dtype)).float())
    return out.to(hidden.dtype)


def moe_layer(x, gate_weight, bias, gate_up_proj, down_proj, top_k, norm_topk=True, scale=1.0,
              logits_dtype=None, idx_override=None):
    """Whole block, differentiable by autograd w.r.t. x, gate_weight and the expert weights:
    router (selection is non-differentiable, weights are) -> experts -> combine.
    logits_dtype: round the logits to this dtype before the sigmoid, as the reference does when it
    runs in bf16 (kernels/sm75/router.py:235 stores logits in x's dtype); gradients pass straight
    through the rounding."""
    xf = x.reshape(-1, x.shape[-1])
    logits = (xf @ gate_weight.t())
    if logits_dtype is not None:
        logits = logits + (logits.detach().to(logits_dtype).to(logits.dtype) - logits.detach())
    with torch.no_grad():
        idx, _, counts = router_epilogue_fwd(logits, bias, top_k, norm_topk, scale)
    if idx_override is not None:
        # the picks of another implementation of the same router (a logit that sits on a rounding boundary of
        # logits_dtype can land on either side and flip a pick): everything downstream of the selection is then
        # compared on identical routing
        idx = idx_override
        counts = torch.bincount(idx.flatten(), minlength=gate_weight.shape[0]).to(torch.int32)
    s = 1.0 / (1.0 + torch.exp(-logits.float()))
    w = s.gather(1, idx)
    if norm_topk and top_k > 1:
        w = w / (w.sum(-1, keepdim=True) + 1e-20)
    w = w * float(scale)
    out = moe_experts(xf, idx, w, gate_up_proj, down_proj)
    return out.view(x.shape), idx, w, counts


def layer_fwd_bwd(x, gate_weight, bias, gate_up_proj, down_proj, top_k, grad_out,
                  norm_topk=True, scale=1.0, logits_dtype=None, idx_override=None):
    """Forward + backward of the block under loss = sum(out * grad_out); returns a dict of the
    output and every gradient (fp32 when the inputs are fp32)."""
    leaves = [t.detach().clone().requires_grad_(True)
              for t in (x, gate_weight, gate_up_proj, down_proj)]
    xl, gl, gul, dl = leaves
    out, idx, w, counts = moe_layer(xl, gl, bias, gul, dl, top_k, norm_topk, scale, logits_dtype, idx_override)
    (out.float() * grad_out.float()).sum().backward()
    return dict(out=out.detach(), idx=idx, w=w.detach(), counts=counts, grad_x=xl.grad,
                grad_gate_weight=gl.grad, grad_gate_up=gul.grad, grad_down=dl.grad)


# ----------------------------------------------------------------------------- comparators
def rel_l2(a: torch.Tensor, b: torch.Tensor) -> float:
    """||a-b|| / ||b|| in fp64 (the reference's rel(), .autoresearch/grouped_parity.py:14-15)."""
    a = a.detach().double().flatten()
    b = b.detach().double().flatten()
    return float((a - b).norm() / b.norm().clamp_min(1e-30))


# ----------------------------------------------------------------------------- inputs
def make_inputs(T, H, E, I, k, seed=0, bias_std=0.0, zipf_s=None, dtype=torch.float32):
    """Seeded synthetic inputs with the distributions the benchmark configs name:
    x~N(0,1), every weight ~N(0,0.02), selection bias ~N(0,bias_std), optional log-Zipf logit
    bias, fixed upstream gradient ~N(0,1).  One generator per tensor so shapes can change independently."""
    def g(i):
        return torch.Generator().manual_seed(seed * 1000 + i)
    x = torch.randn(T, H, generator=g(1))
    wr = torch.randn(E, H, generator=g(2)) * 0.02
    gu = torch.randn(E, 2 * I, H, generator=g(3)) * 0.02
    dn = torch.randn(E, H, I, generator=g(4)) * 0.02
    go = torch.randn(T, H, generator=g(5))
    logit_bias = None
    if zipf_s is not None:
        # additive per-expert LOGIT bias = log of Zipf(s) frequencies, ranks assigned by a seeded
        # permutation of the experts (skewed-routing config)
        ranks = torch.randperm(E, generator=g(7)).float() + 1.0
        p = ranks.pow(-zipf_s)
        logit_bias = torch.log(p / p.sum())
    if bias_std > 0:
        bias = torch.randn(E, generator=g(6)) * bias_std
    else:
        bias = torch.zeros(E)
    cast = lambda t: t.to(dtype)
    return dict(x=cast(x), gate_weight=cast(wr), gate_up=cast(gu), down=cast(dn),
                grad_out=cast(go), bias=bias.float(), logit_bias=logit_bias)


# ----------------------------------------------------------------------------- PolyGLU
RMS_EPS = 1e-6      # _NS_EPS, kernels/sm75/moe.py:80


def polyglu_act(gate: torch.Tensor, code: int, alpha=1.0, gamma=1.0) -> torch.Tensor:
    """Activation of the gate half for act code `code`, fp32 (kernels/sm75/moe.py:859-881):
    0 SiLU, 1 ReLU^2, 2 NormSiLU, 5 SiTU gamma*tanh(alpha g)*sigmoid(g), 6 NormReLU^2, 7 NormSiTU;
    the Norm codes first divide each row by sqrt(mean(g^2) + 1e-6)."""
    g = gate.float()
    if code in (2, 6, 7):
        g = g * torch.rsqrt(g.square().mean(-1, keepdim=True) + RMS_EPS)
    if code in (0, 2):
        return g * torch.sigmoid(g)
    if code in (1, 6):
        return torch.relu(g) ** 2
    if code == 5:
        return gamma * torch.tanh(alpha * g) * torch.sigmoid(g)
    if code == 7:
        return torch.tanh(g) * torch.sigmoid(g)
    raise ValueError(f"not a GLU act code: {code}")


def moe_experts_polyglu(hidden, top_k_indices, top_k_weights, gate_up_proj, down_proj, codes, act_params=None):
    """moe_eager with heterogeneous experts (kernels/sm75/moe.py:884-909): GLU experts use weight
    slot e; Identity (3) passes the weighted input through; Zero (4) contributes nothing."""
    N, H = hidden.shape
    I = gate_up_proj.shape[1] // 2
    E = len(codes)
    order, st, counts, offs = sort_by_expert_stable(top_k_indices, E)
    sw = top_k_weights.flatten()[order]
    out = torch.zeros(N, H, dtype=torch.float32)
    w_gu, w_dn = gate_up_proj.unbind(0), down_proj.unbind(0)
    for e in range(E):
        s, en = int(offs[e]), int(offs[e + 1])
        if en == s or codes[e] == 4:
            continue
        rows = st[s:en]
        w = sw[s:en].unsqueeze(-1)
        if codes[e] == 3:
            out = out.index_add(0, rows, (hidden[rows] * w).float())
            continue
        gu = hidden[rows] @ w_gu[e].t()
        a, g = (act_params[e, 0], act_params[e, 1]) if (codes[e] == 5 and act_params is not None) else (1.0, 1.0)
        inter = polyglu_act(gu[:, :I], codes[e], a, g).to(gu.dtype) * gu[:, I:]
        out = out.index_add(0, rows, ((inter @ w_dn[e].t()) * w).float())
    return out.to(hidden.dtype)


# ----------------------------------------------------------------------------- conv router
def conv_router_logits(x, conv_weight):
    """Causal K-tap conv logits of the reference's conv router: x (B,S,H), conv_weight (E,H,K) ->
    (B*S, E); kernels/sm75/router.py:186-190 (conv1d with padding K-1, first S outputs) and the eager
    statement bench.py:414-416 (left pad K-1)."""
    B, S, H = x.shape
    K = conv_weight.shape[2]
    xp = F.pad(x.transpose(1, 2), (K - 1, 0))
    return F.conv1d(xp, conv_weight).transpose(1, 2).reshape(B * S, -1)


def conv_router_fwd(x, conv_weight, bias, top_k, norm_topk=True, scale=1.0, logits_dtype=None):
    """Forward of `fused_router`: conv logits (rounded to logits_dtype when given, as the reference
    stores them in x's dtype), then the shared epilogue.  Returns idx, w, counts, logits."""
    logits = conv_router_logits(x.float(), conv_weight.float())
    if logits_dtype is not None:
        logits = logits.to(logits_dtype)
    idx, w, counts = router_epilogue_fwd(logits, bias, top_k, norm_topk, scale)
    return idx, w, counts, logits
