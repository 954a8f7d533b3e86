"""Expert-stack optimizer step (Muon) on the grouped tcgen05 GEMMs: the consumer of the MoE layer's weight gradients.

Mirrors kernels/sm75/muon.py of the reference: `newton_schulz(G, coeffs, ns_dtype, eps)` (:62-89), the optimizer
class `FusedMuon` (:91) with its `step` (:366-434), its CUDA-graph mode (:317-352) and `DistributedMuon` (:437-533),
for every scale mode of kernels/muon/muon_scaling.py ("polar", "aurora" with any number of passes, "normuon",
"aurora_ema", "aurora_ema_v2") and a bf16 iteration dtype (the reference's setting for Blackwell,
kernels/sm120/muon.py).  A stack (E, r, c) is orthogonalised as E independent matrices; the three products of each
Newton-Schulz iteration run as grouped GEMMs over a stack whose E row segments are padded to the 256-row GEMM tile,
everything that touches a whole stack (momentum, row norms, row scaling, packing/transposing, weight update) as
streaming kernels through the C ABI.  The per-row modes keep their arithmetic on the (matrices x rows) statistics,
a few thousand numbers per stack, in torch.

Not carried over (ValueError): cross-expert whitening (xorth_post), spectral weight decay, fp16 / fp32 iteration
dtypes, a damped aurora (beta != 0 is not reachable through the reference's constructor either).
"""
from __future__ import annotations

import torch

from . import _lib as L
from . import ops

__all__ = ["newton_schulz", "FusedMuon", "DistributedMuon", "DSV4_COEFFS"]

# the reference's default coefficient schedule (kernels/sm75/muon.py:50)
DSV4_COEFFS = ((3.4445, -4.7750, 2.0315),) * 8 + ((2.0, -1.5, 0.5),) * 2
RMS_TARGET = 0.2      # kernels/muon/muon_scaling.py:33
ROW_EPS = 1e-8        # kernels/muon/muon_scaling.py:36
PERROW_BETA2 = 0.95   # kernels/muon/muon_scaling.py:35
SCALE_MODES = ("polar", "aurora", "normuon", "aurora_ema", "aurora_ema_v2")    # kernels/muon/muon_scaling.py:24-28
PERROW_STATE_MODES = ("normuon", "aurora_ema", "aurora_ema_v2")                # keep a (matrices, rows) fp32 EMA
TILE = ops.TILE_M

_segments = {}


def _uniform_segments(E: int, Rp: int, device) -> ops.Permutation:
    """Row tables of a stack of E equal segments of Rp rows (Rp a multiple of the GEMM tile): what the grouped
    GEMMs read instead of a routing decision."""
    key = (E, Rp, torch.device(device).index)
    seg = _segments.get(key)
    if seg is None:
        i32 = dict(dtype=torch.int32, device=device)
        poffs = torch.arange(E + 1, **i32) * Rp
        tile_expert = torch.arange(E, **i32).repeat_interleave(Rp // TILE)
        counts = torch.full((E,), Rp, **i32)
        seg = ops.Permutation(T=0, k=1, E=E, cap=E * Rp, counts=counts, offs=poffs, poffs=poffs, slot_row=None,
                              row_slot=None, tile_expert=tile_expert, order=None, slot_pos=None)
        _segments[key] = seg
    return seg


def _check_stack(name: str, t: torch.Tensor):
    L.require(t.is_cuda, f"{name} must be a CUDA tensor (this package has no CPU path)")
    L.require(t.dim() in (2, 3), f"{name} must be a matrix or a stack of matrices, got {t.dim()} dimensions")
    r, c = t.shape[-2], t.shape[-1]
    L.require(r % 8 == 0 and c % 8 == 0, f"{name}: both matrix dimensions must be multiples of 8, got {r} x {c}")
    return (t.shape[0] if t.dim() == 3 else 1), r, c


@ops._op("muon_momentum", 1)
def _momentum(grad, mom, mu, nesterov, out=None):
    u = torch.empty_like(mom) if out is None else out
    L.check(L.lib().b200moe_muon_momentum(L.ptr(grad), 1 if grad.dtype == torch.float32 else 0, L.ptr(mom), L.ptr(u),
                                          mom.numel(), float(mu), 1 if nesterov else 0, L.stream_of(mom)))
    return u


@ops._op("muon_row_sumsq", 1)
def _row_sumsq(x, rows, cols):
    out = torch.empty(rows, dtype=torch.float32, device=x.device)
    L.check(L.lib().b200moe_muon_row_sumsq(L.ptr(x), rows, cols, L.ptr(out), L.stream_of(x)))
    return out


@ops._op("muon_prescale_rows", 1)
def _prescale_rows(x, rowss, rows, cols, tgt):
    out = torch.empty_like(x)
    ss = torch.empty_like(rowss)
    L.check(L.lib().b200moe_muon_prescale_rows(L.ptr(x), L.ptr(rowss), rows, cols, float(tgt), ROW_EPS, L.ptr(out),
                                               L.ptr(ss), L.stream_of(x)))
    return out, ss


@ops._op("muon_scale_rows", 1)
def _scale_rows(x, mult, rows, cols):
    """out = bf16(x * mult[row]) and the row sums of squares of out."""
    out = torch.empty_like(x)
    ss = torch.empty(rows, dtype=torch.float32, device=x.device)
    L.check(L.lib().b200moe_muon_scale_rows(L.ptr(x), L.ptr(mult), rows, cols, L.ptr(out), L.ptr(ss), L.stream_of(x)))
    return out, ss


@ops._op("muon_update_rows", 1)
def _update_rows(x, mult, rows, cols, decay, alpha, p):
    """p = decay * p + alpha * bf16(x * mult[row]); x in the parameter's own (rows, cols) layout."""
    L.check(L.lib().b200moe_muon_update_rows(L.ptr(x), L.ptr(mult), rows, cols, float(decay), float(alpha), L.ptr(p),
                                             1 if p.dtype == torch.float32 else 0, L.stream_of(p)))


@ops._op("muon_normalise_pack", 2)
def _normalise_pack(x, rowss, E, r, c, Rp, tall, eps):
    xp = torch.empty(E, Rp, r if tall else c, dtype=torch.bfloat16, device=x.device)
    norms = torch.empty(E, dtype=torch.float32, device=x.device)
    L.check(L.lib().b200moe_muon_normalise_pack(L.ptr(x), L.ptr(rowss), E, r, c, Rp, 1 if tall else 0, float(eps),
                                                L.ptr(norms), L.ptr(xp), L.stream_of(x)))
    return xp


@ops._op("axpby", 1)
def _axpby(x, alpha, y, beta, out, diag=0.0, ld=0):
    L.check(L.lib().b200moe_axpby_bf16(L.ptr(x), float(alpha), L.ptr(y), float(beta), float(diag), ld, L.ptr(out),
                                       x.numel(), L.stream_of(x)))
    return out


@ops._op("muon_apply", 1)
def _apply(xp, E, r, c, Rp, tall, gain, decay, alpha, p):
    L.check(L.lib().b200moe_muon_apply(L.ptr(xp), E, r, c, Rp, 1 if tall else 0, float(gain), float(decay),
                                       float(alpha), L.ptr(p), 1 if p.dtype == torch.float32 else 0, L.stream_of(p)))


def _orthogonalise_packed(u, E, r, c, coeffs, eps, rowss=None):
    """u (E, r, c) bf16 (rowss: its per-row sums of squares, if already known) -> the iterated stack in the
    iteration's layout (E, Rp, max(r,c)), its row padding Rp and whether it is transposed.
    kernels/sm75/muon.py:78-86."""
    tall = r > c
    small, wide = (c, r) if tall else (r, c)
    Rp = -(-small // TILE) * TILE
    if rowss is None:
        rowss = _row_sumsq(u, E * r, c)
    X = _normalise_pack(u, rowss, E, r, c, Rp, tall, eps)
    return _iterate(X, E, Rp, wide, coeffs), Rp, tall


def _iterate(X, E, Rp, wide, coeffs):
    """X <- a X + (b A + c A A) X with A = X X^T (kernels/sm75/muon.py:83-86), evaluated as ((b A + c A A) + a I) X:
    three grouped GEMMs per iteration (two of them over the upper triangle only), X ping-pongs between two buffers."""
    seg = _uniform_segments(E, Rp, X.device)
    rows = E * Rp
    A = torch.empty(rows, Rp, dtype=torch.bfloat16, device=X.device)
    A2 = torch.empty_like(A)
    Xn = torch.empty_like(X)
    for a, b, c in coeffs:
        # A = X X^T and B = c A A + b A + a I are symmetric: their GEMMs compute the upper tiles and store each chunk
        # right of the diagonal tile twice, the second time transposed (A A^T = A A; axpy and identity in the epilogue)
        ops.expert_gram(X.view(rows, wide), seg, out=A)
        ops.expert_linear_axpby(A, A.view(E, Rp, Rp), A, c, b, a, seg, out=A2, symmetric=2)
        ops.expert_linear_t(A2, X, seg, out=Xn.view(rows, wide))      # X = B X
        X, Xn = Xn, X
    return X


def _checked_momentum(mom, E, r, c, dev):
    """The momentum kernel reads and writes the buffer as E*r*c contiguous bf16 values on the parameter's device.
    `Optimizer.load_state_dict` casts floating-point state to the parameter's dtype (fp32 master weights turn a
    restored buffer into fp32) and may leave it on another device: such a buffer is brought back to bf16 (exact: it
    held bf16 values before the cast); a buffer of another size is refused rather than read out of bounds."""
    if not torch.is_tensor(mom) or mom.numel() != E * r * c:
        raise ValueError(f"optimizer state 'muon_mom' has {tuple(getattr(mom, 'shape', ()))}, the parameter needs "
                         f"({E}, {r}, {c})")
    if mom.dtype != torch.bfloat16 or mom.device != dev or not mom.is_contiguous() or mom.dim() != 3:
        mom = mom.to(device=dev, dtype=torch.bfloat16).contiguous().view(E, r, c)
    return mom


def newton_schulz(G: torch.Tensor, coeffs=DSV4_COEFFS, ns_dtype=torch.bfloat16, eps: float = 1e-7) -> torch.Tensor:
    """Orthogonalise every matrix of G ((r,c) or (E,r,c), CUDA, bf16 or fp32); same call as the reference's
    `newton_schulz` (kernels/sm75/muon.py:62).  Returns G's dtype and shape."""
    L.require(ns_dtype == torch.bfloat16, f"the iteration runs in bfloat16 only, got ns_dtype={ns_dtype}")
    E, r, c = _check_stack("G", G)
    L.require(G.dtype in (torch.bfloat16, torch.float32), f"G must be bfloat16 or float32, got {G.dtype}")
    u = G.detach().to(torch.bfloat16).contiguous().view(E, r, c)
    X, Rp, tall = _orthogonalise_packed(u, E, r, c, coeffs, eps)
    out = torch.zeros(E, r, c, dtype=G.dtype, device=G.device)
    _apply(X, E, r, c, Rp, tall, 1.0, 1.0, 1.0, out)              # out = 0 + 1 * X, laid back out as (E, r, c)
    return out.view(G.shape)


def _unpack(X, n, r, c, Rp, tall, gain=1.0):
    """The iteration's stack (n, Rp, max(r,c)) laid back out as (n, r, c) bf16, times `gain` (rounded to bf16)."""
    out = torch.zeros(n, r, c, dtype=torch.bfloat16, device=X.device)
    _apply(X, n, r, c, Rp, tall, gain, 0.0, 1.0, out)
    return out


class FusedMuon(torch.optim.Optimizer):
    """Muon for matrices and stacks of matrices; constructor and state follow the reference's `FusedMuon`
    (kernels/sm75/muon.py:91-137).  Parameters are CUDA tensors, bf16 or fp32 (fp32 master weights), 2-D or 3-D,
    with gradients in bf16 or fp32; the momentum buffer `muon_mom` is bf16 (the iteration dtype) and is kept per
    parameter, shaped (E, r, c); the per-row modes keep `scale_v`, (E, r) fp32.  Same-shape parameters of a group are
    orthogonalised together as one stack."""

    DEFAULT_NS_DTYPE = torch.bfloat16

    def __init__(self, params, lr=3e-4, momentum=0.95, nesterov=True, weight_decay=0.0, coeffs=DSV4_COEFFS,
                 ns_dtype=None, scale_mode="aurora", ns_batch_elems=64 * 1024 * 1024, use_graph=False, graph_warmup=3,
                 aurora_k=None, spectral_wd=0.0, swd_beta=0.99, xorth_post=0.0, xorth_backend="ns", xorth_ns_iters=18,
                 xorth_ema=0.95, xorth_gate_ref=0.3, xorth_warmup_steps=0, xorth_where="post"):
        # the reference's argument list (kernels/sm75/muon.py:112-118).  ns_batch_elems caps the elements of one
        # batched stack of same-shape parameters (the reference defaults to 4M for a 16 GB T4; 64M here = 128 MB of
        # bf16 per buffer); swd_beta and the xorth_* details are accepted and unused: they only act together with
        # options that are rejected below.
        if scale_mode not in SCALE_MODES:
            raise ValueError(f"unknown scale_mode {scale_mode!r}; choose from {SCALE_MODES}")
        aurora_k = 1 if aurora_k is None else int(aurora_k)
        if aurora_k < 1:
            raise ValueError("aurora_k must be at least 1")
        if spectral_wd != 0 or xorth_post != 0:
            raise ValueError("spectral_wd and xorth_post are not built here")
        ns_dtype = self.DEFAULT_NS_DTYPE if ns_dtype is None else ns_dtype
        if ns_dtype != torch.bfloat16:
            raise ValueError(f"the iteration runs in bfloat16 only, got ns_dtype={ns_dtype}")
        super().__init__(params, dict(lr=lr, momentum=momentum, nesterov=nesterov, weight_decay=weight_decay,
                                      xorth_post=0.0))
        self.coeffs, self.ns_dtype, self.scale_mode, self.aurora_k = coeffs, ns_dtype, scale_mode, aurora_k
        self.ns_batch_elems = int(ns_batch_elems)
        # CUDA-graph mode (kernels/sm75/muon.py:317-352): gradients are copied into persistent staging buffers
        # eagerly, the rest of the step is captured once after `graph_warmup` eager steps and replayed.  As in the
        # reference the hyper-parameters are baked into the captured step: call set_graph(True) again after a change.
        self.use_graph, self.graph_warmup = bool(use_graph), max(1, int(graph_warmup))
        self._graph, self._gstep, self._graph_failed = None, 0, False

    def set_graph(self, enabled):
        """Toggle the graph mode and drop a captured graph (kernels/sm75/muon.py:354-358)."""
        self.use_graph = bool(enabled)
        self._graph, self._gstep, self._graph_failed = None, 0, False

    @torch.no_grad()
    def step(self, closure=None):
        loss = None
        if closure is not None:
            with torch.enable_grad():
                loss = closure()
        if self.use_graph:
            self._graph_step()
        else:
            self._eager_step(lambda p: p.grad)
        return loss

    # ------------------------------------------------------------------ graph mode
    def _graph_step(self):
        staged = {}
        for group in self.param_groups:
            for p in group["params"]:
                if p.grad is None or p.dim() not in (2, 3):
                    continue
                st = self.state[p]
                buf = st.get("graph_grad")
                if buf is None or buf.shape != p.grad.shape or buf.dtype != p.grad.dtype:
                    if self._graph is not None:
                        raise RuntimeError("the set of stepped parameters changed after the step was captured; "
                                           "call set_graph(True) to capture again")
                    buf = st["graph_grad"] = torch.empty_like(p.grad, memory_format=torch.contiguous_format)
                buf.copy_(p.grad)                       # always eager: reads whatever tensor holds the gradient now
                staged[p] = buf
        if self._graph is not None:
            self._graph.replay()
            return
        self._gstep += 1
        if self._gstep <= self.graph_warmup or self._graph_failed:
            self._eager_step(lambda p: staged.get(p))
            return
        try:
            g = torch.cuda.CUDAGraph()
            torch.cuda.synchronize()
            with torch.cuda.graph(g):
                self._eager_step(lambda p: staged.get(p))      # recorded, not executed
            self._graph = g
            g.replay()                                          # this step's work
        except Exception as exc:                                # degrade to the eager step, as the reference does
            self._graph, self._graph_failed = None, True
            import warnings
            warnings.warn(f"FusedMuon: CUDA-graph capture failed ({type(exc).__name__}: {exc}); stepping eagerly")
            self._eager_step(lambda p: staged.get(p))

    # ------------------------------------------------------------------ the step
    def _eager_step(self, grad_of):
        for group in self.param_groups:
            lr, mu, wd, nesterov = group["lr"], group["momentum"], group["weight_decay"], group["nesterov"]
            if group.get("xorth_post", 0.0) != 0:               # a group-level option in the reference (:119-124)
                raise ValueError("xorth_post (cross-expert whitening) is not built here")
            # Same-shape parameters are orthogonalised as ONE stack (the reference's batched-state design,
            # kernels/sm75/muon.py:215-248): a 2-D parameter contributes one matrix, a 3-D one its E matrices.  Chunks
            # are capped at ns_batch_elems elements with parameters kept whole, as in the reference (:239-247).
            buckets = {}
            for p in group["params"]:
                if grad_of(p) is None or p.dim() not in (2, 3):  # as the reference: other shapes are not stepped
                    continue
                buckets.setdefault((p.shape[-2], p.shape[-1], p.device), []).append(p)
            for (r, c, _dev), ps in buckets.items():
                cap = max(1, self.ns_batch_elems // (r * c))
                chunk, n = [], 0
                for p in ps:
                    n_p = p.numel() // (r * c)
                    if chunk and n + n_p > cap:
                        self._step_chunk(chunk, n, r, c, lr, mu, wd, nesterov, grad_of)
                        chunk, n = [], 0
                    chunk.append(p)
                    n += n_p
                if chunk:
                    self._step_chunk(chunk, n, r, c, lr, mu, wd, nesterov, grad_of)

    def _momentum_stack(self, ps, n, r, c, mu, nesterov, grad_of):
        """u (n, r, c) bf16 = the momentum (+ Nesterov) of the parameters `ps` gathered into one stack, and the
        spans (parameter, first matrix, matrices) inside it (kernels/sm75/muon.py:386-390)."""
        dev = ps[0].device
        u = torch.empty(n, r, c, dtype=torch.bfloat16, device=dev)
        off, spans = 0, []
        for p in ps:
            E, _, _ = _check_stack("parameter", p)
            g = grad_of(p)
            L.require(p.is_contiguous(), "parameters must be contiguous")
            L.require(p.dtype in (torch.bfloat16, torch.float32) and g.dtype in (torch.bfloat16, torch.float32),
                      f"parameters and gradients must be bfloat16 or float32, got {p.dtype} / {g.dtype}")
            st = self.state[p]
            if "muon_mom" not in st:
                st["muon_mom"] = torch.zeros(E, r, c, dtype=torch.bfloat16, device=dev)
            st["muon_mom"] = _checked_momentum(st["muon_mom"], E, r, c, dev)
            _momentum(g.contiguous(), st["muon_mom"], mu, nesterov, out=u[off:off + E])
            spans.append((p, off, E))
            off += E
        return u, spans

    def _row_state(self, spans, r, dev):
        """The (n, r) fp32 EMA of the per-row modes for this stack, gathered from the parameters' `scale_v`."""
        vs = []
        for p, _o, E in spans:
            st = self.state[p]
            v = st.get("scale_v")
            if not torch.is_tensor(v) or v.numel() != E * r:
                if v is not None:
                    raise ValueError(f"optimizer state 'scale_v' has {tuple(getattr(v, 'shape', ()))}, needs ({E}, {r})")
                v = torch.zeros(E, r, dtype=torch.float32, device=dev)
            st["scale_v"] = v = v.to(device=dev, dtype=torch.float32).contiguous().view(E, r)
            vs.append(v)
        return vs[0] if len(vs) == 1 else torch.cat(vs)

    def _store_row_state(self, spans, v):
        if len(spans) > 1:
            for p, o, E in spans:
                self.state[p]["scale_v"].copy_(v[o:o + E])

    def _aurora_passes(self, u, n, r, c):
        """K times {rows divided by their norm, times sqrt(min(r,c)/r), orthogonalised}
        (kernels/muon/muon_scaling.py:101-120; the Frobenius normalisation in front cancels).  Returns the packed
        iterate."""
        tgt = (min(r, c) / r) ** 0.5
        X = Rp = tall = None
        for k in range(self.aurora_k):
            if k > 0:
                u = _unpack(X, n, r, c, Rp, tall)
            pre, rowss = _prescale_rows(u, _row_sumsq(u, n * r, c), n * r, c, tgt)
            X, Rp, tall = _orthogonalise_packed(pre, n, r, c, self.coeffs, 1e-7, rowss)
        return X, Rp, tall

    def _step_chunk(self, ps, n, r, c, lr, mu, wd, nesterov, grad_of):
        """One stack of n matrices (r, c) gathered from the parameters `ps`."""
        u, spans = self._momentum_stack(ps, n, r, c, mu, nesterov, grad_of)
        dev, mode = u.device, self.scale_mode
        decay = 1.0 - lr * wd
        gain = RMS_TARGET * max(r, c) ** 0.5                      # kernels/muon/muon_scaling.py:79-83, 99-100
        if mode == "polar":
            X, Rp, tall = _orthogonalise_packed(u, n, r, c, self.coeffs, 1e-7)
            for p, o, E in spans:
                _apply(X[o:o + E], E, r, c, Rp, tall, 1.0, decay, -lr * gain, p)
        elif mode == "aurora":
            X, Rp, tall = self._aurora_passes(u, n, r, c)
            for p, o, E in spans:
                _apply(X[o:o + E], E, r, c, Rp, tall, gain, decay, -lr, p)
        elif mode == "aurora_ema":                                # kernels/muon/muon_scaling.py:123-143
            v = self._row_state(spans, r, dev)
            rn = _row_sumsq(u, n * r, c).view(n, r).sqrt()
            fro = torch.linalg.vector_norm(rn, dim=-1).clamp_min(ROW_EPS)
            v.mul_(PERROW_BETA2).add_((rn / fro.unsqueeze(-1)).square() / c, alpha=1.0 - PERROW_BETA2)
            self._store_row_state(spans, v)
            mult = ((min(r, c) / r) ** 0.5) / (fro.unsqueeze(-1) * v.sqrt().clamp_min(ROW_EPS))
            pre, rowss = _scale_rows(u, mult.reshape(-1).contiguous(), n * r, c)
            X, Rp, tall = _orthogonalise_packed(pre, n, r, c, self.coeffs, 1e-7, rowss)
            for p, o, E in spans:
                _apply(X[o:o + E], E, r, c, Rp, tall, gain, decay, -lr, p)
        else:                                                     # per-row rescale AFTER the orthogonalisation
            v = self._row_state(spans, r, dev)
            if mode == "normuon":                                 # kernels/muon/muon_scaling.py:166-195
                X, Rp, tall = _orthogonalise_packed(u, n, r, c, self.coeffs, 1e-7)
                O = _unpack(X, n, r, c, Rp, tall)
                rn2 = _row_sumsq(O, n * r, c).view(n, r)
                v.mul_(PERROW_BETA2).add_(rn2 / c, alpha=1.0 - PERROW_BETA2)
                inv = 1.0 / (v.sqrt() + ROW_EPS)
            else:                                                 # aurora_ema_v2, kernels/muon/muon_scaling.py:146-163
                X, Rp, tall = self._aurora_passes(u, n, r, c)
                O = _unpack(X, n, r, c, Rp, tall, gain)
                rn2 = _row_sumsq(O, n * r, c).view(n, r)
                v.mul_(PERROW_BETA2).add_(rn2 / c, alpha=1.0 - PERROW_BETA2)
                inv = 1.0 / (v.sqrt() + ROW_EPS)
            self._store_row_state(spans, v)
            fro = (rn2 * inv.square()).sum(-1).sqrt().clamp_min(1e-12)
            mult = (inv * (RMS_TARGET * (r * c) ** 0.5 / fro).unsqueeze(-1)).contiguous()
            for p, o, E in spans:
                _update_rows(O[o:o + E], mult[o:o + E].reshape(-1), E * r, c, decay, -lr, p)


class DistributedMuon(FusedMuon):
    """Whole-parameter round-robin Muon for replicated parameters, the reference's `DistributedMuon`
    (kernels/sm75/muon.py:437-533): every rank orthogonalises a size-balanced subset of the parameters (and keeps
    momentum only for those), broadcasts its updates as one packed blob per source rank, and every rank applies all
    updates.  Gradients must already be equal on all ranks (all-reduced, as under DDP).  Expert stacks that are
    SHARDED over the ranks need none of this: each rank steps its own experts with `FusedMuon` and no exchange.
    Scale modes: "polar", "aurora", "normuon" ("aurora_ema*" raise NotImplementedError, as in the reference)."""

    def __init__(self, params, *, process_group=None, **kwargs):
        super().__init__(params, **kwargs)
        if self.scale_mode in ("aurora_ema", "aurora_ema_v2"):
            raise NotImplementedError("scale_mode 'aurora_ema' is only supported by FusedMuon, not DistributedMuon")
        if self.use_graph:
            raise ValueError("DistributedMuon steps eagerly (its broadcasts are not captured)")
        self.pg = process_group
        self._owner = None

    def _ordered(self):
        return [(p, g) for g in self.param_groups for p in g["params"] if p.dim() in (2, 3)]

    @staticmethod
    def _plan(ordered, ws):
        """Greedy least-loaded by element count, the same on every rank (kernels/sm75/muon.py:456-462)."""
        load, owner = [0] * ws, []
        for p, _ in ordered:
            r = min(range(ws), key=lambda i: load[i])
            owner.append(r)
            load[r] += p.numel()
        return owner

    @torch.no_grad()
    def step(self, closure=None):
        import torch.distributed as dist
        loss = None
        if closure is not None:
            with torch.enable_grad():
                loss = closure()
        ws, rank = dist.get_world_size(self.pg), dist.get_rank(self.pg)
        ordered = self._ordered()
        if self._owner is None or len(self._owner) != len(ordered):
            self._owner = self._plan(ordered, ws)
        # 1) the update of every owned parameter, bf16, in the parameter's layout (aurora: gain included)
        upd = {}
        for i, (p, g) in enumerate(ordered):
            if self._owner[i] != rank or p.grad is None:
                continue
            E, r, c = _check_stack("parameter", p)
            u, _ = self._momentum_stack([p], E, r, c, g["momentum"], g["nesterov"], lambda q: q.grad)
            if self.scale_mode == "aurora":
                X, Rp, tall = self._aurora_passes(u, E, r, c)
                upd[i] = _unpack(X, E, r, c, Rp, tall, RMS_TARGET * max(r, c) ** 0.5)
            else:
                X, Rp, tall = _orthogonalise_packed(u, E, r, c, self.coeffs, 1e-7)
                upd[i] = _unpack(X, E, r, c, Rp, tall)
        # 2) one broadcast per source rank of its packed updates; every rank applies them
        for src in range(ws):
            idxs = [i for i in range(len(ordered)) if self._owner[i] == src and ordered[i][0].grad is not None]
            if not idxs:
                continue
            sizes = [ordered[i][0].numel() for i in idxs]
            dev = ordered[idxs[0]][0].device
            blob = (torch.cat([upd[i].reshape(-1) for i in idxs]) if src == rank
                    else torch.empty(sum(sizes), dtype=torch.bfloat16, device=dev))
            dist.broadcast(blob, src=dist.get_global_rank(self.pg, src) if self.pg is not None else src, group=self.pg)
            off = 0
            for i, nel in zip(idxs, sizes):
                p, g = ordered[i]
                E, r, c = _check_stack("parameter", p)
                U = blob[off:off + nel].view(E, r, c)
                off += nel
                lr, decay = g["lr"], 1.0 - g["lr"] * g["weight_decay"]
                if self.scale_mode == "normuon":                  # the per-row rescale runs identically on every rank
                    v = self._row_state([(p, 0, E)], r, p.device)
                    rn2 = _row_sumsq(U, E * r, c).view(E, r)
                    v.mul_(PERROW_BETA2).add_(rn2 / c, alpha=1.0 - PERROW_BETA2)
                    inv = 1.0 / (v.sqrt() + ROW_EPS)
                    fro = (rn2 * inv.square()).sum(-1).sqrt().clamp_min(1e-12)
                    mult, alpha = inv * (RMS_TARGET * (r * c) ** 0.5 / fro).unsqueeze(-1), -lr
                else:
                    mult = torch.ones(E, r, dtype=torch.float32, device=p.device)
                    alpha = -lr if self.scale_mode == "aurora" else -lr * RMS_TARGET * max(r, c) ** 0.5
                _update_rows(U, mult.reshape(-1).contiguous(), E * r, c, decay, alpha, p)
        return loss
