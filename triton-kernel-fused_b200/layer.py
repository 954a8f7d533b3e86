"""nn.Module wiring of the block: sigmoid+bias router -> experts, shaped like the reference's
example module (examples/moe_usage.py:63-77) with the selection-bias buffer of
.autoresearch/train_grok_moe.py:66-90."""
from __future__ import annotations

import torch
import torch.nn as nn

from .moe import moe
from .mxfp8 import moe_mxfp8
from .router import fused_mlp_router, router_bias_update

__all__ = ["MoELayer", "LoadBalanceMixin"]


class LoadBalanceMixin:
    """The load-balance loop around the layer, as the reference's training module keeps it
    (.autoresearch/train_grok_moe.py:70,79-80,86-90): `load` accumulates the per-expert counts of every training
    forward since the last bias update; `update_bias(u)` applies b += u * sign(mean(load) - load) on the accumulated
    load and clears it; `load_stats()` is the per-expert telemetry.  With several ranks (`_load_group()` not None)
    the load is summed over the ranks first, so every rank applies the same update."""

    def _init_load(self, E):
        # `load` is a plain attribute, not a registered buffer: it is per-rank bookkeeping between two bias updates,
        # so it stays out of the state dict and a DistributedDataParallel wrapper does not overwrite it with rank 0's
        self._load_experts = int(E)
        self.load = None
        self.last_counts = None

    def _load_tensor(self, device=None):
        if device is None:      # wherever it already lives, else beside the selection bias
            device = self.load.device if self.load is not None else getattr(getattr(self, "bias", None), "device", "cpu")
        if self.load is None or self.load.device != torch.device(device):
            old = self.load
            self.load = torch.zeros(self._load_experts, dtype=torch.int64, device=device)
            if old is not None:
                self.load += old.to(device)
        return self.load

    def _load_group(self):
        return None            # (group,) for layers whose counts are per rank; None = this process sees every token

    def _record_counts(self, counts):
        self.last_counts = counts
        if self.training and counts is not None:
            self._load_tensor(counts.device).add_(counts)

    def _global_load(self, counts=None):
        if counts is not None:
            return counts
        c = self._load_tensor().clone()
        g = self._load_group()
        if g is not None:
            import torch.distributed as dist
            dist.all_reduce(c, group=g[0])
        return c

    @torch.no_grad()
    def update_bias(self, u, counts=None):
        """Load-balance step on the load accumulated since the last call (or on `counts`, already global, when
        given).  No forward since the last call: nothing happens."""
        if counts is None and self.last_counts is None:
            return
        router_bias_update(self.bias, self._global_load(counts), u)
        self._load_tensor().zero_()
        self.last_counts = None if counts is None else self.last_counts

    @torch.no_grad()
    def load_stats(self):
        """Per-expert load since the last bias update (global over the ranks): the counts and the figures a training
        loop logs.  Reads the device (one synchronising copy)."""
        c = self._global_load().double().cpu()
        total, E = float(c.sum()), c.numel()
        mean = total / E if E else 0.0
        return {"load": c.long().tolist(), "tokens_routed": int(total),
                "max_over_mean": float(c.max() / mean) if mean > 0 else 0.0,
                "min_over_mean": float(c.min() / mean) if mean > 0 else 0.0,
                "cv": float(c.std(unbiased=False) / mean) if mean > 0 else 0.0,
                "idle_experts": int((c == 0).sum())}


class MoELayer(LoadBalanceMixin, nn.Module):
    def __init__(self, H, I, E, top_k=2, norm_topk_prob=True, routed_scaling_factor=1.0, init_std=0.02,
                 precision="bf16", act_codes=None, learnable_situ=False):
        """act_codes: one activation code per expert (default all 0 = SiLU-GLU); Identity (3) / Zero (4)
        experts come last and carry no weights.  learnable_situ adds an (E,2) [alpha,gamma] parameter
        for the code-5 experts."""
        super().__init__()
        if precision not in ("bf16", "mxfp8"):
            raise ValueError("precision must be 'bf16' or 'mxfp8'")
        self.precision = precision
        codes = [0] * E if act_codes is None else [int(c) for c in act_codes]
        if len(codes) != E:
            raise ValueError("act_codes needs one code per expert")
        n_glu = sum(1 for c in codes if c not in (3, 4))
        self.gate = nn.Linear(H, E, bias=False)
        self.gate_up_proj = nn.Parameter(torch.randn(n_glu, 2 * I, H) * init_std)
        self.down_proj = nn.Parameter(torch.randn(n_glu, H, I) * init_std)
        self.act_params = nn.Parameter(torch.ones(E, 2)) if learnable_situ else None
        with torch.no_grad():
            self.gate.weight.normal_(0.0, init_std)
        self.register_buffer("act_codes", torch.tensor(codes, dtype=torch.int32))
        self.register_buffer("bias", torch.zeros(E, dtype=torch.float32))
        self.top_k = top_k
        self.num_experts = E
        self.norm_topk_prob = norm_topk_prob
        self.routed_scaling_factor = routed_scaling_factor
        self._init_load(E)

    def _apply(self, fn, *a, **kw):
        super()._apply(fn, *a, **kw)
        self.bias.data = self.bias.data.float()        # the selection bias stays fp32
        if self.act_params is not None:
            self.act_params.data = self.act_params.data.float()
        return self

    def forward(self, x):                               # x: (B,S,H) or (N,H)
        shape = x.shape
        flat = x.reshape(-1, shape[-1])
        idx, w, counts = fused_mlp_router(flat, self.gate.weight, self.bias, self.top_k, self.num_experts,
                                          self.norm_topk_prob, self.routed_scaling_factor, return_counts=True)
        self._record_counts(counts)
        fn = moe_mxfp8 if self.precision == "mxfp8" else moe
        out = fn(flat, idx, w, self.gate_up_proj, self.down_proj, self.act_codes, self.act_params)
        return out.reshape(shape)
