"""nn.Module wiring of the block: sigmoid+bias router -> experts, shaped like the reference's
example module (examples/moe_usage.py:63-77) with the selection-bias buffer of
.autoresearch/train_grok_moe.py:66-90."""
from __future__ import annotations

import torch
import torch.nn as nn

from .moe import moe
from .mxfp8 import moe_mxfp8
from .router import fused_mlp_router, router_bias_update

__all__ = ["MoELayer"]


class MoELayer(nn.Module):
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
        self.last_counts = None

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
        self.last_counts = counts
        fn = moe_mxfp8 if self.precision == "mxfp8" else moe
        out = fn(flat, idx, w, self.gate_up_proj, self.down_proj, self.act_codes, self.act_params)
        return out.reshape(shape)

    @torch.no_grad()
    def update_bias(self, u, counts=None):
        """Load-balance step: pass the all-reduced counts when running on several ranks."""
        c = self.last_counts if counts is None else counts
        if c is not None:
            router_bias_update(self.bias, c, u)
