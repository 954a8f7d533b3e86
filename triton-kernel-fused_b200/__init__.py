"""B200 (sm_100a) implementation of the MoE block of IsNoobgrammer/triton-kernel-fused:
sigmoid+bias top-k router, device-side expert permutation, grouped tcgen05 expert GEMMs with
fused SwiGLU, weighted combine — forward and backward — behind the reference's Python callables.
Requires the in-tree libb200moe.so (see _lib.build); there is no CPU or library fallback."""
from ._lib import build, check_status, lib, LIB_PATH, EXPORTED
from .moe import moe, moe_grouped, moe_per_expert, GROUPED_MIN_TOKENS
from .router import fused_mlp_router, FusedMLPRouter, fused_router, FusedConvRouter, router_bias_update
from .layer import MoELayer
from .mxfp8 import moe_mxfp8
from . import ops
from .ops import TILE_M
from .ep import ExpertParallelMoELayer, ep_moe
from . import muon
from .muon import DistributedMuon, FusedMuon, newton_schulz

__all__ = ["moe", "moe_grouped", "moe_per_expert", "GROUPED_MIN_TOKENS", "fused_mlp_router", "fused_router", "FusedConvRouter",
           "FusedMLPRouter", "router_bias_update", "MoELayer", "moe_mxfp8", "ExpertParallelMoELayer", "ep_moe", "FusedMuon", "DistributedMuon", "newton_schulz", "muon", "ops", "build", "lib", "check_status"]
