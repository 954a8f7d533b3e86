"""Expert-parallel MoE layer: experts are sharded over the ranks of a process group (one process
per GPU), tokens stay on their home rank, and rows travel with two NCCL all-to-alls per direction.

The reference has no expert parallelism (its only collective is a broadcast in its optimizer); the
single-process layer is the specification: the result on the concatenated batch must equal
`MoELayer` holding all E experts.

Forward on every rank
  1. local router over all E experts                       (router kernels)
  2. stable counting sort of the local slots by expert     (permute kernels; compact order = by
     destination rank, then by expert, then by slot)
  3. gather rows into that order, exchange per-expert counts, all-to-all the rows (dispatch)
  4. counting sort of the received rows by local expert, gather into the padded layout
  5. grouped expert GEMMs with fused SwiGLU                 (tcgen05 kernels)
  6. un-permute to arrival order, all-to-all back, weighted combine on the home rank
Backward mirrors it with the same four exchanges.  Received rows always land in this GPU's own
memory first; kernels never read a peer's memory.
"""
from __future__ import annotations

import torch
import torch.distributed as dist
import torch.nn as nn

from . import _lib as L
from . import ops as _cuda_ops
from .moe import _amp_cast
from .layer import LoadBalanceMixin
from .router import fused_mlp_router

__all__ = ["ExpertParallelMoELayer", "ep_moe", "exchange_plan"]


def exchange_plan(counts, world, group=None):
    """Count exchange.  counts (E,) int32 on this rank -> (recv_counts (world, E/world) int32 device,
    send_splits, recv_splits as Python lists).  One small all-to-all and ONE host sync."""
    E = counts.numel()
    if E % world != 0:
        raise ValueError(f"num_experts = {E} must be divisible by the group size {world}")
    El = E // world
    send_counts = counts.view(world, El).contiguous()
    recv_counts = torch.empty_like(send_counts)
    dist.all_to_all_single(recv_counts, send_counts, group=group)
    both = torch.stack([send_counts.sum(1), recv_counts.sum(1)]).cpu()     # the one D2H sync
    return recv_counts, both[0].tolist(), both[1].tolist()


@_cuda_ops._op("all_to_all", 0)
def _a2a(rows, out_rows, out_splits, in_splits, group):
    out = torch.empty(max(out_rows, 1), rows.shape[1], dtype=rows.dtype, device=rows.device)[:out_rows]
    dist.all_to_all_single(out, rows[: sum(in_splits)].contiguous(), out_splits, in_splits, group=group)
    return out


class _ExpertParallelMoE(torch.autograd.Function):
    @staticmethod
    def forward(ctx, hidden, idx, wt, gate_up_local, down_local, group, num_experts, kern):
        hidden, gate_up_local, down_local = _amp_cast(hidden, gate_up_local, down_local)
        world = dist.get_world_size(group)
        T, H = hidden.shape
        k = idx.shape[1]
        El = num_experts // world
        L.require(gate_up_local.shape[0] == El and down_local.shape[0] == El,
                  f"this rank must hold {El} experts, got {gate_up_local.shape[0]}")
        hidden = hidden.contiguous()
        w32 = wt.detach().float().contiguous()
        M = T * k

        perm = kern.permute_build(idx, num_experts, want_order=True)
        send = kern.gather_compact(hidden, perm)                                   # (M,H) by expert
        recv_counts, send_splits, recv_splits = exchange_plan(perm.counts, world, group)
        R = sum(recv_splits)
        recv = _a2a(send, R, recv_splits, send_splits, group)                      # dispatch
        # expert of every received row: source-major, expert-minor, counts from the exchange
        local_ids = torch.arange(El, device=hidden.device).repeat(world)
        recv_e = torch.repeat_interleave(local_ids, recv_counts.flatten().long(), output_size=R)
        perm_l = kern.permute_build(recv_e.view(R, 1), El)
        x_s = kern.gather_rows(recv, perm_l)
        gate_up, inter = kern.expert_gate_up_swiglu(x_s, gate_up_local.contiguous(), perm_l)
        eo = kern.expert_down(inter, down_local.contiguous(), perm_l)
        back_send = kern.combine(eo, None, perm_l)                                  # arrival order
        back = _a2a(back_send, M, send_splits, recv_splits, group)                  # combine exchange
        out = kern.combine_raw(back, w32, perm.slot_pos, T, k)

        ctx.perm, ctx.perm_l, ctx.group, ctx.kern = perm, perm_l, group, kern
        ctx.splits = (send_splits, recv_splits, R, M)
        ctx.wt_dtype = wt.dtype
        ctx.save_for_backward(back, x_s, gate_up, inter, w32, gate_up_local, down_local)
        return out

    @staticmethod
    def backward(ctx, grad_out):
        back, x_s, gate_up, inter, w32, gate_up_local, down_local = ctx.saved_tensors
        perm, perm_l, group, kern = ctx.perm, ctx.perm_l, ctx.group, ctx.kern
        send_splits, recv_splits, R, M = ctx.splits
        grad_out = grad_out.contiguous().to(back.dtype)
        grad_back, grad_w = kern.combine_bwd_raw(grad_out, back, w32, perm.order, perm.offs[perm.E:], perm.k, M)
        recv_g = _a2a(grad_back, R, recv_splits, send_splits, group)
        grad_eo = kern.gather_rows(recv_g, perm_l)
        grad_gu = kern.expert_down_dgrad_glu(grad_eo, down_local.contiguous(), gate_up, perm_l)
        grad_down = kern.expert_wgrad(grad_eo, inter, perm_l)
        grad_gate_up = kern.expert_wgrad(grad_gu, x_s, perm_l)
        grad_x_s = kern.expert_gate_up_dgrad(grad_gu, gate_up_local.contiguous(), perm_l)
        gx_send = kern.combine(grad_x_s, None, perm_l)
        gx_back = _a2a(gx_send, M, send_splits, recv_splits, group)
        grad_hidden = kern.combine_raw(gx_back, None, perm.slot_pos, perm.T, perm.k)
        return grad_hidden, None, grad_w.to(ctx.wt_dtype), grad_gate_up, grad_down, None, None, None


def ep_moe(hidden, top_k_indices, top_k_weights, gate_up_proj_local, down_proj_local, num_experts,
           group=None, _kernels=None):
    """Expert-parallel counterpart of `moe`: indices address all `num_experts` experts, this rank
    holds experts [rank*E/W, (rank+1)*E/W).  `_kernels` swaps the kernel provider (tests only)."""
    return _ExpertParallelMoE.apply(hidden, top_k_indices, top_k_weights, gate_up_proj_local, down_proj_local,
                                    group, num_experts, _cuda_ops if _kernels is None else _kernels)


class ExpertParallelMoELayer(LoadBalanceMixin, nn.Module):
    """Router replicated on every rank, E/W experts per rank.  transport = "nccl" moves rows with
    all_to_all_single; "p2p" uses the peer-memory kernels of csrc/ep.cu (rows are pulled over NVLink
    inside the gather and combine kernels; needs torch symmetric memory and a fixed token count).  Gradients of the replicated router
    weight are local sums: all-reduce them (or wrap the module in DDP) as for any replicated
    parameter; expert gradients are complete on the owning rank."""

    def __init__(self, H, I, E, top_k=2, group=None, norm_topk_prob=True, routed_scaling_factor=1.0, init_std=0.02,
                 overlap_chunks=1, reserved_sms=0, transport="nccl", exchange="push", expert_groups=1,
                 capacity_factor=None):
        """overlap_chunks > 1 splits the local tokens into that many independent pipelines on their own
        CUDA streams, so the all-to-alls of one chunk run while the expert GEMMs of another do;
        reserved_sms keeps that many SMs free of the persistent GEMM kernels for the communication
        kernels (process-wide setting of the library); with transport="p2p" it is the number of SMs on which
        the backward's last pull runs beside the weight-gradient GEMMs (0 = no overlap).
        exchange (transport="p2p" only): "push" = result rows are sent to the home ranks by the epilogues of the
        GEMMs that produce them, "pull" = home ranks fetch them while combining.
        expert_groups (transport="p2p", exchange="push"): > 1 pipelines the dispatch-side pulls against the expert
        GEMMs by that many groups of local experts; the pulls behind the first run on reserved_sms SMs (default 16).
        capacity_factor (same transport and exchange): the local buffers hold that multiple of a rank's own routed
        rows (T * top_k) and the forward no longer waits on the host for the row count; a step that routes more rows
        to a rank computes nothing and raises status 8 (RuntimeError at the next check_status), it is never truncated."""
        super().__init__()
        if transport not in ("nccl", "p2p"):
            raise ValueError("transport must be 'nccl' (all_to_all_single) or 'p2p' (peer-memory kernels)")
        if exchange not in ("push", "pull"):
            raise ValueError("exchange must be 'push' or 'pull'")
        if transport == "p2p" and int(overlap_chunks) > 1:
            # the peer-memory transport keeps ONE symmetric workspace per layer (inputs, routing tables and receive
            # buffers that peers read and write) and allows one forward in flight on it; chunk pipelines on their own
            # streams would overwrite each other's buffers while peers still use them
            raise ValueError("overlap_chunks > 1 needs transport='nccl': the p2p transport has one workspace per "
                             "layer and one forward in flight")
        self.transport = transport
        self.exchange = exchange
        self._workspace = None
        self.overlap_chunks = max(1, int(overlap_chunks))
        self.reserved_sms = int(reserved_sms)
        if int(expert_groups) > 1 and not (transport == "p2p" and exchange == "push"):
            raise ValueError("expert_groups > 1 needs transport='p2p' with exchange='push'")
        self.expert_groups = max(1, int(expert_groups))
        if capacity_factor is not None and not (transport == "p2p" and exchange == "push" and self.expert_groups == 1):
            raise ValueError("capacity_factor needs transport='p2p' with exchange='push' and expert_groups=1")
        self.capacity_factor = capacity_factor
        self._streams = None
        world = dist.get_world_size(group)
        if E % world != 0:
            raise ValueError(f"num_experts = {E} must be divisible by the group size {world}")
        self.group, self.world, self.rank = group, world, dist.get_rank(group)
        self.num_experts, self.local_experts, self.top_k = E, E // world, top_k
        self.gate = nn.Linear(H, E, bias=False)
        with torch.no_grad():
            self.gate.weight.normal_(0.0, init_std)
        self.gate_up_proj = nn.Parameter(torch.randn(self.local_experts, 2 * I, H) * init_std)
        self.down_proj = nn.Parameter(torch.randn(self.local_experts, H, I) * init_std)
        self.register_buffer("bias", torch.zeros(E, dtype=torch.float32))
        self.norm_topk_prob, self.routed_scaling_factor = norm_topk_prob, routed_scaling_factor
        self._init_load(E)

    def _apply(self, fn, *a, **kw):
        super()._apply(fn, *a, **kw)
        self.bias.data = self.bias.data.float()
        return self

    def _load_group(self):
        # counts are those of this rank's tokens: the load-balance step and the telemetry sum them over the ranks
        # (the reference leaves that all-reduce to the caller, kernels/sm75/router.py:293-297)
        return (self.group,)

    def _pipeline(self, flat):
        idx, w, counts = fused_mlp_router(flat, self.gate.weight, self.bias, self.top_k, self.num_experts,
                                          self.norm_topk_prob, self.routed_scaling_factor, return_counts=True)
        if self.transport == "p2p":
            from .ep_p2p import SymmetricWorkspace, ep_moe_p2p
            T, H = flat.shape
            ws = self._workspace
            if ws is None or (ws.T, ws.H, ws.k) != (T, H, self.top_k):
                ws = self._workspace = SymmetricWorkspace(T, H, self.top_k, self.num_experts, self.group, flat.device,
                                                          overlap_sms=self.reserved_sms, exchange=self.exchange,
                                                          expert_groups=self.expert_groups,
                                                          capacity_factor=self.capacity_factor)
            return ep_moe_p2p(flat, idx, w, self.gate_up_proj, self.down_proj, ws), counts
        return ep_moe(flat, idx, w, self.gate_up_proj, self.down_proj, self.num_experts, self.group), counts

    def forward(self, x):
        shape = x.shape
        flat = x.reshape(-1, shape[-1])
        n = self.overlap_chunks
        if n == 1 or flat.shape[0] < n:
            out, counts = self._pipeline(flat)
            self._record_counts(counts)
            return out.reshape(shape)
        if self._streams is None:
            self._streams = [torch.cuda.Stream(device=flat.device) for _ in range(n)]
            L.check(L.lib().b200moe_set_reserved_sms(self.reserved_sms))
        cur = torch.cuda.current_stream(flat.device)
        outs, counts = [], None
        for st, chunk in zip(self._streams, flat.chunk(n)):
            st.wait_stream(cur)
            chunk.record_stream(st)
            with torch.cuda.stream(st):
                o, c = self._pipeline(chunk)
                counts = c if counts is None else counts + c
            o.record_stream(cur)
            outs.append(o)
        for st in self._streams:
            cur.wait_stream(st)
        self._record_counts(counts)
        return torch.cat(outs).reshape(shape)
