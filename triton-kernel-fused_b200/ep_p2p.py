"""Expert-parallel exchange over peer memory: the payload of dispatch and combine never goes through
a library collective or a staging buffer.  Owners PULL token rows from the home ranks' buffers while
gathering them into their padded expert layout; home ranks PULL expert outputs while combining.
Buffers that peers read live in one symmetric allocation per layer (torch symmetric memory gives
the peer mappings and the cross-rank barrier); the kernels are in csrc/ep.cu.

Two ways to bring results home: `exchange="push"` (default) fuses the transfer into the producing GEMM -- the
epilogue of the down projection (forward) and of the gate/up dgrad (backward) sends every output row to its
slot of the home rank's receive buffer, tile by tile while the GEMM runs, and the home rank combines locally;
`exchange="pull"` keeps the rows on the owner and lets the home ranks pull them while combining.

`expert_groups` > 1 (push exchange) splits the rank's local experts into that many groups of about equal rows and
pipelines them: the rows of group g+1 are pulled on a few SMs (`overlap_sms`, one 1024-thread CTA each, on a
stream of its own) while the gate/up GEMM of group g runs on the others, and likewise the grad_out rows of group
g+1 beside the GLU-backward GEMM of group g; only the pull of the first group is exposed.  Off by default: on
8 GPUs at the benchmark's layer the two extra GEMM launches and the SMs the GEMMs give up cost more than the hidden
half of the pulls saves (a pull confined to 16-24 SMs keeps too few loads in flight to fill NVLink).

`capacity_factor` (push exchange) sizes the local buffers once, for that multiple of a rank's own routed rows, and
drops the forward's host wait: nothing is read back, the host runs ahead of the GPU for the whole step.  A routing
decision that sends more rows to some rank than that is not truncated: `b200moe_ep_plan` raises status 8 on every
rank, the step computes nothing, and `check_status` reports it.

Per step and direction there is one tiny NCCL all-gather (the (W,E) count matrix, which also orders
the phases), one host read of that matrix (to size the local buffers) and two device-side barriers
(`b200moe_ep_barrier`: flag words in the symmetric buffer, plain peer stores and bounded local waits).
Constraint: one forward/backward in flight per workspace, because the symmetric buffers are reused.
"""
from __future__ import annotations

import os

import torch
import torch.distributed as dist

from . import _lib as L
from . import ops
from .moe import _amp_cast


@ops._op("ep_plan", 1)
def _plan(*a):
    L.check(L.lib().b200moe_ep_plan(*a))


@ops._op("ep_publish", 1)
def _publish(*a):
    L.check(L.lib().b200moe_ep_publish(*a))


@ops._op("ep_gather_pull", 1)
def _gather_pull(*a):
    L.check(L.lib().b200moe_ep_gather_pull(*a))


@ops._op("ep_combine_pull", 1)
def _combine_pull(*a):
    L.check(L.lib().b200moe_ep_combine_pull(*a))


@ops._op("ep_combine_bwd_pull", 1)
def _combine_bwd_pull(*a):
    L.check(L.lib().b200moe_ep_combine_bwd_pull(*a))


@ops._op("expert_linear_push", 1)
def _linear_push(*a):
    L.check(L.lib().b200moe_expert_linear_push(*a))


@ops._op("slot_dots", 1)
def _slot_dots(*a):
    L.check(L.lib().b200moe_slot_dots(*a))


# SM clocks a rank waits for its peers at a barrier before it gives up with status 7 (about 10 s; ranks reach a
# barrier within microseconds of each other once a step is under way, the margin is for a peer delayed on its host)
BARRIER_LIMIT_CYCLES = int(float(os.environ.get("B200MOE_EP_BARRIER_LIMIT_S", "10")) * 1.9e9)


@ops._op("ep_barrier", 1)
def _barrier(ws):
    """Bounded cross-rank barrier on the workspace's flag words (csrc/ep.cu ep_barrier_kernel): a peer that never
    arrives raises the status word (read by `check_status`) instead of hanging the GPU."""
    ws.barrier_generation += 1
    L.check(L.lib().b200moe_ep_barrier(ws.peers["flags"], ws.W, ws.rank, ws.barrier_generation & 0xFFFFFFFF,
                                       BARRIER_LIMIT_CYCLES, L.ptr(L.status_word(ws.buf.device)),
                                       torch.cuda.current_stream(ws.buf.device).cuda_stream))


def _align(n, a=256):
    return (n + a - 1) // a * a


def fixed_capacity_rows(W, T, k, capacity_factor):
    """Routed rows the fixed-capacity buffers of one rank are sized for: capacity_factor times the rank's own routed
    rows (T * k), rounded up, never more than the W * T * k rows that exist."""
    cf = float(capacity_factor)
    if not cf > 0:
        raise ValueError("capacity_factor must be positive")
    M = int(T) * int(k)
    return min(int(W) * M, int(-(-cf * M // 1)))


def expert_groups(ends, n):
    """Split local experts 0..len(ends)-1 into at most `n` runs of consecutive experts with about equal padded rows.
    ends[j] = padded row at which expert j ends.  Returns [(e_lo, e_hi, row_lo, row_hi)], empty runs left out."""
    import bisect
    El, total = len(ends), (ends[-1] if ends else 0)
    cuts = [0]
    for g in range(1, max(1, int(n))):
        j = bisect.bisect_left(ends, total * g / n) + 1      # first cut at or behind the g-th share of the rows
        cuts.append(min(max(j, cuts[-1]), El))
    cuts.append(El)
    starts = [0] + list(ends)
    return [(lo, hi, starts[lo], starts[hi]) for lo, hi in zip(cuts, cuts[1:]) if starts[hi] > starts[lo]]


def _pipelined(ws, groups, pull, gemm):
    """pull(e_lo, e_hi, max_sms, stream) / gemm(g, grp): group 0 is pulled by the whole GPU on the current stream,
    the others on `ws.overlap_sms` SMs on the side stream, each beside the GEMMs of the groups before it, which
    leave those SMs free."""
    dev = ws.buf.device
    main, side = torch.cuda.current_stream(dev), ws.side_stream
    pull(groups[0][0], groups[0][1], 0, main.cuda_stream)
    start, arrived = ws.pipe_events[0], ws.pipe_events[1:]
    start.record(main)
    side.wait_event(start)
    for g, (e_lo, e_hi, _, _) in enumerate(groups[1:]):
        pull(e_lo, e_hi, ws.overlap_sms, side.cuda_stream)
        arrived[g].record(side)
    try:
        for g, grp in enumerate(groups):
            if g > 0:
                main.wait_event(arrived[g - 1])
            # the last GEMM starts when the last pull is over and takes every SM
            L.check(L.lib().b200moe_set_reserved_sms(ws.overlap_sms if g + 1 < len(groups) else 0))
            gemm(g, grp)
    finally:
        L.check(L.lib().b200moe_set_reserved_sms(0))


class SymmetricWorkspace:
    """One symmetric allocation carved into the buffers peers read.  Sized for the worst case
    (every routed row of every rank lands on one rank), so it is allocated once."""

    def __init__(self, T, H, k, E, group, device, overlap_sms=0, exchange="push", expert_groups=1,
                 capacity_factor=None):
        """exchange="pull", overlap_sms > 0: in the backward pass the last pull (grad_hidden) runs on that many SMs
        beside the weight-gradient GEMMs, which leave them free and run on a high-priority stream of their own.
        exchange="push", expert_groups > 1: the dispatch-side pulls are pipelined against the GEMMs by groups of
        local experts, on overlap_sms SMs (default 16)."""
        import torch.distributed._symmetric_memory as symm
        if exchange not in ("push", "pull"):
            raise ValueError("exchange must be 'push' or 'pull'")
        self.exchange = exchange
        self.expert_groups = max(1, int(expert_groups)) if exchange == "push" else 1
        if exchange == "pull":
            self.overlap_sms = int(overlap_sms)
        else:
            self.overlap_sms = (int(overlap_sms) or 16) if self.expert_groups > 1 else 0
        self.gemm_stream = torch.cuda.Stream(device=device, priority=-1) if exchange == "pull" and self.overlap_sms > 0 else None
        # fixed-capacity buffers: rows (a multiple of the tile) every step's local buffers have; None = sized per step
        self.rows_fixed = None
        if capacity_factor is not None:
            if exchange != "push" or self.expert_groups > 1:
                raise ValueError("capacity_factor needs exchange='push' and expert_groups=1")
            W_ = dist.get_world_size(group)
            self.rows_fixed = L.padded_rows_cap(fixed_capacity_rows(W_, T, k, capacity_factor), E // W_)
        self.side_stream = torch.cuda.Stream(device=device) if self.expert_groups > 1 else None
        self.pipe_events = [torch.cuda.Event() for _ in range(self.expert_groups)] if self.expert_groups > 1 else []
        self.group = group
        self.W = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.T, self.H, self.k, self.E = T, H, k, E
        M = T * k
        self.cap_w = L.padded_rows_cap(self.W * M, E // self.W)
        W = self.W
        # x / go: payload rows that peers pull.  tab_*: replicas of EVERY rank's routing tables ([W][M] idx, slot_pos,
        # routing weight; [W][E+1] offs), written by the owners of the tables (b200moe_ep_publish) so that the pull
        # kernels resolve rows from local memory
        self.slot_stride, self.offs_stride = _align(M, 4), _align(E + 1, 4)     # elements: every replica 16-byte aligned
        Ms, Es = self.slot_stride, self.offs_stride
        fields = [("flags", 16 * 4), ("x", T * H * 2), ("go", T * H * 2), ("tab_idx", W * Ms * 8), ("tab_spos", W * Ms * 4),
                  ("tab_w", W * Ms * 4), ("tab_offs", W * Es * 4)]
        if exchange == "pull":     # owners keep their result rows; sized for every routed row landing on one rank
            fields += [("eo", self.cap_w * H * 2), ("gxs", self.cap_w * H * 2), ("gw", self.cap_w * 4)]
        else:                      # home ranks receive the result rows of their own slots
            fields += [("recv", M * H * 2), ("recvg", M * H * 2)]
        self.offsets, total = {}, 0
        for name, nbytes in fields:
            self.offsets[name] = total
            total += _align(nbytes)
        self.buf = symm.empty(total, dtype=torch.uint8, device=device)
        self.handle = symm.rendezvous(self.buf, group if group is not None else dist.group.WORLD)
        base = [int(p) for p in self.handle.buffer_ptrs]
        self.peers = {name: L.ptr_table([b + off for b in base]) for name, off in self.offsets.items()}
        v = lambda name, n, dt: self.buf[self.offsets[name]: self.offsets[name] + n * dt.itemsize].view(dt)
        self.x = v("x", T * H, torch.bfloat16).view(T, H)
        self.go = v("go", T * H, torch.bfloat16).view(T, H)
        # host arrays of W pointers into THIS rank's replicas: entry s = the table rank s published here
        mine = base[self.rank]
        self.tabs = {name: L.ptr_table([mine + self.offsets[name] + s * stride for s in range(W)])
                     for name, stride in (("tab_idx", Ms * 8), ("tab_spos", Ms * 4), ("tab_w", Ms * 4), ("tab_offs", Es * 4))}
        if exchange == "pull":
            self.eo = v("eo", self.cap_w * H, torch.bfloat16).view(self.cap_w, H)
            self.gxs = v("gxs", self.cap_w * H, torch.bfloat16).view(self.cap_w, H)
            self.gw = v("gw", self.cap_w, torch.float32)
        else:
            self.recv = v("recv", M * H, torch.bfloat16).view(M, H)
            self.recvg = v("recvg", M * H, torch.bfloat16).view(M, H)
            # device arrays of the peers' receive-buffer addresses, read by the pushing GEMM epilogues
            self.recv_base = torch.tensor([b + self.offsets["recv"] for b in base], dtype=torch.int64, device=device)
            self.recvg_base = torch.tensor([b + self.offsets["recvg"] for b in base], dtype=torch.int64, device=device)
            self.ident = torch.arange(M, dtype=torch.int32, device=device)   # slot -> row of the receive buffers
        self.generation = 0
        self.rows_host = torch.zeros(1 + E // W, dtype=torch.int32).pin_memory()   # written by ep_local_rows_kernel
        self.rows_event = torch.cuda.Event()
        # barrier flags: one word per peer, zero before the first barrier on every rank (the rendezvous below is the
        # one library barrier of the workspace's life: nobody announces itself into an array that is still being zeroed)
        self.flags = v("flags", 16, torch.int32)
        self.flags.zero_()
        self.barrier_generation = 0
        torch.cuda.synchronize(device)
        dist.barrier(group=group)

    def barrier(self):
        _barrier(self)


def _backward_push(ctx, grad_out, grad_eo):
    """Backward of the push exchange (the barrier that put grad_out / w in place has been issued)."""
    idx, x_s, gate_up, inter, w32, gate_up_local, down_local = ctx.saved_tensors
    ws, perm_l = ctx.ws, ctx.perm_l
    _, src_base, row_rank, row_slot = ctx.tables
    W, E, T, H, k = ws.W, ws.E, ws.T, ws.H, ws.k
    El, cap_l = E // W, perm_l.cap
    dev = x_s.device
    st = L.stream_of(x_s)
    status = L.ptr(L.status_word(dev))
    # the expert outputs of this rank's tokens are still in its receive buffer: grad of the routing weights
    grad_w = torch.empty(T, k, dtype=torch.float32, device=dev)
    _slot_dots(L.ptr(ws.go), L.ptr(ws.recv), T, k, H, L.ptr(grad_w), st)

    def pull(e_lo, e_hi, max_sms, stream):
        _combine_bwd_pull(ws.peers["go"], ws.tabs["tab_w"], ws.tabs["tab_idx"], ws.tabs["tab_spos"], ws.tabs["tab_offs"],
                          None, L.ptr(perm_l.counts), L.ptr(perm_l.poffs), L.ptr(src_base), W, ws.rank, E, e_lo, e_hi,
                          max_sms, T, k, H, L.ptr(grad_eo), None, stream)

    if len(ctx.groups) > 1:
        grad_gu = torch.empty(cap_l, gate_up.shape[1], dtype=torch.bfloat16, device=dev)
        _pipelined(ws, ctx.groups, pull, lambda g, grp: ops.expert_down_dgrad_glu(
            grad_eo, down_local, gate_up, perm_l, out=grad_gu, rows=grp[2:]))
    else:
        pull(0, El, 0, st)
        grad_gu = ops.expert_down_dgrad_glu(grad_eo, down_local, gate_up, perm_l)
    # gate/up dgrad whose epilogue sends each grad_x row to its slot at the token's home rank
    twoI = gate_up_local.shape[1]
    _linear_push(L.ptr(grad_gu), L.ptr(gate_up_local), 1, L.ptr(perm_l.tile_expert), L.ptr(perm_l.poffs), cap_l, El, H,
                 twoI, L.ptr(row_rank), L.ptr(row_slot), L.ptr(ws.recvg_base), status, st)
    grad_down = ops.expert_wgrad(grad_eo, inter, perm_l)
    grad_gate_up = ops.expert_wgrad(grad_gu, x_s, perm_l)
    ws.barrier()                                                    # every owner's grad_x rows have arrived
    grad_hidden = ops.combine_raw(ws.recvg, None, ws.ident, T, k)
    return grad_hidden, None, grad_w.to(ctx.wt_dtype), grad_gate_up, grad_down, None


class _ExpertParallelP2P(torch.autograd.Function):
    @staticmethod
    def forward(ctx, hidden, idx, wt, gate_up_local, down_local, ws: SymmetricWorkspace):
        hidden, gate_up_local, down_local = _amp_cast(hidden, gate_up_local, down_local)
        for name, t in (("hidden", hidden), ("gate_up_proj", gate_up_local), ("down_proj", down_local)):
            L.require_cuda_bf16(name, t)
        W, rank, E = ws.W, ws.rank, ws.E
        El = E // W
        T, H = hidden.shape
        k = idx.shape[1]
        L.require((T, H, k) == (ws.T, ws.H, ws.k), f"workspace was built for T,H,k = {(ws.T, ws.H, ws.k)}, got {(T, H, k)}")
        L.require(gate_up_local.shape[0] == El and down_local.shape[0] == El, f"this rank must hold {El} experts")
        dev = hidden.device
        st = L.stream_of(hidden)
        i32 = dict(dtype=torch.int32, device=dev)
        idx = idx.contiguous()
        w32 = wt.detach().float().contiguous()
        gate_up_local, down_local = gate_up_local.contiguous(), down_local.contiguous()

        perm = ops.permute_build(idx, E, want_order=True)   # slot_pos comes with the order tables
        ws.x.copy_(hidden)
        # routing tables (and the routing weights the backward needs) go to every rank's replicas
        _publish(L.ptr(idx), L.ptr(perm.slot_pos), L.ptr(w32), L.ptr(perm.offs), T * k, E, W, rank, ws.slot_stride,
                 ws.offs_stride, ws.peers["tab_idx"],
                 ws.peers["tab_spos"], ws.peers["tab_w"], ws.peers["tab_offs"], st)
        counts_all = torch.empty(W, E, **i32)
        # the count exchange is also the ordering point: behind it every rank's x is in place and every table replica
        # has arrived (each rank's contribution is sent after its own copies and stores in stream order)
        dist.all_gather_into_tensor(counts_all, perm.counts, group=ws.group)
        # the one host wait of the step: a kernel stores the row count into pinned host memory and the host waits
        # for an event behind it (a .item() would be a device-to-host copy, and that copy queues behind any large
        # transfer the caller's input pipeline has on the copy engines)
        if ws.rows_fixed is None:
            L.check(L.lib().b200moe_ep_local_rows(L.ptr(counts_all), W, rank, E, ws.rows_host.data_ptr(), st))
            ws.rows_event.record(torch.cuda.current_stream(dev))
            ws.rows_event.synchronize()
            words = ws.rows_host.tolist()
            R = words[0]
            groups = expert_groups(words[1:], ws.expert_groups) if ws.expert_groups > 1 else []
            cap_l = L.padded_rows_cap(R, El)
        else:               # buffers of a fixed size: no host wait; the plan kernel checks that the rows fit
            R, groups, cap_l = 0, [], ws.rows_fixed
        poffs_l = torch.empty(El + 1, **i32)
        counts_l = torch.empty(El, **i32)
        tile_expert_l = torch.empty(cap_l // ops.TILE_M, **i32)
        src_base = torch.empty(W * El, **i32)
        dest_base = torch.empty(E, **i32)
        _plan(L.ptr(counts_all), W, rank, E, L.ptr(poffs_l), L.ptr(counts_l), L.ptr(tile_expert_l), L.ptr(src_base),
              L.ptr(dest_base), cap_l if ws.rows_fixed is not None else 0, L.ptr(L.status_word(dev)), st)
        x_s = torch.empty(cap_l, H, dtype=torch.bfloat16, device=dev)
        push = ws.exchange == "push"
        row_rank = torch.empty(cap_l, **i32) if push else None
        row_slot = torch.empty(cap_l, **i32) if push else None

        def pull(e_lo, e_hi, max_sms, stream):
            _gather_pull(ws.peers["x"], ws.tabs["tab_idx"], ws.tabs["tab_spos"], ws.tabs["tab_offs"], L.ptr(counts_l),
                         L.ptr(poffs_l), L.ptr(src_base), W, rank, E, e_lo, e_hi, max_sms, T, k, H, L.ptr(x_s),
                         L.ptr(row_rank), L.ptr(row_slot), stream)

        perm_l = ops.Permutation(R, 1, El, cap_l, counts_l, None, poffs_l, None, None, tile_expert_l, None, None)
        if len(groups) > 1:
            twoI = gate_up_local.shape[1]
            gate_up = torch.empty(cap_l, twoI, dtype=torch.bfloat16, device=dev)
            inter = torch.empty(cap_l, twoI // 2, dtype=torch.bfloat16, device=dev)
            _pipelined(ws, groups, pull, lambda g, grp: ops.expert_gate_up_swiglu(
                x_s, gate_up_local, perm_l, out=(gate_up, inter), rows=grp[2:]))
        else:
            groups = []
            pull(0, El, 0, st)
            gate_up, inter = ops.expert_gate_up_swiglu(x_s, gate_up_local, perm_l)
        status = L.ptr(L.status_word(dev))
        if push:
            # down projection whose epilogue sends each output row to its slot at the token's home rank
            I = down_local.shape[2]
            _linear_push(L.ptr(inter), L.ptr(down_local), 0, L.ptr(tile_expert_l), L.ptr(poffs_l), cap_l, El, H, I,
                         L.ptr(row_rank), L.ptr(row_slot), L.ptr(ws.recv_base), status, st)
            ws.barrier()                                            # every owner's rows have arrived
            out = ops.combine_raw(ws.recv, w32, ws.ident, T, k)
        else:
            ops.expert_down(inter, down_local, perm_l, out=ws.eo[:cap_l])
            ws.barrier()                                            # every owner's eo is complete
            out = torch.empty(T, H, dtype=torch.bfloat16, device=dev)
            _combine_pull(ws.peers["eo"], L.ptr(w32), L.ptr(idx), L.ptr(perm.slot_pos),
                          L.ptr(perm.offs), L.ptr(dest_base), W, E, T, k, H, L.ptr(out), None, None, status, st)
        ws.generation += 1
        ctx.ws, ctx.perm, ctx.perm_l, ctx.gen = ws, perm, perm_l, ws.generation
        ctx.tables = (dest_base, src_base, row_rank, row_slot)
        ctx.groups = groups
        ctx.wt_dtype = wt.dtype
        ctx.save_for_backward(idx, x_s, gate_up, inter, w32, gate_up_local, down_local)
        return out

    @staticmethod
    def backward(ctx, grad_out):
        idx, x_s, gate_up, inter, w32, gate_up_local, down_local = ctx.saved_tensors
        ws, perm, perm_l = ctx.ws, ctx.perm, ctx.perm_l
        dest_base, src_base, row_rank, row_slot = ctx.tables
        if ws.generation != ctx.gen:
            raise RuntimeError("the symmetric workspace was reused by another forward before this backward ran; "
                               "use one workspace per forward in flight")
        W, E = ws.W, ws.E
        T, H, k = ws.T, ws.H, ws.k
        cap_l = perm_l.cap
        dev = x_s.device
        st = L.stream_of(x_s)
        ws.go.copy_(grad_out)
        ws.barrier()                                                # every home rank's grad_out is in place
        grad_eo = torch.empty(cap_l, H, dtype=torch.bfloat16, device=dev)
        if ws.exchange == "push":
            return _backward_push(ctx, grad_out, grad_eo)
        _combine_bwd_pull(ws.peers["go"], ws.tabs["tab_w"], ws.tabs["tab_idx"], ws.tabs["tab_spos"], ws.tabs["tab_offs"],
                          L.ptr(ws.eo), L.ptr(perm_l.counts), L.ptr(perm_l.poffs), L.ptr(src_base), W, ws.rank, E, 0,
                          E // W, 0, T, k, H, L.ptr(grad_eo), L.ptr(ws.gw), st)
        grad_gu = ops.expert_down_dgrad_glu(grad_eo, down_local, gate_up, perm_l)
        grad_hidden = torch.empty(T, H, dtype=torch.bfloat16, device=dev)
        grad_w = torch.empty(T, k, dtype=torch.float32, device=dev)

        def pull_grad_hidden():
            _combine_pull(ws.peers["gxs"], None, L.ptr(idx), L.ptr(perm.slot_pos), L.ptr(perm.offs),
                          L.ptr(dest_base), W, E, T, k, H, L.ptr(grad_hidden), ws.peers["gw"], L.ptr(grad_w),
                          L.ptr(L.status_word(dev)), st)

        if ws.overlap_sms <= 0:
            grad_down = ops.expert_wgrad(grad_eo, inter, perm_l)
            grad_gate_up = ops.expert_wgrad(grad_gu, x_s, perm_l)
            ops.expert_gate_up_dgrad(grad_gu, gate_up_local, perm_l, out=ws.gxs[:cap_l])
            ws.barrier()                                            # every owner's grad_x_s / gw are complete
            pull_grad_hidden()
        else:
            # the dgrad that peers wait for goes first; the pull of grad_hidden then runs on overlap_sms SMs
            # while the two weight-gradient GEMMs run on the others (the pull's CTAs each fill an SM, the GEMMs'
            # persistent grids leave that many SMs out, so neither kernel waits for the other's SMs)
            ops.expert_gate_up_dgrad(grad_gu, gate_up_local, perm_l, out=ws.gxs[:cap_l])
            ws.barrier()
            main, side = torch.cuda.current_stream(dev), ws.gemm_stream
            side.wait_stream(main)
            L.check(L.lib().b200moe_set_reserved_sms(ws.overlap_sms))
            L.check(L.lib().b200moe_set_exchange_sms(ws.overlap_sms))
            try:
                with torch.cuda.stream(side):
                    grad_gate_up = ops.expert_wgrad(grad_gu, x_s, perm_l)
                    grad_down = ops.expert_wgrad(grad_eo, inter, perm_l)
                pull_grad_hidden()
            finally:
                L.check(L.lib().b200moe_set_reserved_sms(0))
                L.check(L.lib().b200moe_set_exchange_sms(0))
            for t_ in (grad_gu, x_s, grad_eo, inter):
                t_.record_stream(side)
            main.wait_stream(side)
            grad_gate_up.record_stream(main)
            grad_down.record_stream(main)
        return grad_hidden, None, grad_w.to(ctx.wt_dtype), grad_gate_up, grad_down, None


def ep_moe_p2p(hidden, top_k_indices, top_k_weights, gate_up_proj_local, down_proj_local, workspace):
    """Expert-parallel `moe` over peer memory; `workspace` is a SymmetricWorkspace of this layer."""
    return _ExpertParallelP2P.apply(hidden, top_k_indices, top_k_weights, gate_up_proj_local, down_proj_local,
                                    workspace)
