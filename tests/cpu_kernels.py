"""TEST INFRASTRUCTURE: a CPU stand-in for the kernel provider of the expert-parallel layer.

`ep_moe(..., _kernels=CpuKernels)` lets the gloo tests exercise the distributed plumbing (count
exchange, split sizes, all-to-all order, local re-sort, backward mirror) on CPU ranks.  Every stage
here is plain PyTorch built on the oracle's tables; the product never imports this module."""
import importlib

import torch

from oracle import moe_oracle as O

_ops = importlib.import_module("triton-kernel-fused_b200.ops")
Permutation = _ops.Permutation


class CpuKernels:
    @staticmethod
    def permute_build(idx, E, want_order=False):
        T, k = idx.shape
        tb = O.permutation_tables(idx, E) if T > 0 else None
        M = T * k
        cap = ((M + 255) // 256 + E) * 256
        if tb is None:
            z = torch.zeros
            return Permutation(T, k, E, cap, z(E, dtype=torch.int32), z(E + 1, dtype=torch.int32),
                               z(E + 1, dtype=torch.int32), z(0, dtype=torch.int32), z(cap, dtype=torch.int32),
                               z(cap // 256, dtype=torch.int32), z(0, dtype=torch.int32), z(0, dtype=torch.int32))
        total = int(tb["poffs"][-1])
        row_slot = torch.full((cap,), -1, dtype=torch.int32)
        row_slot[:total] = tb["row_slot"]
        tile_expert = torch.zeros(cap // 256, dtype=torch.int32)
        tile_expert[: total // 256] = tb["tile_expert"]
        order = tb["order"].to(torch.int32)
        slot_pos = torch.empty(M, dtype=torch.int32)
        slot_pos[tb["order"]] = torch.arange(M, dtype=torch.int32)
        return Permutation(T, k, E, cap, tb["counts"], tb["offs"], tb["poffs"], tb["slot_row"], row_slot,
                           tile_expert, order, slot_pos)

    @staticmethod
    def gather_rows_raw(x, row_slot, total_rows, k, rows_cap):
        total = int(total_rows[0])
        out = torch.zeros(max(rows_cap, 1), x.shape[1], dtype=x.dtype)
        rs = row_slot[:total].long()
        live = rs >= 0
        out[:total][live] = x[(rs[live] // k)]
        return out

    @classmethod
    def gather_rows(cls, x, perm):
        return cls.gather_rows_raw(x, perm.row_slot, perm.poffs[perm.E:], perm.k, perm.cap)

    @classmethod
    def gather_compact(cls, x, perm):
        return cls.gather_rows_raw(x, perm.order, perm.offs[perm.E:], perm.k, perm.T * perm.k)

    @staticmethod
    def _segments(perm):
        p = perm.poffs.tolist()
        return [(e, p[e], p[e + 1]) for e in range(perm.E) if p[e + 1] > p[e]]

    @classmethod
    def expert_gate_up_swiglu(cls, x_s, w_gu, perm):
        I = w_gu.shape[1] // 2
        gate_up = torch.zeros(perm.cap, 2 * I, dtype=x_s.dtype)
        for e, a, b in cls._segments(perm):
            gate_up[a:b] = x_s[a:b] @ w_gu[e].t()
        return gate_up, O.swiglu(gate_up, I)

    @classmethod
    def expert_down(cls, inter, w_d, perm):
        eo = torch.zeros(perm.cap, w_d.shape[1], dtype=inter.dtype)
        for e, a, b in cls._segments(perm):
            eo[a:b] = inter[a:b] @ w_d[e].t()
        return eo

    @classmethod
    def expert_down_dgrad_glu(cls, grad_eo, w_d, gate_up, perm):
        I = w_d.shape[2]
        gi = torch.zeros(perm.cap, I, dtype=grad_eo.dtype)
        for e, a, b in cls._segments(perm):
            gi[a:b] = grad_eo[a:b] @ w_d[e]
        g, u = gate_up[:, :I], gate_up[:, I:]
        s = torch.sigmoid(g)
        return torch.cat([gi * u * s * (1 + g * (1 - s)), gi * g * s], 1)

    @classmethod
    def expert_gate_up_dgrad(cls, grad_gu, w_gu, perm):
        gx = torch.zeros(perm.cap, w_gu.shape[2], dtype=grad_gu.dtype)
        for e, a, b in cls._segments(perm):
            gx[a:b] = grad_gu[a:b] @ w_gu[e]
        return gx

    @classmethod
    def expert_wgrad(cls, a_, b_, perm):
        out = torch.zeros(perm.E, a_.shape[1], b_.shape[1], dtype=a_.dtype)
        for e, a, b in cls._segments(perm):
            out[e] = a_[a:b].t() @ b_[a:b]
        return out

    @staticmethod
    def combine_raw(rows, w, slot_table, T, k):
        st = slot_table.long()
        live = (st >= 0).view(T, k, 1).to(rows.dtype)          # a slot without a row (-1) adds nothing
        r = rows[st.clamp_min(0)].view(T, k, -1) * live
        if w is None:
            return r.sum(1)
        return (r * w.view(T, k, 1).to(rows.dtype)).sum(1)

    @classmethod
    def combine(cls, rows, w, perm):
        return cls.combine_raw(rows, w, perm.slot_row, perm.T, perm.k)

    @staticmethod
    def combine_bwd_raw(grad_out, eo, w, row_slot, total_rows, k, rows_cap):
        total = int(total_rows[0])
        grad_eo = torch.zeros_like(eo)
        grad_w = torch.zeros(w.shape, dtype=torch.float32)
        rs = row_slot[:total].long()
        live = rs >= 0
        go = grad_out[rs[live] // k]
        grad_eo[:total][live] = go * w.flatten()[rs[live]][:, None].to(go.dtype)
        grad_w.view(-1)[rs[live]] = (go.float() * eo[:total][live].float()).sum(1)
        return grad_eo, grad_w

    @staticmethod
    def ep_plan(counts_all, W, rank, E, rows_cap=0, tile=256):
        """CPU model of the expert-parallel plan (csrc/ep.cu ep_plan_kernel): from the (W, E) count matrix, this rank's
        padded segments, the first row of every source's block in them, and the first row of this rank's block inside
        every expert's owner.  rows_cap > 0: if any owner's padded rows exceed it, every rank returns the tables of a
        step that computes nothing."""
        El = E // W
        tot = counts_all.sum(0)
        pad = lambda c: (int(c) + tile - 1) // tile * tile
        start = torch.zeros(E, dtype=torch.int64)
        owner_rows = []
        for d in range(W):
            run = 0
            for j in range(El):
                start[d * El + j] = run
                run += pad(tot[d * El + j])
            owner_rows.append(run)
        if rows_cap > 0 and any(r > rows_cap for r in owner_rows):
            return dict(overflow=True, poffs_l=torch.zeros(El + 1, dtype=torch.int64), counts_l=torch.zeros(El, dtype=torch.int64),
                        src_base=torch.full((W * El,), -(1 << 30), dtype=torch.int64), dest_base=torch.zeros(E, dtype=torch.int64))
        dest_base = start + counts_all[:rank].sum(0)
        mine = slice(rank * El, (rank + 1) * El)
        poffs_l = torch.cat([start[mine], torch.tensor([owner_rows[rank]])])
        src_base = torch.stack([start[mine] + counts_all[:s, mine].sum(0) for s in range(W)]).reshape(-1)
        return dict(overflow=False, poffs_l=poffs_l, counts_l=tot[mine].clone(), src_base=src_base, dest_base=dest_base)

