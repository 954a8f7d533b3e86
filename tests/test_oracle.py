"""CPU: the oracle against the golden vectors made by the reference itself (tests/golden)."""
import os

import numpy as np
import pytest
import torch

from oracle import moe_oracle as O
from tests.golden.cases import CASES, routing_for, sub


def _load(golden_dir, kind, name):
    return np.load(os.path.join(golden_dir, f"{kind}_{name}.npz"))


@pytest.mark.parametrize("name", list(CASES))
def test_experts_match_reference_golden(golden_dir, name):
    T, H, E, I, k, seed, bstd, cap = CASES[name]
    g = _load(golden_dir, "experts", name)
    inp = O.make_inputs(T, H, E, I, k, seed=seed, bias_std=bstd)
    idx = torch.from_numpy(g["idx"])
    hidden = inp["x"].clone().requires_grad_(True)
    wt = torch.from_numpy(g["w"]).clone().requires_grad_(True)
    gu = inp["gate_up"].clone().requires_grad_(True)
    dn = inp["down"].clone().requires_grad_(True)
    out = O.moe_experts(hidden, idx, wt, gu, dn)
    (out * inp["grad_out"]).sum().backward()
    tol = 1e-5     # fp32 on both sides; only the summation order differs
    assert O.rel_l2(out.detach(), torch.from_numpy(g["out"])) < tol
    assert O.rel_l2(hidden.grad, torch.from_numpy(g["grad_hidden"])) < tol
    assert O.rel_l2(wt.grad, torch.from_numpy(g["grad_w"])) < tol
    assert O.rel_l2(sub(gu.grad), torch.from_numpy(g["grad_gate_up_sub"])) < tol
    assert O.rel_l2(sub(dn.grad), torch.from_numpy(g["grad_down_sub"])) < tol
    assert abs(float(gu.grad.double().norm()) - float(g["grad_gate_up_norm"])) < 1e-5 * float(g["grad_gate_up_norm"])
    assert abs(float(dn.grad.double().norm()) - float(g["grad_down_norm"])) < 1e-5 * float(g["grad_down_norm"])


@pytest.mark.parametrize("name", list(CASES))
def test_routing_in_golden_is_the_oracle_router(golden_dir, name):
    """The routing stored in the fixture is reproducible from the seeds (bit-exact)."""
    T, H, E, I, k, seed, bstd, cap = CASES[name]
    g = _load(golden_dir, "experts", name)
    inp = O.make_inputs(T, H, E, I, k, seed=seed, bias_std=bstd)
    idx, w = routing_for(inp, E, k, cap)
    assert torch.equal(idx, torch.from_numpy(g["idx"]))
    assert torch.equal(w, torch.from_numpy(g["w"]))


@pytest.mark.parametrize("name", list(CASES))
def test_stable_sort_vs_reference_sort(golden_dir, name):
    """counts/bounds exact; each expert segment equal as a set (reference order is unspecified)."""
    T, H, E, I, k, seed, bstd, cap = CASES[name]
    g = _load(golden_dir, "sort", name)
    idx = torch.from_numpy(_load(golden_dir, "experts", name)["idx"])
    order, st, counts, offs = O.sort_by_expert_stable(idx, E)
    assert counts.tolist() == g["counts"].tolist()
    assert offs.tolist() == g["bounds"].tolist()
    seg = torch.cat([torch.sort(st[int(offs[e]):int(offs[e + 1])]).values for e in range(E)])
    assert torch.equal(seg, torch.from_numpy(g["seg_sorted_tokens"]))
    # stability: within a segment the slot ids ascend
    for e in range(E):
        s = order[int(offs[e]):int(offs[e + 1])]
        assert bool((s[1:] > s[:-1]).all())
    if cap is not None:
        assert counts[cap:].sum() == 0


def test_router_restatement_matches_eager_statement():
    """Tie-free fp32 inputs: the iterative-argmax rule and the eager topk statement agree on the
    picked set, the pick order (both descending) and the weights."""
    inp = O.make_inputs(2048, 64, 16, 8, 4, seed=11, bias_std=0.01)
    idx, w, counts, logits = O.mlp_router_fwd(inp["x"], inp["gate_weight"], inp["bias"], 4)
    idx2, w2 = O.eager_router_topk(inp["x"], inp["gate_weight"], inp["bias"], 4)
    assert torch.equal(idx, idx2)
    assert O.rel_l2(w, w2) < 1e-6
    assert counts.tolist() == torch.bincount(idx.flatten(), minlength=16).tolist()


def test_router_tie_rule_lowest_index_first():
    scores = torch.tensor([[.5, .7, .7, .7, .1]])
    idx, w, _ = O.topk_from_scores(scores, None, 2)
    assert idx.tolist() == [[1, 2]]              # torch.topk would give [1, 3]
    assert torch.allclose(w, torch.tensor([[.5, .5]]))


@pytest.mark.parametrize("norm", [True, False])
def test_router_backward_matches_autograd(norm):
    torch.manual_seed(5)
    N, E, k = 257, 24, 3
    logits = torch.randn(N, E, dtype=torch.float64).float().requires_grad_(True)
    bias = torch.randn(E) * 0.01
    idx, w, _ = O.router_epilogue_fwd(logits.detach(), bias, k, norm, 2.5)
    s = 1.0 / (1.0 + torch.exp(-logits))
    ww = s.gather(1, idx)
    if norm:
        ww = ww / (ww.sum(-1, keepdim=True) + 1e-20)
    ww = ww * 2.5
    G = torch.randn(N, k)
    (ww * G).sum().backward()
    got = O.router_epilogue_bwd(logits.detach(), idx, G, norm, 2.5)
    assert O.rel_l2(got, logits.grad) < 1e-5
    assert O.rel_l2(ww.detach(), w) < 1e-6


def test_layer_autograd_equals_manual_router_backward():
    """Whole-block autograd (oracle.moe_layer) == experts autograd + manual router backward."""
    inp = O.make_inputs(256, 64, 8, 32, 2, seed=2, bias_std=0.01)
    r = O.layer_fwd_bwd(inp["x"], inp["gate_weight"], inp["bias"], inp["gate_up"], inp["down"], 2,
                        inp["grad_out"])
    idx, w, counts, logits = O.mlp_router_fwd(inp["x"], inp["gate_weight"], inp["bias"], 2)
    assert torch.equal(idx, r["idx"])
    hidden = inp["x"].clone().requires_grad_(True)
    wt = w.clone().requires_grad_(True)
    out = O.moe_experts(hidden, idx, wt, inp["gate_up"], inp["down"])
    (out * inp["grad_out"]).sum().backward()
    gx_r, gw_r, _ = O.mlp_router_bwd(inp["x"], inp["gate_weight"], logits, idx, wt.grad)
    assert O.rel_l2(hidden.grad + gx_r, r["grad_x"]) < 1e-5
    assert O.rel_l2(gw_r, r["grad_gate_weight"]) < 1e-5


def test_permutation_tables_consistent():
    torch.manual_seed(1)
    E, k, T = 10, 3, 300
    idx = torch.stack([torch.randperm(E)[:k] for _ in range(T)])
    tb = O.permutation_tables(idx, E, tile=16)
    poffs, slot_row, row_slot = tb["poffs"], tb["slot_row"], tb["row_slot"]
    assert int(poffs[-1]) % 16 == 0
    assert (row_slot >= 0).sum() == T * k
    assert torch.equal(row_slot[slot_row.long()], torch.arange(T * k, dtype=torch.int32))
    flat = idx.flatten()
    for e in range(E):
        rows = row_slot[int(poffs[e]):int(poffs[e + 1])]
        live = rows[rows >= 0]
        assert (flat[live.long()] == e).all()
        assert (live[1:] > live[:-1]).all()
        assert (rows[len(live):] == -1).all()
    assert tb["tile_expert"].numel() == int(poffs[-1]) // 16


def test_bias_update_rule():
    b = torch.zeros(4)
    O.router_bias_update(b, torch.tensor([10, 0, 5, 5]), 0.1)
    assert torch.allclose(b, torch.tensor([-0.1, 0.1, 0.0, 0.0]))
    b2 = b.clone()
    O.router_bias_update(b2, torch.tensor([1, 2, 3, 4]), 0.0)
    assert torch.equal(b, b2)
