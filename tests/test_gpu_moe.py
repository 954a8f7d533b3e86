"""GPU: expert pipeline stage by stage and end to end, against the CPU oracle and the golden
vectors the reference itself produced."""
import os

import numpy as np
import pytest
import torch

from oracle import moe_oracle as O
from tests.golden.cases import CASES, sub

pytestmark = pytest.mark.gpu
DEV = "cuda"
TOL_BF16 = 2e-2        # relative L2 vs the fp32 reference, outputs and gradients (stated gate)


def _stage_reference(x, idx, w, gu, dn, go):
    """fp32 CPU values of every intermediate in the padded layout, from bf16-rounded inputs."""
    E, twoI, H = gu.shape
    I = twoI // 2
    tb = O.permutation_tables(idx, E)
    total = int(tb["poffs"][-1])
    rs = tb["row_slot"]
    live = rs >= 0
    tok = (rs.clamp_min(0) // idx.shape[1]).long()
    x_s = torch.zeros(total, H)
    x_s[live] = x.float()[tok[live]]
    te = torch.repeat_interleave(tb["tile_expert"].long(), 256)
    gate_up = torch.zeros(total, twoI)
    eo = torch.zeros(total, H)
    inter = torch.zeros(total, I)
    for e in range(E):
        m = te == e
        gate_up[m] = x_s[m] @ gu[e].float().t()
        inter[m] = O.swiglu(gate_up[m], I)
        eo[m] = inter[m] @ dn[e].float().t()
    return tb, total, x_s, gate_up, inter, eo, te


@pytest.mark.parametrize("T,H,E,I,k", [(1024, 256, 8, 192, 2), (700, 128, 6, 96, 2), (2048, 512, 16, 320, 4)])
def test_forward_stages(pkg, T, H, E, I, k):
    inp = O.make_inputs(T, H, E, I, k, seed=21, bias_std=0.01, dtype=torch.bfloat16)
    idx, w, _ = O.router_epilogue_fwd(inp["x"].float() @ inp["gate_weight"].float().t(), inp["bias"], k)
    tb, total, x_s, gate_up, inter, eo, te = _stage_reference(inp["x"], idx, w, inp["gate_up"], inp["down"], None)
    ops = pkg.ops
    perm = ops.permute_build(idx.to(DEV), E)
    xs_d = ops.gather_rows(inp["x"].to(DEV), perm)
    gu_d, it_d = ops.expert_gate_up_swiglu(xs_d, inp["gate_up"].to(DEV), perm)
    pkg.check_status()
    assert O.rel_l2(gu_d[:total].float().cpu(), gate_up) < 4e-3
    assert O.rel_l2(it_d[:total].float().cpu(), inter) < 8e-3
    eo_d = ops.expert_down(it_d, inp["down"].to(DEV), perm)
    pkg.check_status()
    assert O.rel_l2(eo_d[:total].float().cpu(), eo) < 1e-2
    out = ops.combine(eo_d, w.to(DEV), perm)
    ref = O.moe_experts(inp["x"].float(), idx, w, inp["gate_up"].float(), inp["down"].float())
    assert O.rel_l2(out.float().cpu(), ref) < TOL_BF16
    # pad rows stay zero through the whole forward
    pad = (tb["row_slot"] < 0)
    assert (gu_d[:total].cpu()[pad] == 0).all() and (eo_d[:total].cpu()[pad] == 0).all()


def test_row_windows_compose_to_the_whole_launch(pkg):
    """gate/up + SwiGLU and dgrad(down) + GLU backward over two windows of rows (the expert-parallel layer runs groups
    of experts this way) write exactly what one launch over all rows writes; a misaligned window is refused."""
    T, H, E, I, k = 2048, 256, 8, 192, 2
    inp = O.make_inputs(T, H, E, I, k, seed=23, bias_std=0.01, dtype=torch.bfloat16)
    idx, w, _ = O.router_epilogue_fwd(inp["x"].float() @ inp["gate_weight"].float().t(), inp["bias"], k)
    ops = pkg.ops
    perm = ops.permute_build(idx.to(DEV), E)
    xs = ops.gather_rows(inp["x"].to(DEV), perm)
    gu_w, dn_w = inp["gate_up"].to(DEV), inp["down"].to(DEV)
    gu_full, it_full = ops.expert_gate_up_swiglu(xs, gu_w, perm)
    cut = int(perm.poffs[E // 2])                       # a tile-aligned expert boundary
    total = int(perm.poffs[E])
    gu_two, it_two = torch.zeros_like(gu_full), torch.zeros_like(it_full)
    ops.expert_gate_up_swiglu(xs, gu_w, perm, out=(gu_two, it_two), rows=(0, cut))
    assert (gu_two[cut:total] == 0).all()                # the first window leaves the other rows alone
    ops.expert_gate_up_swiglu(xs, gu_w, perm, out=(gu_two, it_two), rows=(cut, perm.cap))
    pkg.check_status()
    assert torch.equal(gu_two[:total], gu_full[:total]) and torch.equal(it_two[:total], it_full[:total])
    geo = torch.randn(perm.cap, H, device=DEV).to(torch.bfloat16)
    gg_full = ops.expert_down_dgrad_glu(geo, dn_w, gu_full, perm)
    gg_two = torch.zeros_like(gg_full)
    ops.expert_down_dgrad_glu(geo, dn_w, gu_full, perm, out=gg_two, rows=(cut, perm.cap))
    ops.expert_down_dgrad_glu(geo, dn_w, gu_full, perm, out=gg_two, rows=(0, cut))
    pkg.check_status()
    assert torch.equal(gg_two[:total], gg_full[:total])
    with pytest.raises(ValueError):
        ops.expert_gate_up_swiglu(xs, gu_w, perm, out=(gu_two, it_two), rows=(100, cut))


@pytest.mark.parametrize("T,H,E,I,k", [(1024, 256, 8, 192, 2), (2048, 512, 16, 320, 4)])
def test_backward_stages(pkg, T, H, E, I, k):
    inp = O.make_inputs(T, H, E, I, k, seed=22, bias_std=0.01, dtype=torch.bfloat16)
    idx, w, _ = O.router_epilogue_fwd(inp["x"].float() @ inp["gate_weight"].float().t(), inp["bias"], k)
    tb, total, x_s, gate_up, inter, eo, te = _stage_reference(inp["x"], idx, w, inp["gate_up"], inp["down"], None)
    rs = tb["row_slot"]
    live = rs >= 0
    tok = (rs.clamp_min(0) // k).long()
    go = inp["grad_out"].float()
    grad_eo = torch.zeros(total, H)
    grad_eo[live] = go[tok[live]] * w.flatten()[rs[live].long()][:, None]
    grad_w = torch.zeros(T * k)
    grad_w[rs[live].long()] = (go[tok[live]] * eo[live]).sum(1)
    ops = pkg.ops
    perm = ops.permute_build(idx.to(DEV), E)
    to = lambda t: t.to(torch.bfloat16).to(DEV)
    cap = perm.cap

    def padded(t):
        buf = torch.zeros(cap, t.shape[1], dtype=torch.bfloat16, device=DEV)
        buf[:total] = to(t)
        return buf

    geo_d, gw_d = ops.combine_bwd(to(go), padded(eo), w.to(DEV), perm)
    assert O.rel_l2(geo_d[:total].float().cpu(), grad_eo) < 4e-3
    assert O.rel_l2(gw_d.flatten().cpu(), grad_w) < 1e-2

    # dgrad(down) + GLU backward
    gu_b = padded(gate_up)
    ggu_d = ops.expert_down_dgrad_glu(padded(grad_eo), inp["down"].to(DEV), gu_b, perm)
    pkg.check_status()
    g = gu_b[:total].float().cpu()
    gate, up = g[:, :I], g[:, I:]
    grad_inter = torch.zeros(total, I)
    for e in range(E):
        m = te == e
        grad_inter[m] = padded(grad_eo)[:total].float().cpu()[m] @ inp["down"][e].float()
    s = torch.sigmoid(gate)
    ref_ggu = torch.cat([grad_inter * up * s * (1 + gate * (1 - s)), grad_inter * gate * s], 1)
    assert O.rel_l2(ggu_d[:total].float().cpu(), ref_ggu) < 1.2e-2

    # dgrad(gate_up)
    gx_d = ops.expert_gate_up_dgrad(padded(ref_ggu), inp["gate_up"].to(DEV), perm)
    pkg.check_status()
    ref_gx = torch.zeros(total, H)
    rg = padded(ref_ggu)[:total].float().cpu()
    for e in range(E):
        m = te == e
        ref_gx[m] = rg[m] @ inp["gate_up"][e].float()
    assert O.rel_l2(gx_d[:total].float().cpu(), ref_gx) < 4e-3

    # wgrads
    a, b = padded(grad_eo), padded(inter)
    gwd_d = ops.expert_wgrad(a, b, perm)
    pkg.check_status()
    ref = torch.stack([a[:total].float().cpu()[te == e].t() @ b[:total].float().cpu()[te == e] for e in range(E)])
    assert O.rel_l2(gwd_d.float().cpu(), ref) < 4e-3
    a, b = padded(ref_ggu), padded(x_s)
    gwu_d = ops.expert_wgrad(a, b, perm)
    pkg.check_status()
    ref = torch.stack([a[:total].float().cpu()[te == e].t() @ b[:total].float().cpu()[te == e] for e in range(E)])
    assert O.rel_l2(gwu_d.float().cpu(), ref) < 4e-3


def _run_moe(pkg, inp, idx, w):
    leaves = dict(hidden=inp["x"].to(torch.bfloat16).to(DEV).requires_grad_(True),
                  wt=w.to(DEV).requires_grad_(True),
                  gu=inp["gate_up"].to(torch.bfloat16).to(DEV).requires_grad_(True),
                  dn=inp["down"].to(torch.bfloat16).to(DEV).requires_grad_(True))
    E = inp["gate_up"].shape[0]
    codes = torch.zeros(E, dtype=torch.int32, device=DEV)
    out = pkg.moe(leaves["hidden"], idx.to(DEV), leaves["wt"], leaves["gu"], leaves["dn"], codes)
    (out.float() * inp["grad_out"].to(DEV).float()).sum().backward()
    pkg.check_status()
    return out, leaves


@pytest.mark.parametrize("name", list(CASES))
def test_moe_against_reference_golden(pkg, golden_dir, name):
    """bf16 CUDA path vs the fp32 outputs of the reference's own moe_eager (stored fixtures)."""
    T, H, E, I, k, seed, bstd, cap = CASES[name]
    g = np.load(os.path.join(golden_dir, f"experts_{name}.npz"))
    inp = O.make_inputs(T, H, E, I, k, seed=seed, bias_std=bstd)
    idx, w = torch.from_numpy(g["idx"]), torch.from_numpy(g["w"])
    out, lv = _run_moe(pkg, inp, idx, w)
    assert out.dtype == torch.bfloat16 and out.shape == (T, H)
    assert O.rel_l2(out.float().cpu(), torch.from_numpy(g["out"])) < TOL_BF16
    assert O.rel_l2(lv["hidden"].grad.float().cpu(), torch.from_numpy(g["grad_hidden"])) < TOL_BF16
    assert O.rel_l2(lv["wt"].grad.float().cpu(), torch.from_numpy(g["grad_w"])) < TOL_BF16
    assert O.rel_l2(sub(lv["gu"].grad.float().cpu()), torch.from_numpy(g["grad_gate_up_sub"])) < TOL_BF16
    assert O.rel_l2(sub(lv["dn"].grad.float().cpu()), torch.from_numpy(g["grad_down_sub"])) < TOL_BF16
    if cap is not None:     # experts without tokens: exactly zero weight gradients, no NaN
        assert (lv["gu"].grad[cap:] == 0).all() and (lv["dn"].grad[cap:] == 0).all()
    for t in lv.values():
        assert torch.isfinite(t.grad).all()


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16])
def test_moe_takes_fp32_and_fp16_tensors(pkg, golden_dir, dtype):
    """Benchmark config 1 is stated in fp32: fp32 / fp16 callers get the bf16 computation with results and
    gradients in their own dtypes, within the bf16 tolerance of the reference's fp32 outputs."""
    T, H, E, I, k, seed, bstd, cap = CASES["cfg1"]
    g = np.load(os.path.join(golden_dir, "experts_cfg1.npz"))
    inp = O.make_inputs(T, H, E, I, k, seed=seed, bias_std=bstd)
    idx, w = torch.from_numpy(g["idx"]).to(DEV), torch.from_numpy(g["w"]).to(DEV).requires_grad_(True)
    hidden = inp["x"].to(dtype).to(DEV).requires_grad_(True)
    gu = inp["gate_up"].to(dtype).to(DEV).requires_grad_(True)
    dn = inp["down"].to(dtype).to(DEV).requires_grad_(True)
    out = pkg.moe(hidden, idx, w, gu, dn, torch.zeros(E, dtype=torch.int32, device=DEV))
    (out.float() * inp["grad_out"].to(DEV).float()).sum().backward()
    pkg.check_status()
    assert out.dtype == dtype and hidden.grad.dtype == dtype and gu.grad.dtype == dtype and dn.grad.dtype == dtype
    assert O.rel_l2(out.float().cpu(), torch.from_numpy(g["out"])) < TOL_BF16
    assert O.rel_l2(hidden.grad.float().cpu(), torch.from_numpy(g["grad_hidden"])) < TOL_BF16
    assert O.rel_l2(w.grad.float().cpu(), torch.from_numpy(g["grad_w"])) < TOL_BF16
    assert O.rel_l2(sub(gu.grad.float().cpu()), torch.from_numpy(g["grad_gate_up_sub"])) < TOL_BF16
    assert O.rel_l2(sub(dn.grad.float().cpu()), torch.from_numpy(g["grad_down_sub"])) < TOL_BF16


def test_moe_mid_size_vs_oracle_and_determinism(pkg):
    T, H, E, I, k = 4096, 1024, 16, 704, 4
    inp = O.make_inputs(T, H, E, I, k, seed=5, dtype=torch.bfloat16)
    idx, w, _, _ = O.mlp_router_fwd(inp["x"], inp["gate_weight"], None, k)
    out, lv = _run_moe(pkg, inp, idx, w)
    out2, lv2 = _run_moe(pkg, inp, idx, w)
    assert torch.equal(out, out2)
    for n in lv:
        assert torch.equal(lv[n].grad, lv2[n].grad), n      # no atomics anywhere: bit-identical reruns
    hidden = inp["x"].float().requires_grad_(True)
    wt = w.clone().requires_grad_(True)
    gu = inp["gate_up"].float().requires_grad_(True)
    dn = inp["down"].float().requires_grad_(True)
    ref = O.moe_experts(hidden, idx, wt, gu, dn)
    (ref * inp["grad_out"].float()).sum().backward()
    assert O.rel_l2(out.float().cpu(), ref.detach()) < TOL_BF16
    assert O.rel_l2(lv["hidden"].grad.float().cpu(), hidden.grad) < TOL_BF16
    assert O.rel_l2(lv["wt"].grad.float().cpu(), wt.grad) < TOL_BF16
    assert O.rel_l2(lv["gu"].grad.float().cpu(), gu.grad) < TOL_BF16
    assert O.rel_l2(lv["dn"].grad.float().cpu(), dn.grad) < TOL_BF16


def test_layer_module_vs_oracle(pkg):
    T, H, E, I, k = 2048, 512, 32, 256, 6
    inp = O.make_inputs(T, H, E, I, k, seed=8, bias_std=0.01, dtype=torch.bfloat16)
    layer = pkg.MoELayer(H, I, E, top_k=k).to(DEV).to(torch.bfloat16)
    with torch.no_grad():
        layer.gate.weight.copy_(inp["gate_weight"])
        layer.gate_up_proj.copy_(inp["gate_up"])
        layer.down_proj.copy_(inp["down"])
        layer.bias.copy_(inp["bias"])
    assert layer.bias.dtype == torch.float32
    x = inp["x"].to(DEV).view(4, T // 4, H).requires_grad_(True)
    out = layer(x)
    (out.float() * inp["grad_out"].to(DEV).view_as(out).float()).sum().backward()
    pkg.check_status()
    # A logit on a bf16 rounding boundary can land on either side and flip a pick.  The flip rate is asserted on
    # its own; the values are then compared on IDENTICAL routing (the oracle's experts and backward run on the
    # device's picks), every tensor at the 2e-2 gate.
    idx_d, _, _ = pkg.fused_mlp_router(inp["x"].to(DEV), layer.gate.weight, layer.bias, k, E, return_counts=True)
    own = O.layer_fwd_bwd(inp["x"].float(), inp["gate_weight"].float(), inp["bias"], inp["gate_up"].float(),
                          inp["down"].float(), k, inp["grad_out"].float(), logits_dtype=torch.bfloat16)
    assert (idx_d.cpu() != own["idx"]).any(1).float().mean() < 0.005
    r = O.layer_fwd_bwd(inp["x"].float(), inp["gate_weight"].float(), inp["bias"], inp["gate_up"].float(),
                        inp["down"].float(), k, inp["grad_out"].float(), logits_dtype=torch.bfloat16,
                        idx_override=idx_d.cpu())
    assert O.rel_l2(out.view(T, H).float().cpu(), r["out"]) < TOL_BF16
    assert O.rel_l2(x.grad.view(T, H).float().cpu(), r["grad_x"]) < TOL_BF16
    assert O.rel_l2(layer.gate_up_proj.grad.float().cpu(), r["grad_gate_up"]) < TOL_BF16
    assert O.rel_l2(layer.down_proj.grad.float().cpu(), r["grad_down"]) < TOL_BF16
    assert O.rel_l2(layer.gate.weight.grad.float().cpu(), r["grad_gate_weight"]) < TOL_BF16
    assert torch.equal(layer.last_counts.cpu().long(), torch.bincount(idx_d.flatten().cpu(), minlength=E))
    layer.update_bias(0.001)
    assert (layer.bias != inp["bias"].to(DEV)).any()


def test_load_balance_loop_accumulates_between_bias_updates(pkg):
    """The reference's training loop (.autoresearch/train_grok_moe.py:79-80, 86-90): the load of every training
    forward since the last update is summed, the update uses the sum and clears it; evaluation forwards do not
    count; a second update without a forward changes nothing."""
    T, H, E, I, k = 1024, 256, 8, 128, 2
    inp = O.make_inputs(T, H, E, I, k, seed=13, bias_std=0.05, dtype=torch.bfloat16)
    layer = pkg.MoELayer(H, I, E, top_k=k).to(DEV).to(torch.bfloat16)
    with torch.no_grad():
        layer.gate.weight.copy_(inp["gate_weight"])
        layer.bias.copy_(inp["bias"])
    x1, x2 = inp["x"][:T // 2].to(DEV), inp["x"][T // 2:].to(DEV)
    with torch.no_grad():
        layer(x1)
        c1 = layer.last_counts.clone().long()
        layer(x2)
        c2 = layer.last_counts.clone().long()
        layer.eval()
        layer(x1)                                     # not counted
        layer.train()
    assert torch.equal(layer.load, c1 + c2) and layer.load.dtype == torch.int64
    st = layer.load_stats()
    assert st["load"] == (c1 + c2).tolist() and st["tokens_routed"] == T * k
    ref = O.router_bias_update(inp["bias"].clone(), (c1 + c2).cpu(), 0.01)
    layer.update_bias(0.01)
    assert torch.equal(layer.bias.cpu(), ref) and int(layer.load.sum()) == 0
    layer.update_bias(0.01)                           # nothing routed since: no change
    assert torch.equal(layer.bias.cpu(), ref)


def test_skewed_routing_with_empty_experts(pkg):
    """Zipf-skewed logit bias (reduced size of the many-expert skewed config): some experts get no
    tokens; their weight gradients are exactly zero and nothing is NaN."""
    T, H, E, I, k = 4096, 256, 128, 128, 8
    inp = O.make_inputs(T, H, E, I, k, seed=3, zipf_s=1.1, dtype=torch.bfloat16)
    logits = inp["x"].float() @ inp["gate_weight"].float().t() + 3.0 * inp["logit_bias"][None, :]
    idx, w, counts = O.router_epilogue_fwd(logits, None, k)
    assert (counts == 0).any()
    out, lv = _run_moe(pkg, inp, idx, w)
    empty = counts == 0
    assert (lv["gu"].grad.cpu()[empty] == 0).all() and (lv["dn"].grad.cpu()[empty] == 0).all()
    ref = O.moe_experts(inp["x"].float(), idx, w, inp["gate_up"].float(), inp["down"].float())
    assert O.rel_l2(out.float().cpu(), ref) < TOL_BF16
    for t in lv.values():
        assert torch.isfinite(t.grad).all()


def test_full_size_properties(pkg):
    """Benchmark-size layer (T=16384, H=2048, E=64, I=1408, k=6): size-independent properties.
    (1) doubling the routing weights doubles the output bit-exactly; (2) permuting the tokens
    permutes the output rows bit-exactly; (3) the permutation tables invert each other."""
    T, H, E, I, k = 16384, 2048, 64, 1408, 6
    g = torch.Generator(device=DEV).manual_seed(0)
    x = torch.randn(T, H, device=DEV, generator=g).to(torch.bfloat16)
    gu = (torch.randn(E, 2 * I, H, device=DEV, generator=g) * 0.02).to(torch.bfloat16)
    dn = (torch.randn(E, H, I, device=DEV, generator=g) * 0.02).to(torch.bfloat16)
    wr = (torch.randn(E, H, device=DEV, generator=g) * 0.02).to(torch.bfloat16)
    codes = torch.zeros(E, dtype=torch.int32, device=DEV)
    idx, w = pkg.fused_mlp_router(x, wr, None, k, E)
    out = pkg.moe(x, idx, w, gu, dn, codes)
    out2 = pkg.moe(x, idx, w * 2, gu, dn, codes)
    pkg.check_status()
    assert torch.isfinite(out).all()
    assert torch.equal(out2, out * 2)
    p = torch.randperm(T, device=DEV, generator=g)
    out3 = pkg.moe(x[p], idx[p], w[p], gu, dn, codes)
    assert torch.equal(out3, out[p])
    perm = pkg.ops.permute_build(idx, E)
    total = int(perm.poffs[-1])
    rs = perm.row_slot[:total]
    assert int((rs >= 0).sum()) == T * k
    assert torch.equal(rs[perm.slot_row.long()].long(), torch.arange(T * k, device=DEV))
    assert int(perm.counts.sum()) == T * k


def _torch_gpu_fp32_reference(x, idx, w, gu, dn, go):
    """Independent fp32 reference on the GPU (plain torch ops, per-expert loop, autograd): used at the
    benchmark sizes where the CPU oracle would take minutes."""
    E = gu.shape[0]
    I = gu.shape[1] // 2
    xf = x.float().requires_grad_(True)
    wf = w.float().requires_grad_(True)
    guf = gu.float().requires_grad_(True)
    dnf = dn.float().requires_grad_(True)
    out = torch.zeros_like(xf)
    flat_e = idx.flatten()
    tok = torch.arange(idx.shape[0], device=x.device).repeat_interleave(idx.shape[1])
    order = torch.sort(flat_e, stable=True).indices
    counts = torch.bincount(flat_e, minlength=E).tolist()
    pos = 0
    wu, wd = guf.unbind(0), dnf.unbind(0)
    for e in range(E):
        c = counts[e]
        if c == 0:
            continue
        sl = order[pos:pos + c]
        pos += c
        rows = tok[sl]
        g = xf[rows] @ wu[e].t()
        inter = torch.nn.functional.silu(g[:, :I]) * g[:, I:]
        out = out.index_add(0, rows, (inter @ wd[e].t()) * wf.flatten()[sl].unsqueeze(-1))
    (out * go.float()).sum().backward()
    return out.detach(), xf.grad, wf.grad, guf.grad, dnf.grad, counts


@pytest.mark.parametrize("name,T,H,E,I,k,zipf", [("config2", 16384, 2048, 64, 1408, 6, None),
                                                 ("config3_skewed", 32768, 2048, 128, 768, 8, 1.1)])
def test_benchmark_size_configs_vs_fp32(pkg, name, T, H, E, I, k, zipf):
    """The bf16 single-GPU configurations at FULL size: output and every gradient within 2e-2 relative
    L2 of an fp32 computation; the skewed configuration must leave some experts without tokens and
    their weight gradients exactly zero."""
    g = torch.Generator(device=DEV).manual_seed(7)
    x = torch.randn(T, H, device=DEV, generator=g).to(torch.bfloat16)
    gu = (torch.randn(E, 2 * I, H, device=DEV, generator=g) * 0.02).to(torch.bfloat16)
    dn = (torch.randn(E, H, I, device=DEV, generator=g) * 0.02).to(torch.bfloat16)
    wr = (torch.randn(E, H, device=DEV, generator=g) * 0.02).to(torch.bfloat16)
    go = torch.randn(T, H, device=DEV, generator=g).to(torch.bfloat16)
    logits = pkg.ops.gemm_nt(x, wr)
    if zipf is not None:
        ranks = torch.randperm(E, device=DEV, generator=g).float() + 1.0
        p = ranks.pow(-zipf)
        logits = (logits.float() + 3.0 * torch.log(p / p.sum())[None, :]).to(torch.bfloat16)
    idx, w, counts = pkg.ops.router_topk_fwd(logits, None, k)
    lv = dict(x=x.clone().requires_grad_(True), w=w.clone().requires_grad_(True),
              gu=gu.clone().requires_grad_(True), dn=dn.clone().requires_grad_(True))
    out = pkg.moe(lv["x"], idx, lv["w"], lv["gu"], lv["dn"], torch.zeros(E, dtype=torch.int32, device=DEV))
    out.backward(go)
    pkg.check_status()
    ref_out, gx, gw, ggu, gdn, cnt = _torch_gpu_fp32_reference(x, idx, w, gu, dn, go)
    assert cnt == counts.tolist()
    rel = lambda a, b: float((a.float() - b).norm() / b.norm())
    errs = dict(out=rel(out, ref_out), grad_x=rel(lv["x"].grad, gx), grad_w=rel(lv["w"].grad, gw),
                grad_gate_up=rel(lv["gu"].grad, ggu), grad_down=rel(lv["dn"].grad, gdn))
    print(name, {k_: f"{v:.2e}" for k_, v in errs.items()})
    for k_, v in errs.items():
        assert v < TOL_BF16, (name, k_, v)
    if zipf is not None:
        empty = counts == 0
        assert bool(empty.any()), "the skewed routing must leave some experts without tokens"
        assert (lv["gu"].grad[empty] == 0).all() and (lv["dn"].grad[empty] == 0).all()


def test_empty_input_gives_empty_output_and_zero_grads(pkg):
    """No tokens at all (an empty micro-batch): nothing is launched, shapes and zero gradients come back."""
    H, I, E, k = 256, 128, 8, 2
    gu = (torch.randn(E, 2 * I, H, device=DEV) * 0.02).to(torch.bfloat16).requires_grad_(True)
    dn = (torch.randn(E, H, I, device=DEV) * 0.02).to(torch.bfloat16).requires_grad_(True)
    codes = torch.zeros(E, dtype=torch.int32, device=DEV)
    for fn in (pkg.moe, pkg.moe_mxfp8):
        x = torch.zeros(0, H, device=DEV, dtype=torch.bfloat16, requires_grad=True)
        w = torch.zeros(0, k, device=DEV, dtype=torch.float32, requires_grad=True)
        out = fn(x, torch.zeros(0, k, device=DEV, dtype=torch.int64), w, gu, dn, codes)
        assert out.shape == (0, H) and out.dtype == torch.bfloat16
        gu.grad = dn.grad = None
        out.sum().backward()
        assert x.grad.shape == (0, H) and w.grad.shape == (0, k)
        assert float(gu.grad.abs().sum()) == 0.0 and float(dn.grad.abs().sum()) == 0.0
    layer = pkg.MoELayer(H, I, E, top_k=k).to(DEV).to(torch.bfloat16)
    x = torch.zeros(2, 0, H, device=DEV, dtype=torch.bfloat16, requires_grad=True)
    out = layer(x)
    assert out.shape == (2, 0, H)
    out.sum().backward()
    assert float(layer.gate.weight.grad.abs().sum()) == 0.0
    pkg.check_status()
