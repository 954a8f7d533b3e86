"""GPU: MXFP8 quantisers (bit-exact against the CPU quantise oracle) and the MXFP8 expert pipeline
(forward + backward within 5e-2 relative L2 of the quantise->dequantise oracle)."""
import pytest
import torch

from oracle import moe_oracle as O
from oracle import mxfp8_oracle as Q

pytestmark = pytest.mark.gpu
DEV = "cuda"
TOL_MX = 5e-2       # stated gate for the MXFP8 path


def _sf_equal(sf_dev, cs):
    """Scale atoms agree on every live (row, k-block); the bytes that pad the last 128-row block or
    the last 4-block chunk are never read by a GEMM and are left unwritten by the quantisers."""
    live = Q.sf_atoms(torch.ones_like(cs)) == 1
    return torch.equal(sf_dev.cpu()[live], Q.sf_atoms(cs)[live])


def test_quant_rows_bit_exact(pkg):
    g = torch.Generator().manual_seed(0)
    x = (torch.randn(333, 384, generator=g) * torch.logspace(-4, 4, 333)[:, None]).to(torch.bfloat16)
    x[5] = 0                                              # an all-zero row
    x[7, :32] = torch.tensor(500.0).to(torch.bfloat16)    # saturating block
    q, sf = pkg.ops.mxfp8_quant_rows(x.to(DEV))
    cq, cs = Q.quantise(x.float())
    assert torch.equal(q.cpu(), cq)
    assert _sf_equal(sf, cs)


def test_quant_rows_interleave_and_transpose_bit_exact(pkg):
    g = torch.Generator().manual_seed(1)
    E, I, H = 3, 128, 256
    w = (torch.randn(E, 2 * I, H, generator=g) * 0.02).to(torch.bfloat16)
    q, sf = pkg.ops.mxfp8_quant_rows(w.view(E * 2 * I, H).to(DEV), interleave_I=I)
    perm = torch.cat([torch.cat([torch.arange(j, j + 64), I + torch.arange(j, j + 64)]) for j in range(0, I, 64)])
    wi = w[:, perm, :].reshape(E * 2 * I, H)
    cq, cs = Q.quantise(wi.float())
    assert torch.equal(q.cpu(), cq) and _sf_equal(sf, cs)
    qt, sft = pkg.ops.mxfp8_quant_transpose(w.to(DEV))
    wt = w.float().transpose(1, 2).contiguous()
    cq, cs = Q.quantise(wt)
    assert torch.equal(qt.cpu(), cq)
    assert _sf_equal(sft, cs.reshape(-1, cs.shape[-1]))


@pytest.mark.parametrize("G,R,C", [(1, 32, 2), (1, 160, 200), (2, 96, 130), (3, 256, 384), (1, 4000 * 32, 64)])
def test_quant_transpose_ragged_tiles_bit_exact(pkg, G, R, C):
    """Tiles of 128 x 128 with partial row blocks and column tails, several groups, many row tiles."""
    g = torch.Generator().manual_seed(3)
    x = (torch.randn(G, R, C, generator=g) * torch.logspace(-3, 3, C)[None, None, :]).to(torch.bfloat16)
    x[0, :32, 0] = 0                                      # an all-zero block
    qt, sft = pkg.ops.mxfp8_quant_transpose(x.to(DEV))
    cq, cs = Q.quantise(x.float().transpose(1, 2).contiguous())
    assert torch.equal(qt.cpu(), cq)
    assert _sf_equal(sft, cs.reshape(-1, cs.shape[-1]))


@pytest.mark.parametrize("G,R,C,I", [(1, 160, 224, 0), (3, 256, 384, 128), (2, 128, 96, 64), (1, 2048, 4096, 0)])
def test_quant_both_equals_the_two_passes(pkg, G, R, C, I):
    g = torch.Generator().manual_seed(4)
    x = (torch.randn(G, R, C, generator=g) * 0.3).to(torch.bfloat16).to(DEV)
    q, sf, qt, sft = pkg.ops.mxfp8_quant_both(x, interleave_I=I)
    q1, sf1 = pkg.ops.mxfp8_quant_rows(x.view(G * R, C), interleave_I=I)
    qt1, sft1 = pkg.ops.mxfp8_quant_transpose(x)
    assert torch.equal(q, q1) and torch.equal(qt, qt1)
    live = Q.sf_atoms(torch.ones(G * R, C // 32, dtype=torch.uint8)) == 1
    assert torch.equal(sf.cpu()[live], sf1.cpu()[live])
    live_t = Q.sf_atoms(torch.ones(G * C, R // 32, dtype=torch.uint8)) == 1
    assert torch.equal(sft.cpu()[live_t], sft1.cpu()[live_t])


@pytest.mark.parametrize("T,E,k,H", [(700, 6, 2, 256), (1500, 8, 3, 384), (33, 4, 1, 64)])
def test_gather_quant_both_equals_gather_then_quantise(pkg, T, E, k, H):
    """The fused gather + dual quantiser against gather_quant followed by the transposing quantiser of x_s."""
    g = torch.Generator().manual_seed(6)
    idx = torch.stack([torch.randperm(E, generator=g)[:k] for _ in range(T)])
    perm = pkg.ops.permute_build(idx.to(DEV), E)
    x = (torch.randn(T, H, generator=g) * torch.logspace(-2, 2, T)[:, None]).to(torch.bfloat16).to(DEV)
    q, sf, qt, sft = pkg.ops.mxfp8_gather_quant_both(x, perm)
    x_s, q1, sf1 = pkg.ops.mxfp8_gather_quant(x, perm)
    total = int(perm.poffs[-1])
    x_s[total:] = 0                                  # rows past the padded total are not written by the plain gather
    qt1, sft1 = pkg.ops.mxfp8_quant_transpose(x_s)
    assert torch.equal(q[:total], q1[:total]) and torch.equal(qt, qt1)
    ones = torch.zeros(perm.cap, H // 32, dtype=torch.uint8)
    ones[:total] = 1
    live = Q.sf_atoms(ones) == 1
    assert torch.equal(sf.cpu()[live], sf1.cpu()[live])
    live_t = Q.sf_atoms(torch.ones(H, perm.cap // 32, dtype=torch.uint8)) == 1
    assert torch.equal(sft.cpu()[live_t], sft1.cpu()[live_t])


@pytest.mark.parametrize("M,N,K", [(128, 128, 128), (300, 264, 1024), (1000, 2048, 512), (64, 72, 256)])
def test_mxfp8_gemm_matches_dequantised_product(pkg, M, N, K):
    g = torch.Generator().manual_seed(2)
    a = torch.randn(M, K, generator=g).to(torch.bfloat16)
    b = (torch.randn(N, K, generator=g) * 0.05).to(torch.bfloat16)
    aq, asf = pkg.ops.mxfp8_quant_rows(a.to(DEV))
    bq, bsf = pkg.ops.mxfp8_quant_rows(b.to(DEV))
    d = pkg.ops.mxfp8_gemm_nt(aq, asf, bq, bsf)
    pkg.check_status()
    ref = Q.qdq(a.float()) @ Q.qdq(b.float()).t()
    assert O.rel_l2(d.float().cpu(), ref) < 4e-3          # identical operands, bf16 output rounding only


@pytest.mark.parametrize("T,H,E,I,k", [(1024, 256, 8, 256, 2), (1536, 384, 6, 128, 3)])
def test_moe_mxfp8_forward_backward(pkg, T, H, E, I, k):
    inp = O.make_inputs(T, H, E, I, k, seed=51, bias_std=0.01, dtype=torch.bfloat16)
    idx, w, _, _ = O.mlp_router_fwd(inp["x"], inp["gate_weight"], inp["bias"], k)
    lv = dict(hidden=inp["x"].to(DEV).requires_grad_(True), wt=w.to(DEV).requires_grad_(True),
              gu=inp["gate_up"].to(DEV).requires_grad_(True), dn=inp["down"].to(DEV).requires_grad_(True))
    codes = torch.zeros(E, dtype=torch.int32, device=DEV)
    out = pkg.moe_mxfp8(lv["hidden"], idx.to(DEV), lv["wt"], lv["gu"], lv["dn"], codes)
    (out.float() * inp["grad_out"].to(DEV).float()).sum().backward()
    pkg.check_status()
    # the quantise -> dequantise oracle on the same bf16 inputs
    hid = inp["x"].float().requires_grad_(True)
    wt = w.clone().requires_grad_(True)
    gu = inp["gate_up"].float().requires_grad_(True)
    dn = inp["down"].float().requires_grad_(True)
    ref = Q.moe_experts_mxfp8(hid, idx, wt, gu, dn)
    (ref * inp["grad_out"].float()).sum().backward()
    errs = dict(out=O.rel_l2(out.float().cpu(), ref.detach()),
                grad_x=O.rel_l2(lv["hidden"].grad.float().cpu(), hid.grad),
                grad_w=O.rel_l2(lv["wt"].grad.float().cpu(), wt.grad),
                grad_gate_up=O.rel_l2(lv["gu"].grad.float().cpu(), gu.grad),
                grad_down=O.rel_l2(lv["dn"].grad.float().cpu(), dn.grad))
    print("mxfp8 vs quantised oracle:", {k_: f"{v:.3e}" for k_, v in errs.items()})
    for name, e in errs.items():
        assert e < TOL_MX, (name, e)
    # for the record: distance to the unquantised fp32 block
    full = O.moe_experts(inp["x"].float(), idx, w, inp["gate_up"].float(), inp["down"].float())
    assert O.rel_l2(out.float().cpu(), full) < 0.1


def test_quantised_weights_are_reused_until_the_stack_changes(pkg):
    """The cache of quantised expert stacks: a second call on unchanged weights launches no weight quantiser and
    returns the same bits; an in-place update (what an optimizer step does) invalidates it; a forward-only call
    that cached the row-wise copy alone is followed correctly by a call that needs the transposed copy too."""
    import importlib
    mx = importlib.import_module("triton-kernel-fused_b200.mxfp8")
    T, H, E, I, k = 512, 256, 4, 128, 2
    inp = O.make_inputs(T, H, E, I, k, seed=52, bias_std=0.01, dtype=torch.bfloat16)
    idx, w, _, _ = O.mlp_router_fwd(inp["x"], inp["gate_weight"], inp["bias"], k)
    x, idx_d, w_d = inp["x"].to(DEV), idx.to(DEV), w.to(DEV)
    gu = inp["gate_up"].to(DEV).requires_grad_(True)
    dn = inp["down"].to(DEV).requires_grad_(True)
    codes = torch.zeros(E, dtype=torch.int32, device=DEV)
    seen = []
    mx._QUANTISED.clear()
    assert mx.WEIGHT_CACHE
    weights = {gu.data_ptr(): "gate_up", dn.data_ptr(): "down"}
    real_rows, real_both = pkg.ops.mxfp8_quant_rows, pkg.ops.mxfp8_quant_both

    def spy(fn):
        def wrapped(t, *a, **kw):
            if t.data_ptr() in weights:
                seen.append(weights[t.data_ptr()])
            return fn(t, *a, **kw)
        return wrapped

    def run(grad):
        seen.clear()
        pkg.ops.mxfp8_quant_rows, pkg.ops.mxfp8_quant_both = spy(real_rows), spy(real_both)
        try:
            if grad:
                gu.grad = dn.grad = None
                out = pkg.moe_mxfp8(x, idx_d, w_d, gu, dn, codes)
                out.float().sum().backward()
                return out.detach().clone(), gu.grad.clone(), dn.grad.clone()
            with torch.no_grad():
                return pkg.moe_mxfp8(x, idx_d, w_d, gu, dn, codes).clone(), None, None
        finally:
            pkg.ops.mxfp8_quant_rows, pkg.ops.mxfp8_quant_both = real_rows, real_both

    o_inf, _, _ = run(False)
    assert sorted(seen) == ["down", "gate_up"]    # first call: both stacks quantised (row-wise only)
    o_inf2, _, _ = run(False)
    assert seen == [] and torch.equal(o_inf, o_inf2)
    o0, _, _ = run(True)                          # weight gradients only: the copies kept so far still serve
    assert seen == [] and torch.equal(o0, o_inf)
    x.requires_grad_(True)                        # grad_x needs gate_up quantised along 2I too: the row-only entry does not serve
    o1, g1, d1 = run(True)
    assert seen == ["gate_up"]
    o2, g2, d2 = run(True)
    assert seen == []
    assert torch.equal(o1, o2) and torch.equal(g1, g2) and torch.equal(d1, d2) and torch.equal(o1, o_inf)
    with torch.no_grad():
        gu.mul_(0.5)                              # version moves: the stale copy must not be used
    o3, _, _ = run(True)
    assert seen == ["gate_up"]                    # gate_up re-quantised, down still cached
    mx.WEIGHT_CACHE = False
    try:
        o4, _, _ = run(True)
        assert sorted(seen) == ["down", "gate_up"] and torch.equal(o3, o4)
    finally:
        mx.WEIGHT_CACHE = True
    assert not torch.equal(o3, o1)
    pkg.check_status()


def test_mxfp8_rejects_unaligned_width(pkg):
    x = torch.zeros(8, 192, dtype=torch.bfloat16, device=DEV)
    idx = torch.zeros(8, 1, dtype=torch.int64, device=DEV)
    w = torch.ones(8, 1, device=DEV)
    gu = torch.zeros(2, 256, 192, dtype=torch.bfloat16, device=DEV)
    dn = torch.zeros(2, 192, 128, dtype=torch.bfloat16, device=DEV)
    with pytest.raises(ValueError, match="multiples of 128"):
        pkg.moe_mxfp8(x, idx, w, gu, dn, torch.zeros(2, dtype=torch.int32, device=DEV))


def test_producer_epilogues_quantise_bit_identically(pkg):
    """The quantised copies written by the gather and by the SwiGLU / GLU-backward epilogues equal a
    separate quant_rows pass over the bf16 results, bit for bit (live rows)."""
    T, H, E, I, k = 1024, 256, 4, 256, 2
    ops = pkg.ops
    inp = O.make_inputs(T, H, E, I, k, seed=61, dtype=torch.bfloat16)
    idx, w, _, _ = O.mlp_router_fwd(inp["x"], inp["gate_weight"], None, k)
    perm = ops.permute_build(idx.to(DEV), E)
    total = int(perm.poffs[-1])
    x_s, xq, xsf = ops.mxfp8_gather_quant(inp["x"].to(DEV), perm)
    q_ref, _ = ops.mxfp8_quant_rows(x_s)
    assert torch.equal(x_s[:total], ops.gather_rows(inp["x"].to(DEV), perm)[:total])
    assert torch.equal(xq[:total], q_ref[:total])
    wq, wsf = ops.mxfp8_quant_rows(inp["gate_up"].to(DEV).view(E * 2 * I, H), interleave_I=I)
    gate_up = torch.empty(perm.cap, 2 * I, dtype=torch.bfloat16, device=DEV)
    inter = torch.empty(perm.cap, I, dtype=torch.bfloat16, device=DEV)
    _, iq, isf = ops.mxfp8_expert_gemm(ops.EPI_SWIGLU, xq, xsf, wq, wsf, perm, 2 * I, H, I, gate_up, inter,
                                       quantise_result=True)
    iq_ref, isf_ref = ops.mxfp8_quant_rows(inter)
    pkg.check_status()
    assert torch.equal(iq[:total], iq_ref[:total])
    cs = Q.quantise(inter[:total].float().cpu())[1]
    assert _sf_equal(isf[: Q.sf_atoms(cs).numel()], cs)


def test_mxfp8_configuration_at_full_size(pkg):
    """T=32768, H=4096, E=8, I=14336, top-2 (the MXFP8 configuration of the benchmark) at FULL size: output and
    every gradient within 5e-2 relative L2 of the quantise -> dequantise restatement, evaluated in fp32 on the
    GPU (the same oracle code, run on CUDA tensors; the CPU would need an hour for its 69 TFLOP)."""
    T, H, E, I, k = 32768, 4096, 8, 14336, 2
    g = torch.Generator(device=DEV).manual_seed(9)
    x = torch.randn(T, H, device=DEV, generator=g).to(torch.bfloat16)
    gu = (torch.randn(E, 2 * I, H, device=DEV, generator=g) * 0.02).to(torch.bfloat16)
    dn = (torch.randn(E, H, I, device=DEV, generator=g) * 0.02).to(torch.bfloat16)
    go = torch.randn(T, H, device=DEV, generator=g).to(torch.bfloat16)
    idx, w, _ = pkg.ops.router_topk_fwd(torch.randn(T, E, device=DEV, generator=g), None, k)
    lv = dict(x=x.clone().requires_grad_(True), w=w.clone().requires_grad_(True),
              gu=gu.clone().requires_grad_(True), dn=dn.clone().requires_grad_(True))
    out = pkg.moe_mxfp8(lv["x"], idx, lv["w"], lv["gu"], lv["dn"], torch.zeros(E, dtype=torch.int32, device=DEV))
    out.backward(go)
    pkg.check_status()
    got = dict(out=out.detach().float(), grad_x=lv["x"].grad.float(), grad_w=lv["w"].grad.float(),
               grad_gate_up=lv["gu"].grad.float(), grad_down=lv["dn"].grad.float())
    del out, lv
    rx, rw = x.float().requires_grad_(True), w.clone().requires_grad_(True)
    rgu, rdn = gu.float().requires_grad_(True), dn.float().requires_grad_(True)
    ref = Q.moe_experts_mxfp8(rx, idx, rw, rgu, rdn)
    ref.backward(go.float())
    want = dict(out=ref.detach(), grad_x=rx.grad, grad_w=rw.grad, grad_gate_up=rgu.grad, grad_down=rdn.grad)
    errs = {n: float((got[n] - want[n]).norm() / want[n].norm()) for n in got}
    print("config 4 at full size vs quantised fp32 reference:", {n: f"{v:.3e}" for n, v in errs.items()})
    for n, v in errs.items():
        assert v < TOL_MX, (n, v)
