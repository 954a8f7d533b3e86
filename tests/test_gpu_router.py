"""GPU: router epilogue kernels through the C ABI against the CPU oracle."""
import pytest
import torch

from oracle import moe_oracle as O

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _scores(N, E, seed, bf16_grid):
    g = torch.Generator().manual_seed(seed)
    s = torch.sigmoid(torch.randn(N, E, generator=g))
    if bf16_grid:                      # many exact ties inside a row
        s = s.to(torch.bfloat16).float()
    return s


@pytest.mark.parametrize("N,E,k", [(1000, 8, 2), (4099, 64, 6), (2048, 128, 8), (1024, 256, 8), (257, 40, 1),
                                   (512, 16, 16), (300, 64, 32), (64, 256, 32)])
@pytest.mark.parametrize("bf16_grid", [False, True])
@pytest.mark.parametrize("with_bias", [False, True])
def test_topk_from_identical_scores_is_bit_exact(pkg, N, E, k, bf16_grid, with_bias):
    s = _scores(N, E, 100 + E + k, bf16_grid)
    bias = torch.randn(E, generator=torch.Generator().manual_seed(3)) * 0.01 if with_bias else None
    idx_o, w_o, c_o = O.topk_from_scores(s, bias, k, True, 1.0)
    idx, w, c = pkg.ops.router_topk_fwd(s.to(DEV), None if bias is None else bias.to(DEV), k, True, 1.0,
                                        scores=True)
    assert torch.equal(idx.cpu(), idx_o)
    assert torch.equal(c.cpu(), c_o)
    assert torch.equal(w.cpu(), w_o)          # same fp32 operations in the same order


def test_topk_tie_rule_and_order(pkg):
    s = torch.tensor([[.5, .7, .7, .7, .1, 0, 0, 0]], device=DEV)
    idx, w, c = pkg.ops.router_topk_fwd(s, None, 2, True, 1.0, scores=True)
    assert idx.tolist() == [[1, 2]]
    assert c.tolist() == [0, 1, 1, 0, 0, 0, 0, 0]


@pytest.mark.parametrize("norm,scale", [(True, 1.0), (False, 2.5), (True, 0.5)])
def test_topk_from_bf16_logits(pkg, norm, scale):
    N, E, k = 8192, 64, 6
    g = torch.Generator().manual_seed(9)
    logits = (torch.randn(N, E, generator=g) * 0.9).to(torch.bfloat16)
    idx_o, w_o, c_o = O.router_epilogue_fwd(logits, None, k, norm, scale)
    idx, w, c = pkg.ops.router_topk_fwd(logits.to(DEV), None, k, norm, scale)
    # without a bias the selection only depends on the order of the logits: exact
    assert torch.equal(idx.cpu(), idx_o)
    assert torch.equal(c.cpu(), c_o)
    assert O.rel_l2(w.cpu(), w_o) < 1e-6      # sigmoid differs by an ulp between CPU and GPU


def test_topk_bwd_matches_oracle(pkg):
    N, E, k = 4096, 64, 6
    g = torch.Generator().manual_seed(10)
    logits = (torch.randn(N, E, generator=g) * 0.9).to(torch.bfloat16)
    G = torch.randn(N, k, generator=g)
    for norm, scale in ((True, 1.0), (False, 2.0)):
        idx_o, _, _ = O.router_epilogue_fwd(logits, None, k, norm, scale)
        ref = O.router_epilogue_bwd(logits, idx_o, G, norm, scale, out_dtype=torch.float32)
        gl = pkg.ops.router_topk_bwd(logits.to(DEV), idx_o.to(DEV), G.to(DEV), norm, scale)
        assert gl.dtype == torch.bfloat16
        assert O.rel_l2(gl.float().cpu(), ref) < 4e-3      # bf16 rounding of the output only
        nz = (gl != 0).sum(1).max().item()
        assert nz <= k


def test_bias_update(pkg):
    b = torch.zeros(64, device=DEV)
    counts = torch.randint(0, 100, (64,), dtype=torch.int32)
    ref = O.router_bias_update(torch.zeros(64), counts, 0.001)
    pkg.router_bias_update(b, counts.to(DEV), 0.001)
    assert torch.equal(b.cpu(), ref)
    pkg.router_bias_update(b, counts.to(DEV), 0.0)
    assert torch.equal(b.cpu(), ref)


def test_fused_mlp_router_forward_backward(pkg):
    T, H, E, k = 2048, 512, 64, 6
    inp = O.make_inputs(T, H, E, 8, k, seed=4, bias_std=0.01, dtype=torch.bfloat16)
    x = inp["x"].to(DEV).requires_grad_(True)
    W = inp["gate_weight"].to(DEV).requires_grad_(True)
    bias = inp["bias"].to(DEV)
    idx, w, counts = pkg.fused_mlp_router(x.view(4, T // 4, H), W, bias, k, E, return_counts=True)
    assert idx.shape == (4, T // 4, k) and w.dtype == torch.float32 and idx.dtype == torch.int64
    pkg.check_status()
    # oracle on the same bf16 inputs
    idx_o, w_o, c_o, logits_o = O.mlp_router_fwd(inp["x"], inp["gate_weight"], inp["bias"], k)
    idx_dev = idx.view(T, k).cpu()
    # logits may differ by one bf16 ulp at a rounding boundary and flip a pick: the flip rate is gated on its own,
    # the gradients are compared on the device's picks
    assert (idx_dev != idx_o).any(1).float().mean().item() < 0.005
    G = torch.randn(T, k, generator=torch.Generator().manual_seed(1))
    (w.view(T, k) * G.to(DEV)).sum().backward()
    gx_o, gw_o, _ = O.mlp_router_bwd(inp["x"], inp["gate_weight"], logits_o, idx_dev, G)
    assert O.rel_l2(x.grad.float().cpu(), gx_o.float()) < 2e-2
    assert O.rel_l2(W.grad.float().cpu(), gw_o.float()) < 2e-2
    pkg.check_status()
