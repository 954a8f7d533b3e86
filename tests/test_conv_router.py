"""Conv router (`fused_router`): CPU checks of the oracle, GPU parity of the CUDA path."""
import pytest
import torch

from oracle import moe_oracle as O

DEV = "cuda"


def test_conv_logits_equal_unfolded_gemm():
    """The causal conv equals one GEMM over the unfolded input (the formulation the CUDA path uses)."""
    g = torch.Generator().manual_seed(0)
    B, S, H, E, K = 3, 17, 16, 5, 4
    x = torch.randn(B, S, H, generator=g)
    w = torch.randn(E, H, K, generator=g)
    ref = O.conv_router_logits(x, w)
    xu = torch.zeros(B, S, K, H)
    for j in range(K):
        sh = K - 1 - j
        xu[:, sh:, j] = x[:, :S - sh] if sh > 0 else x
    wf = w.permute(0, 2, 1).reshape(E, K * H)
    assert torch.allclose(xu.reshape(B * S, K * H) @ wf.t(), ref, atol=1e-5)
    # causality: changing x[b, s] never changes logits before s
    x2 = x.clone()
    x2[:, 10] += 1.0
    d = (O.conv_router_logits(x2, w) - ref).view(B, S, E).abs().amax(-1)
    assert (d[:, :10] == 0).all() and (d[:, 10:10 + K] > 0).all() and (d[:, 10 + K:] == 0).all()


@pytest.mark.gpu
@pytest.mark.parametrize("B,S,H,E,K", [(2, 256, 128, 64, 4), (3, 384, 320, 128, 2), (1, 128, 64, 64, 1),
                                       (5, 128, 512, 256, 3)])
def test_conv_gemms_without_the_unfolded_copy(pkg, B, S, H, E, K):
    """The GEMMs that read x in place through shifted TMA boxes against the same GEMMs over the unfolded copy:
    the forward runs the identical MMA sequence (bit-equal logits); dX and dW differ only in summation grouping."""
    ops = pkg.ops
    g = torch.Generator().manual_seed(9)
    x = torch.randn(B, S, H, generator=g).to(torch.bfloat16).to(DEV)
    w = (torch.randn(E, H, K, generator=g) * 0.05).to(torch.bfloat16).to(DEV)
    gl = torch.randn(B * S, E, generator=g).to(torch.bfloat16).to(DEV)
    assert ops.conv_direct_ok(S, H)
    wf = w.permute(0, 2, 1).reshape(E, K * H).contiguous()
    wb = w.permute(2, 0, 1).reshape(K * E, H).contiguous()
    xu = ops.conv_unfold(x, K)
    assert torch.equal(ops.conv_gemm_fwd(x, wf, K), ops.gemm_nt(xu, wf))
    gx_ref = ops.conv_fold(ops.gemm_nn(gl, wf), B, S, H, K)
    gx = ops.conv_gemm_dx(gl, wb, B, S, K)
    assert O.rel_l2(gx.float().cpu(), gx_ref.float().cpu()) < 6e-3
    # fp32 reference of dX: the fold of the fp32 product
    gxu32 = (gl.float() @ wf.float()).view(B, S, K, H)
    gx32 = torch.zeros(B, S, H, device=DEV)
    for j in range(K):
        sh = K - 1 - j
        gx32[:, :S - sh] += gxu32[:, sh:, j]
    assert O.rel_l2(gx.float().cpu(), gx32.cpu()) < 4e-3
    gw = ops.conv_gemm_dw(gl, x, K)
    gw32 = gl.float().t() @ xu.float()
    assert O.rel_l2(gw.float().cpu(), gw32.cpu()) < 4e-3
    assert O.rel_l2(ops.gemm_tn(gl, xu).float().cpu(), gw32.cpu()) < 4e-3
    pkg.check_status()


@pytest.mark.gpu
@pytest.mark.parametrize("B,S,H,E,K,k", [(4, 512, 256, 16, 4, 2), (2, 300, 512, 64, 3, 6), (2, 256, 128, 64, 4, 2),
                                         (3, 384, 320, 128, 2, 4)])
def test_fused_conv_router_forward_backward(pkg, B, S, H, E, K, k):
    g = torch.Generator().manual_seed(5)
    x = torch.randn(B, S, H, generator=g).to(torch.bfloat16)
    w = (torch.randn(E, H, K, generator=g) * 0.02).to(torch.bfloat16)
    bias = torch.randn(E, generator=g) * 0.01
    G = torch.randn(B, S, k, generator=g)
    xd = x.to(DEV).requires_grad_(True)
    wd = w.to(DEV).requires_grad_(True)
    idx, wt, counts = pkg.fused_router(xd, wd, bias.to(DEV), k, E, return_counts=True)
    assert idx.shape == (B, S, k) and wt.dtype == torch.float32
    (wt * G.to(DEV)).sum().backward()
    pkg.check_status()
    # oracle: same bf16 inputs, logits rounded to bf16 like the CUDA path
    xo = x.float().requires_grad_(True)
    wo = w.float().requires_grad_(True)
    logits = O.conv_router_logits(xo, wo)
    logits_r = logits + (logits.detach().to(torch.bfloat16).float() - logits.detach())
    idx_o, _, counts_o = O.router_epilogue_fwd(logits_r.detach(), bias, k)
    idx_dev = idx.view(B * S, k).cpu()
    # a logit on a bf16 rounding boundary can flip a pick: the flip rate is asserted on its own, the values are
    # compared on the device's picks at the 2e-2 gate
    assert (idx_dev != idx_o).any(1).float().mean() < 0.005
    s = torch.sigmoid(logits_r)
    ww = s.gather(1, idx_dev)
    ww = ww / (ww.sum(-1, keepdim=True) + 1e-20)
    (ww * G.view(B * S, k)).sum().backward()
    assert O.rel_l2(wt.view(B * S, k).cpu(), ww.detach()) < 1e-2
    assert torch.equal(counts.cpu().long(), torch.bincount(idx.flatten().cpu(), minlength=E))
    gx, gxo = xd.grad.float().cpu().view(B * S, H), xo.grad.view(B * S, H)
    assert O.rel_l2(gx, gxo) < 2e-2
    assert O.rel_l2(wd.grad.float().cpu(), wo.grad) < 2e-2
