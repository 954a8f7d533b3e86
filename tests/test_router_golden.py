"""The router against fixtures made by the reference's OWN kernels (tests/golden/make_golden_router.py runs
kernels/sm75/router.py under the Triton interpreter on CPU tensors and stores tests/golden/router.npz).

CPU tests pin the oracle's restatement on those outputs; the GPU tests hold the CUDA kernels to the same
fixtures through the C ABI.  Gates: picked experts and counts bit-exact (also where rows are full of exact
ties), weights <= 1e-6, gradients <= 1e-5 relative L2 (bf16-stored gradients: one bf16 rounding)."""
import os

import numpy as np
import pytest
import torch

from oracle import moe_oracle as O
from tests.golden.cases import ROUTER_EPI_CASES, ROUTER_FULL_CASES, router_epi_inputs, router_full_inputs

DEV = "cuda"


@pytest.fixture(scope="module")
def gold(golden_dir):
    return np.load(os.path.join(golden_dir, "router.npz"))


def _t(a):
    return torch.from_numpy(np.asarray(a))


# ----------------------------------------------------------------------------- CPU: oracle vs reference
@pytest.mark.parametrize("name", list(ROUTER_EPI_CASES))
def test_oracle_epilogue_matches_reference_kernels(gold, name):
    N, E, k, norm, scale, _ub, kind, _seed = ROUTER_EPI_CASES[name]
    logits, bias, grad_w = router_epi_inputs(name)
    idx, w, counts = O.router_epilogue_fwd(logits, bias, k, norm, scale)
    assert torch.equal(idx, _t(gold[f"epi.{name}.idx"]))                 # ties included: lowest index first
    assert torch.equal(counts, _t(gold[f"epi.{name}.counts"]))
    assert torch.equal(counts, _t(gold[f"epi.{name}.counts_kernel"]))    # the reference's stand-alone bincount kernel
    assert O.rel_l2(w, _t(gold[f"epi.{name}.w"])) < 1e-6
    assert O.router_epilogue_bwd(logits, idx, grad_w, norm, scale).dtype == logits.dtype   # router.py:250
    gl = O.router_epilogue_bwd(logits, idx, grad_w, norm, scale, out_dtype=torch.float32)
    if kind == "bf16":
        # the Triton interpreter stores fp32 -> bf16 by dropping the low 16 bits (checked: the fixture equals the
        # truncated fp32 values bit for bit; a GPU rounds to nearest), so the fp32 result is truncated the same way
        gl = (gl.view(torch.int32) & ~0xFFFF).view(torch.float32)
    assert O.rel_l2(gl, _t(gold[f"epi.{name}.grad_logits"])) < 1e-5


def test_fixture_holds_real_ties(gold):
    """The grid cases are there for the tie rule: most rows must hold a tie among the picked scores."""
    for name in ("grid_e64_k6_bias", "grid_e256_k8", "bf16_e64_k6"):
        logits, bias, _ = router_epi_inputs(name)
        k = ROUTER_EPI_CASES[name][2]
        sel = O.sigmoid_scores(logits) + (bias if bias is not None else 0.0)
        idx = _t(gold[f"epi.{name}.idx"])
        picked = sel.gather(1, idx)
        tied_rows = (picked[:, 1:] == picked[:, :-1]).any(1).float().mean()
        assert tied_rows > 0.5, (name, float(tied_rows))
        # and inside a tie the lower expert index comes first
        same = picked[:, 1:] == picked[:, :-1]
        assert bool((idx[:, 1:][same] > idx[:, :-1][same]).all())
        assert bool((picked[:, 1:] <= picked[:, :-1]).all())             # picks in descending order of sel


def _oracle_full(name):
    B, S, H, E, k, K, norm, scale, _ub, _seed = ROUTER_FULL_CASES[name]
    x, w, bias, grad_w = router_full_inputs(name)
    if K == 0:
        idx, wt, counts, logits = O.mlp_router_fwd(x, w, bias, k, norm, scale)
        gx, gw, _ = O.mlp_router_bwd(x, w, logits, idx, grad_w, norm, scale)
        return idx, wt, counts, gx, gw
    xl, wl = x.clone().requires_grad_(True), w.clone().requires_grad_(True)
    logits = O.conv_router_logits(xl, wl)
    idx, wt, counts = O.router_epilogue_fwd(logits.detach(), bias, k, norm, scale)
    gl = O.router_epilogue_bwd(logits.detach(), idx, grad_w, norm, scale)
    logits.backward(gl)
    return idx, wt, counts, xl.grad, wl.grad


@pytest.mark.parametrize("name", list(ROUTER_FULL_CASES))
def test_oracle_whole_router_matches_reference(gold, name):
    """FusedMLPRouter / FusedConvRouterCuDNN of the reference, forward and backward, against the oracle."""
    idx, wt, counts, gx, gw = _oracle_full(name)
    assert torch.equal(idx, _t(gold[f"full.{name}.idx"]))
    assert torch.equal(counts, _t(gold[f"full.{name}.counts"]))
    assert O.rel_l2(wt, _t(gold[f"full.{name}.w"])) < 1e-6
    assert O.rel_l2(gx, _t(gold[f"full.{name}.grad_x"])) < 1e-5
    assert O.rel_l2(gw, _t(gold[f"full.{name}.grad_weight"])) < 1e-5


def test_oracle_bias_update_matches_reference(gold):
    b = _t(gold["bias_update.in"]).clone()
    O.router_bias_update(b, _t(gold["bias_update.counts"]), 0.01)
    assert torch.equal(b, _t(gold["bias_update.out"]))
    b0 = _t(gold["bias_update.in"]).clone()
    O.router_bias_update(b0, _t(gold["bias_update.counts"]), 0.0)
    assert torch.equal(b0, _t(gold["bias_update.out_u0"]))


# ----------------------------------------------------------------------------- GPU: CUDA kernels vs reference
@pytest.mark.gpu
@pytest.mark.parametrize("name", list(ROUTER_EPI_CASES))
def test_cuda_topk_from_identical_scores_matches_reference_picks(pkg, gold, name):
    """Given identical fp32 scores the CUDA top-k reproduces the reference kernel's picks, order and counts bit for
    bit, and its weights."""
    N, E, k, norm, scale, _ub, _kind, _seed = ROUTER_EPI_CASES[name]
    logits, bias, _ = router_epi_inputs(name)
    s = O.sigmoid_scores(logits)
    idx, w, c = pkg.ops.router_topk_fwd(s.to(DEV), None if bias is None else bias.to(DEV), k, norm, scale, scores=True)
    assert torch.equal(idx.cpu(), _t(gold[f"epi.{name}.idx"]))
    assert torch.equal(c.cpu(), _t(gold[f"epi.{name}.counts"]))
    assert O.rel_l2(w.cpu(), _t(gold[f"epi.{name}.w"])) < 1e-6


@pytest.mark.gpu
@pytest.mark.parametrize("name", list(ROUTER_EPI_CASES))
def test_cuda_epilogue_from_logits_matches_reference(pkg, gold, name):
    """From the logits themselves (the device computes the sigmoid): forward picks and the backward Jacobian."""
    N, E, k, norm, scale, _ub, kind, _seed = ROUTER_EPI_CASES[name]
    logits, bias, grad_w = router_epi_inputs(name)
    idx, w, c = pkg.ops.router_topk_fwd(logits.to(DEV), None if bias is None else bias.to(DEV), k, norm, scale)
    ref_idx = _t(gold[f"epi.{name}.idx"])
    # equal logits give equal scores on any device, so every tie is kept; a pick can only differ where two
    # DIFFERENT scores lie within one ulp of the device's exp, which none of these seeded cases contains
    assert torch.equal(idx.cpu(), ref_idx)
    assert torch.equal(c.cpu(), _t(gold[f"epi.{name}.counts"]))
    assert O.rel_l2(w.cpu(), _t(gold[f"epi.{name}.w"])) < 1e-6
    gl = pkg.ops.router_topk_bwd(logits.to(DEV), ref_idx.to(DEV), grad_w.to(DEV), norm, scale)
    # the device stores grad_logits in bf16, round to nearest: one bf16 rounding from the fp32 fixture (two for
    # the bf16 cases, whose fixture the interpreter truncated)
    assert O.rel_l2(gl.float().cpu(), _t(gold[f"epi.{name}.grad_logits"])) < (8e-3 if kind == "bf16" else 4e-3)


@pytest.mark.gpu
def test_cuda_bias_update_matches_reference(pkg, gold):
    b = _t(gold["bias_update.in"]).clone().to(DEV)
    pkg.router_bias_update(b, _t(gold["bias_update.counts"]).to(DEV), 0.01)
    assert torch.equal(b.cpu(), _t(gold["bias_update.out"]))
