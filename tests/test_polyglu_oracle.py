"""CPU: the PolyGLU restatement of the oracle against the reference's own moe_eager outputs
(tests/golden/polyglu.npz: heterogeneous act codes, Identity/Zero experts, learnable SiTU)."""
import os

import numpy as np
import pytest
import torch

from oracle import moe_oracle as O
from tests.golden.cases import POLY_CASES, poly_inputs


@pytest.fixture(scope="module")
def poly_golden(golden_dir):
    return np.load(os.path.join(golden_dir, "polyglu.npz"))


@pytest.mark.parametrize("name", list(POLY_CASES))
def test_polyglu_oracle_matches_reference(poly_golden, name):
    c = poly_inputs(name)
    h, wt, gu, dn = (c[k].clone().requires_grad_(True) for k in ("hidden", "w", "gate_up", "down"))
    ap = c["act_params"].clone().requires_grad_(True) if c["act_params"] is not None else None
    out = O.moe_experts_polyglu(h, c["idx"], wt, gu, dn, c["codes"], ap)
    (out * c["grad_out"]).sum().backward()
    g = lambda k: torch.from_numpy(poly_golden[f"{name}.{k}"]).float()
    tol = 2e-3        # the fixture stores fp16
    assert O.rel_l2(out.detach(), g("out")) < tol
    assert O.rel_l2(h.grad, g("grad_hidden")) < tol
    assert O.rel_l2(wt.grad, g("grad_w")) < 1e-4
    assert O.rel_l2(gu.grad[:, ::4, ::4], g("grad_gate_up_sub")) < tol
    assert O.rel_l2(dn.grad[:, ::4, ::4], g("grad_down_sub")) < tol
    assert abs(float(gu.grad.double().norm()) - float(poly_golden[f"{name}.grad_gate_up_norm"])) < 1e-4 * float(gu.grad.norm())
    if f"{name}.grad_act_params" in poly_golden.files and ap is not None and ap.grad is not None:
        assert O.rel_l2(ap.grad, g("grad_act_params")) < 1e-4
