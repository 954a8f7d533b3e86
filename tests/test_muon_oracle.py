"""The optimizer oracle (oracle/muon_oracle.py) against results of the reference's own `newton_schulz` and
`FusedMuon`, stored in tests/golden/muon.npz by tests/golden/make_golden_muon.py.  CPU only."""
import os

import numpy as np
import pytest
import torch

from oracle import muon_oracle as MO
from tests.golden.cases import (MUON_LR, MUON_MOMENTUM, MUON_NS_CASES, MUON_STEP_CASES, muon_ns_input,
                                muon_step_inputs)

GOLD = np.load(os.path.join(os.path.dirname(__file__), "golden", "muon.npz"))


@pytest.mark.parametrize("name", list(MUON_NS_CASES))
def test_newton_schulz_fp32_matches_reference(name):
    got = MO.newton_schulz(muon_ns_input(name), ns_dtype=torch.float32)
    ref = torch.from_numpy(GOLD[f"ns_{name}_f32"])
    assert got.shape == ref.shape
    assert MO.rel_l2(got, ref) < 1e-5


@pytest.mark.parametrize("name", list(MUON_NS_CASES))
def test_newton_schulz_bf16_close_to_reference_bf16(name):
    # different rounding points inside the bf16 products (library GEMM with folded axpy against product-then-axpy):
    # same algorithm, agreement at the level of bf16 noise after ten iterations
    got = MO.newton_schulz(muon_ns_input(name), ns_dtype=torch.bfloat16)
    ref = torch.from_numpy(GOLD[f"ns_{name}_bf16"])
    assert MO.rel_l2(got, ref) < 5e-2
    assert MO.rel_l2(got, torch.from_numpy(GOLD[f"ns_{name}_f32"])) < 5e-2


def test_singular_values_near_one():
    # the reference's own stability gate (bench.py:1054-1058): mean singular value in [0.8, 1.2], no NaN
    Y = MO.newton_schulz(muon_ns_input("tall"), ns_dtype=torch.bfloat16).float()
    sv = torch.linalg.svdvals(Y)
    assert not Y.isnan().any() and 0.8 <= sv.mean().item() <= 1.2


@pytest.mark.parametrize("name", list(MUON_STEP_CASES))
def test_step_matches_reference(name):
    _shape, _seed, mode, nesterov, wd, steps = MUON_STEP_CASES[name]
    p0, grads = muon_step_inputs(name)
    p, mom = p0.clone(), torch.zeros_like(p0)
    for i in range(steps):
        MO.muon_step(p, grads[i], mom, MUON_LR, MUON_MOMENTUM, nesterov, wd, ns_dtype=torch.float32, scale_mode=mode)
    # the reference's own gate for this comparison is max |dp| < 1e-4 (bench.py:1048-1049)
    assert (p - torch.from_numpy(GOLD[f"step_{name}_p"])).abs().max().item() < 1e-5
    assert MO.rel_l2(mom, torch.from_numpy(GOLD[f"step_{name}_mom"])) < 1e-6


def test_unknown_scale_mode_is_rejected():
    p = torch.zeros(1, 8, 8)
    with pytest.raises(ValueError):
        MO.muon_step(p, p.clone(), p.clone(), 0.1, scale_mode="no_such_mode")


from tests.golden.cases import MUON_MODE_CASES   # noqa: E402


@pytest.mark.parametrize("name", list(MUON_MODE_CASES))
def test_per_row_modes_and_two_pass_aurora_match_reference(name):
    """normuon, aurora_ema, aurora_ema_v2 and aurora with two passes against the reference's FusedMuon (fp32)."""
    shape, _seed, mode, nesterov, wd, steps, k = MUON_MODE_CASES[name]
    p0, grads = muon_step_inputs(name)
    p, mom = p0.clone(), torch.zeros_like(p0)
    v = torch.zeros(shape[0], shape[1])
    for i in range(steps):
        MO.muon_step(p, grads[i], mom, MUON_LR, MUON_MOMENTUM, nesterov, wd, ns_dtype=torch.float32, scale_mode=mode,
                     aurora_k=k or 1, scale_v=v)
    assert (p - torch.from_numpy(GOLD[f"step_{name}_p"])).abs().max().item() < 1e-5
    assert MO.rel_l2(mom, torch.from_numpy(GOLD[f"step_{name}_mom"])) < 1e-6
    if f"step_{name}_v" in GOLD.files:
        assert MO.rel_l2(v, torch.from_numpy(GOLD[f"step_{name}_v"])) < 1e-5
