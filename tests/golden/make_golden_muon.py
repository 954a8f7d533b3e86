"""Generate muon.npz by running the REFERENCE's own optimizer code on the CPU.

    python tests/golden/make_golden_muon.py /path/to/triton-kernel-fused

It imports `newton_schulz` and `FusedMuon` from the reference's kernels/sm75/muon.py (pure PyTorch, runs on the
CPU), feeds them the seeded inputs of tests/golden/cases.py and stores
  * ns_<case>_f32 / ns_<case>_bf16 : newton_schulz(G, ns_dtype=float32 / bfloat16) of the reference;
  * step_<case>_p / step_<case>_mom: the parameters and the momentum buffer after the case's last step of
                                     FusedMuon(ns_dtype=float32) in the case's scale mode (polar, aurora with one
                                     and two passes, normuon, aurora_ema, aurora_ema_v2), and step_<case>_v, the
                                     per-row EMA state of the modes that keep one.
Inputs are reproducible from their seeds, so only outputs are stored.
"""
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)
REF = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("REFERENCE_DIR", "")
if not REF:
    raise SystemExit("usage: make_golden_muon.py /path/to/reference-checkout")
sys.path.insert(0, REF)

from kernels.sm75.muon import FusedMuon, newton_schulz   # noqa: E402  (the reference itself)

from tests.golden.cases import (MUON_LR, MUON_MODE_CASES, MUON_MOMENTUM, MUON_NS_CASES, MUON_STEP_CASES,  # noqa: E402
                                muon_ns_input, muon_step_inputs)


def main():
    out = {}
    for name in MUON_NS_CASES:
        G = muon_ns_input(name)
        out[f"ns_{name}_f32"] = newton_schulz(G, ns_dtype=torch.float32).numpy()
        out[f"ns_{name}_bf16"] = newton_schulz(G, ns_dtype=torch.bfloat16).numpy()
    for name, (_shape, _seed, mode, nesterov, wd, steps) in MUON_STEP_CASES.items():
        p0, grads = muon_step_inputs(name)
        p = torch.nn.Parameter(p0.clone())
        opt = FusedMuon([p], lr=MUON_LR, momentum=MUON_MOMENTUM, nesterov=nesterov, weight_decay=wd,
                        ns_dtype=torch.float32, scale_mode=mode)
        for i in range(steps):
            p.grad = grads[i].clone()
            opt.step()
        out[f"step_{name}_p"] = p.detach().clone().numpy()
        out[f"step_{name}_mom"] = opt.state[p]["muon_mom"].float().numpy()
    for name, (_shape, _seed, mode, nesterov, wd, steps, k) in MUON_MODE_CASES.items():
        p0, grads = muon_step_inputs(name)
        p = torch.nn.Parameter(p0.clone())
        opt = FusedMuon([p], lr=MUON_LR, momentum=MUON_MOMENTUM, nesterov=nesterov, weight_decay=wd,
                        ns_dtype=torch.float32, scale_mode=mode, aurora_k=k)
        for i in range(steps):
            p.grad = grads[i].clone()
            opt.step()
        out[f"step_{name}_p"] = p.detach().clone().numpy()
        out[f"step_{name}_mom"] = opt.state[p]["muon_mom"].float().numpy()
        if "scale_v" in opt.state[p]:
            out[f"step_{name}_v"] = opt.state[p]["scale_v"].float().numpy()
    np.savez_compressed(os.path.join(HERE, "muon.npz"), **out)
    print("wrote muon.npz:", {k: v.shape for k, v in out.items()})


if __name__ == "__main__":
    main()
