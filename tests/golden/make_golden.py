"""Generate the golden fixtures in this folder by running the REFERENCE's own CPU-runnable code.

Run once on a machine that has a checkout of the reference; pass its path as argv[1] (or set
REFERENCE_DIR):   python tests/golden/make_golden.py /path/to/triton-kernel-fused

It imports `moe_eager` and `_sort_by_expert` from the reference's kernels/sm75/moe.py (they run on
the CPU), feeds them seeded inputs built by oracle.moe_oracle.make_inputs, and stores:
  * experts_<case>.npz : routing that was fed in (idx, w), the reference forward output and its
    autograd gradients w.r.t. hidden, top-k weights, gate_up_proj and down_proj.  Large weight
    gradients are stored sub-sampled ([:, ::8, ::8]) together with their full L2 norm and sum.
  * sort_<case>.npz    : counts, bounds and, per expert segment, the sorted token ids that the
    reference's (unstable) sort produced.
The fixtures are reproducible: inputs come from fixed seeds, so only outputs are stored.
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
    raise SystemExit("usage: make_golden.py /path/to/reference-checkout")
sys.path.insert(0, REF)

from kernels.sm75.moe import moe_eager, _sort_by_expert   # noqa: E402  (the reference itself)
from oracle import moe_oracle as O                        # noqa: E402

from tests.golden.cases import CASES, POLY_CASES, poly_inputs, routing_for, sub  # noqa: E402


def main():
    torch.manual_seed(0)
    for name, (T, H, E, I, k, seed, bstd, cap) in CASES.items():
        inp = O.make_inputs(T, H, E, I, k, seed=seed, bias_std=bstd)
        idx, w = routing_for(inp, E, k, cap)
        hidden = inp["x"].clone().requires_grad_(True)
        wt = w.clone().requires_grad_(True)
        gu = inp["gate_up"].clone().requires_grad_(True)
        dn = inp["down"].clone().requires_grad_(True)
        codes = torch.zeros(E, dtype=torch.int32)
        out = moe_eager(hidden, idx, wt, gu, dn, codes)
        (out * inp["grad_out"]).sum().backward()
        np.savez_compressed(
            os.path.join(HERE, f"experts_{name}.npz"),
            idx=idx.numpy(), w=w.numpy(), out=out.detach().numpy(),
            grad_hidden=hidden.grad.numpy(), grad_w=wt.grad.numpy(),
            grad_gate_up_sub=sub(gu.grad).numpy(), grad_down_sub=sub(dn.grad).numpy(),
            grad_gate_up_norm=np.float64(gu.grad.double().norm()),
            grad_down_norm=np.float64(dn.grad.double().norm()),
            grad_gate_up_sum=np.float64(gu.grad.double().sum()),
            grad_down_sum=np.float64(dn.grad.double().sum()))
        st, sw, order, counts, bounds = _sort_by_expert(idx, w, E)
        seg_sorted = torch.cat([torch.sort(st[bounds[e]:bounds[e + 1]]).values for e in range(E)])
        np.savez_compressed(
            os.path.join(HERE, f"sort_{name}.npz"),
            counts=np.asarray(counts, dtype=np.int64), bounds=np.asarray(bounds, dtype=np.int64),
            seg_sorted_tokens=seg_sorted.numpy())
        print(name, "out", tuple(out.shape), "counts", counts)
    # PolyGLU cases: the reference's moe_eager with heterogeneous act codes, specials and act_params
    poly = {}
    for name in POLY_CASES:
        c = poly_inputs(name)
        h, wt, gu, dn = (c[k].clone().requires_grad_(True) for k in ("hidden", "w", "gate_up", "down"))
        ap = c["act_params"].clone().requires_grad_(True) if c["act_params"] is not None else None
        codes = torch.tensor(c["codes"], dtype=torch.int32)
        out = moe_eager(h, c["idx"], wt, gu, dn, codes, ap)
        (out * c["grad_out"]).sum().backward()
        f16 = lambda t: t.detach().to(torch.float16).numpy()
        poly[f"{name}.out"] = f16(out)
        poly[f"{name}.grad_hidden"] = f16(h.grad)
        poly[f"{name}.grad_w"] = wt.grad.numpy()
        poly[f"{name}.grad_gate_up_sub"] = f16(gu.grad[:, ::4, ::4])
        poly[f"{name}.grad_down_sub"] = f16(dn.grad[:, ::4, ::4])
        poly[f"{name}.grad_gate_up_norm"] = np.float64(gu.grad.double().norm())
        poly[f"{name}.grad_down_norm"] = np.float64(dn.grad.double().norm())
        if ap is not None and ap.grad is not None:
            poly[f"{name}.grad_act_params"] = ap.grad.numpy()
        print("poly", name, float(out.abs().max()))
    np.savez_compressed(os.path.join(HERE, "polyglu.npz"), **poly)


if __name__ == "__main__":
    main()
