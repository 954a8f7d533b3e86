"""Generate router.npz by running the REFERENCE's own router kernels under the Triton interpreter on the CPU.

    python tests/golden/make_golden_router.py /path/to/triton-kernel-fused

With TRITON_INTERPRET=1 (set below, before triton is imported) the reference's Triton kernels run on CPU tensors,
so its fused router needs no GPU.  From the reference's kernels/sm75/router.py this calls
  * `_epilogue_fwd` (:129-148, kernel :39-83) and `_router_epilogue_bwd_kernel` (:86-126) on the epilogue cases of
    tests/golden/cases.py (tie-free fp32 logits; logits on a coarse grid and in bf16, where every row holds exact
    ties; with and without bias, norm_topk on and off, scale != 1, k in {1,2,4,6,8}, E in {8..256});
  * `_count_experts` (:151-169) on the picks of every epilogue case;
  * `FusedMLPRouter.apply` (:221-260) and `FusedConvRouterCuDNN.apply` (:172-218) forward + backward;
  * `router_bias_update` (:292-301).
and stores idx / w / counts / grad_logits / grad_x / grad_weight per case.  Inputs are reproducible from their
seeds, so only outputs are stored.
"""
import os
import sys

os.environ["TRITON_INTERPRET"] = "1"

import numpy as np   # noqa: E402
import torch         # noqa: E402

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)
REF = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("REFERENCE_DIR", "")
if not REF:
    raise SystemExit("usage: make_golden_router.py /path/to/reference-checkout")
sys.path.insert(0, REF)

import triton   # noqa: E402
from kernels.sm75 import router as R   # noqa: E402  (the reference itself)

from tests.golden.cases import ROUTER_EPI_CASES, ROUTER_FULL_CASES, router_epi_inputs, router_full_inputs  # noqa: E402


def epilogue_bwd(logits, idx, grad_w, norm, scale):
    """The launch of the reference's backward epilogue kernel, as FusedMLPRouter.backward makes it (:252-257)."""
    N, E = logits.shape
    k = idx.shape[1]
    gl = torch.empty(N, E, dtype=logits.dtype)
    gw = grad_w.contiguous()
    BLOCK_N = 128
    R._router_epilogue_bwd_kernel[(triton.cdiv(N, BLOCK_N),)](
        logits, idx, gw, gl, N, logits.stride(0), logits.stride(1), idx.stride(0), idx.stride(1),
        gw.stride(0), gw.stride(1), gl.stride(0), gl.stride(1), float(scale), NORM=bool(norm and k > 1),
        E=E, TOPK=k, BLOCK_N=BLOCK_N, BLOCK_E=max(16, triton.next_power_of_2(E)))
    return gl


def main():
    out = {}
    for name, (N, E, k, norm, scale, _ub, _kind, _seed) in ROUTER_EPI_CASES.items():
        logits, bias, grad_w = router_epi_inputs(name)
        idx, w, counts = R._epilogue_fwd(logits, bias, k, E, norm_topk=norm, scale=scale)
        gl = epilogue_bwd(logits, idx, grad_w, norm, scale)
        out[f"epi.{name}.idx"] = idx.numpy()
        out[f"epi.{name}.w"] = w.numpy()
        out[f"epi.{name}.counts"] = counts.numpy()
        out[f"epi.{name}.grad_logits"] = gl.float().numpy()
        out[f"epi.{name}.counts_kernel"] = R._count_experts(idx, E).numpy()
        print("epilogue", name, counts.tolist()[:8])
    for name, (B, S, H, E, k, K, norm, scale, _ub, _seed) in ROUTER_FULL_CASES.items():
        x, w, bias, grad_w = router_full_inputs(name)
        xl, wl = x.clone().requires_grad_(True), w.clone().requires_grad_(True)
        fn = R.FusedConvRouterCuDNN if K else R.FusedMLPRouter
        idx, wt, counts = fn.apply(xl, wl, bias, k, E, norm, scale)
        (wt * grad_w).sum().backward()
        out[f"full.{name}.idx"] = idx.numpy()
        out[f"full.{name}.w"] = wt.detach().numpy()
        out[f"full.{name}.counts"] = counts.numpy()
        out[f"full.{name}.grad_x"] = xl.grad.numpy()
        out[f"full.{name}.grad_weight"] = wl.grad.numpy()
        print("router", name, counts.tolist()[:8])
    # the load-balance step
    bias = torch.linspace(-0.1, 0.1, 16)
    counts = torch.tensor([5, 0, 9, 4, 4, 7, 1, 12, 3, 3, 8, 2, 6, 4, 4, 0], dtype=torch.int32)
    b1 = bias.clone()
    R.router_bias_update(b1, counts, 0.01)
    b0 = bias.clone()
    R.router_bias_update(b0, counts, 0.0)
    out["bias_update.in"] = bias.numpy()
    out["bias_update.counts"] = counts.numpy()
    out["bias_update.out"] = b1.numpy()
    out["bias_update.out_u0"] = b0.numpy()
    np.savez_compressed(os.path.join(HERE, "router.npz"), **out)


if __name__ == "__main__":
    main()
