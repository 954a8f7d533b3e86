"""CPU: host-side logic of the package that needs no kernel launch."""
import importlib

import torch

PKG = "triton-kernel-fused_b200"


def test_empty_batch_never_reaches_the_library():
    """T = 0: the public callables return empty results that still carry zero gradients, before any pointer is
    handed to the C ABI (so this runs without a GPU)."""
    pkg = importlib.import_module(PKG)
    H, I, E, k = 64, 32, 4, 2
    gu = torch.randn(E, 2 * I, H, requires_grad=True)
    dn = torch.randn(E, H, I, requires_grad=True)
    x = torch.zeros(0, H, requires_grad=True)
    w = torch.zeros(0, k, requires_grad=True)
    codes = torch.zeros(E, dtype=torch.int32)
    for fn in (pkg.moe, pkg.moe_grouped, pkg.moe_mxfp8):
        out = fn(x, torch.zeros(0, k, dtype=torch.int64), w, gu, dn, codes)
        assert out.shape == (0, H)
        gu.grad = dn.grad = None
        out.sum().backward()
        assert gu.grad.shape == gu.shape and float(gu.grad.abs().sum()) == 0.0
        assert dn.grad.shape == dn.shape and float(dn.grad.abs().sum()) == 0.0
    gate = torch.randn(E, H, requires_grad=True)
    idx, wts, counts = pkg.fused_mlp_router(torch.zeros(3, 0, H, requires_grad=True), gate, None, k, E,
                                            return_counts=True)
    assert idx.shape == (3, 0, k) and idx.dtype == torch.int64
    assert wts.shape == (3, 0, k) and wts.dtype == torch.float32
    assert counts.tolist() == [0] * E and counts.dtype == torch.int32
    wts.sum().backward()
    assert float(gate.grad.abs().sum()) == 0.0


def test_unknown_activation_codes_raise_value_error():
    pkg = importlib.import_module(PKG)
    H, I, E, k = 64, 32, 2, 1
    args = (torch.zeros(4, H), torch.zeros(4, k, dtype=torch.int64), torch.ones(4, k), torch.zeros(E, 2 * I, H),
            torch.zeros(E, H, I))
    try:
        pkg.moe(*args, torch.tensor([0, 9], dtype=torch.int32))
    except ValueError:
        return
    raise AssertionError("act code 9 must be rejected")
