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


def test_muon_rejects_what_is_not_built_and_cpu_tensors():
    """Constructor checks of the optimizer and the device check of newton_schulz run before any launch."""
    import pytest
    pkg = importlib.import_module(PKG)
    p = torch.nn.Parameter(torch.zeros(2, 64, 64))
    for kw in (dict(scale_mode="no_such_mode"), dict(aurora_k=0), dict(ns_dtype=torch.float32),
               dict(xorth_post=0.1), dict(spectral_wd=0.1)):
        with pytest.raises(ValueError):
            pkg.FusedMuon([p], **kw)
    for mode in ("polar", "aurora", "normuon", "aurora_ema", "aurora_ema_v2"):     # every mode of the reference
        assert pkg.FusedMuon([p], scale_mode=mode, aurora_k=2, use_graph=True).scale_mode == mode
    opt = pkg.FusedMuon([p], lr=0.1, scale_mode="polar")
    opt.step()                                   # no gradient: nothing is stepped, nothing is launched
    assert float(p.detach().abs().sum()) == 0.0 and not opt.state[p]
    p.grad = torch.ones_like(p)
    with pytest.raises(ValueError):              # a CPU parameter never reaches the library
        opt.step()
    with pytest.raises(ValueError):
        pkg.newton_schulz(torch.zeros(8, 8))


def test_muon_uniform_segment_tables():
    """The row tables that stand in for a routing decision when the grouped GEMMs run over a stack."""
    pkg = importlib.import_module(PKG)
    seg = pkg.muon._uniform_segments(3, 512, "cpu")
    assert seg.cap == 1536 and seg.E == 3
    assert seg.poffs.tolist() == [0, 512, 1024, 1536]
    assert seg.tile_expert.tolist() == [0, 0, 1, 1, 2, 2]
    assert seg.tile_expert.dtype == torch.int32 and seg.poffs.dtype == torch.int32


def test_muon_accepts_the_reference_argument_list():
    """Every keyword of the reference's FusedMuon constructor is accepted; the ones that act only together with
    rejected options are ignored, a group that switches whitening on is rejected at step time."""
    import pytest
    pkg = importlib.import_module(PKG)
    p = torch.nn.Parameter(torch.zeros(2, 64, 64))
    opt = pkg.FusedMuon([{"params": [p], "xorth_post": 0.01}], lr=3e-4, momentum=0.95, nesterov=True, weight_decay=0.0,
                        ns_dtype=None, scale_mode="aurora", ns_batch_elems=4 * 1024 * 1024, use_graph=False,
                        graph_warmup=3, aurora_k=None, spectral_wd=0.0, swd_beta=0.99, xorth_post=0.0,
                        xorth_backend="ns", xorth_ns_iters=18, xorth_ema=0.95, xorth_gate_ref=0.3,
                        xorth_warmup_steps=0, xorth_where="post")
    p.grad = torch.zeros_like(p)
    with pytest.raises(ValueError):
        opt.step()


def test_muon_momentum_buffer_is_checked_before_the_kernel_sees_it():
    """A momentum buffer that `load_state_dict` cast to fp32 comes back as bf16 with the same values; a buffer of
    another size is refused (the kernel would otherwise read and write out of bounds)."""
    import pytest
    pkg = importlib.import_module(PKG)
    check = pkg.muon._checked_momentum
    cpu = torch.device("cpu")
    m = (torch.randn(2, 8, 16) * 0.1).to(torch.bfloat16)
    assert check(m, 2, 8, 16, cpu) is m                       # already right: passed through untouched
    back = check(m.float(), 2, 8, 16, cpu)
    assert back.dtype == torch.bfloat16 and torch.equal(back, m)
    flat = check(m.float().view(-1), 2, 8, 16, cpu)
    assert flat.shape == (2, 8, 16) and torch.equal(flat, m)
    for bad in (torch.zeros(1, 8, 16), torch.zeros(2, 8, 8), None):
        with pytest.raises(ValueError):
            check(bad, 2, 8, 16, cpu)


def test_status_codes_become_runtime_errors():
    """What a kernel leaves in the status word reaches the caller as a RuntimeError naming the cause; 7 is the
    cross-rank barrier that gave up waiting for a peer."""
    import pytest
    L = importlib.import_module(PKG + "._lib")
    L.raise_for_status(0)
    with pytest.raises(RuntimeError, match="peer rank did not arrive"):
        L.raise_for_status(7)
    with pytest.raises(RuntimeError, match="expert index"):
        L.raise_for_status(5)
    # argument errors of the barrier never reach the GPU
    lib = L.lib()
    assert lib.b200moe_ep_barrier(None, 2, 0, 1, 10**6, None, None) < 0
    assert b"status" in lib.b200moe_last_error_string()


def test_bf16_copies_of_frozen_stacks_are_reused_until_the_stack_changes():
    """fp32 / fp16 callers: the bf16 copy of an expert stack that needs no gradient is made once and reused until the
    stack is updated in place or freed; stacks that need a gradient are cast afresh (autograd needs the cast)."""
    moe_mod = importlib.import_module(PKG + ".moe")
    w = torch.randn(2, 8, 4)
    a = moe_mod._bf16_copy(w)
    assert a.dtype == torch.bfloat16 and moe_mod._bf16_copy(w) is a
    w.mul_(2.0)                                           # an optimizer step moves the version counter
    b = moe_mod._bf16_copy(w)
    assert b is not a and torch.equal(b, w.to(torch.bfloat16))
    p = torch.nn.Parameter(torch.randn(2, 8, 4))
    c = moe_mod._bf16_copy(p)
    assert c.requires_grad and moe_mod._bf16_copy(p) is not c
    with torch.no_grad():
        assert moe_mod._bf16_copy(p) is moe_mod._bf16_copy(p)
    n = len(moe_mod._BF16_COPIES)
    del w, a, b
    import gc
    gc.collect()
    assert len(moe_mod._BF16_COPIES) == n - 1             # freed with its tensor


def test_expert_groups_split_local_experts_by_rows():
    """The expert-parallel pipeline's grouping: consecutive experts, about equal padded rows, empty groups dropped,
    every row in exactly one group."""
    ep = importlib.import_module("triton-kernel-fused_b200.ep_p2p")
    ends = [256, 512, 768, 1024, 1280, 1536, 1792, 2048]
    assert ep.expert_groups(ends, 2) == [(0, 4, 0, 1024), (4, 8, 1024, 2048)]
    assert ep.expert_groups(ends, 4) == [(0, 2, 0, 512), (2, 4, 512, 1024), (4, 6, 1024, 1536), (6, 8, 1536, 2048)]
    assert ep.expert_groups(ends, 1) == [(0, 8, 0, 2048)]
    # one expert holds nearly everything: the cut falls behind it, nothing is lost, nothing is empty
    skew = [256, 256, 5120, 5376]
    for n in (2, 3, 4, 7):
        g = ep.expert_groups(skew, n)
        assert g[0][0] == 0 and g[-1][1] == 4 and g[0][2] == 0 and g[-1][3] == 5376
        assert all(a[1] == b[0] and a[3] == b[2] for a, b in zip(g, g[1:]))
        assert all(r_hi > r_lo for _, _, r_lo, r_hi in g)
    # experts without rows (ends repeat) and a rank without any row
    assert ep.expert_groups([0, 0, 256, 256], 2) == [(0, 3, 0, 256)] or ep.expert_groups([0, 0, 256, 256], 2) == [(0, 4, 0, 256)]
    assert ep.expert_groups([0, 0, 0, 0], 2) == []
    assert ep.expert_groups([], 2) == []


def test_load_telemetry_figures():
    """`load_stats` of the layers' load-balance mixin: the figures follow from the accumulated counts."""
    layer_mod = importlib.import_module("triton-kernel-fused_b200.layer")

    class Loop(layer_mod.LoadBalanceMixin, torch.nn.Module):
        def __init__(self):
            super().__init__()
            self._init_load(4)

    loop = Loop()
    assert loop.load_stats() == {"load": [0, 0, 0, 0], "tokens_routed": 0, "max_over_mean": 0.0, "min_over_mean": 0.0,
                                 "cv": 0.0, "idle_experts": 4}
    loop._record_counts(torch.tensor([6, 2, 0, 0], dtype=torch.int32))
    loop._record_counts(torch.tensor([2, 2, 4, 0], dtype=torch.int32))
    st = loop.load_stats()
    assert st["load"] == [8, 4, 4, 0] and st["tokens_routed"] == 16 and st["idle_experts"] == 1
    assert st["max_over_mean"] == 2.0 and st["min_over_mean"] == 0.0
    assert abs(st["cv"] - (8.0 ** 0.5) / 4.0) < 1e-12          # std of (8,4,4,0) = sqrt(8), mean 4


def test_fixed_capacity_rows():
    """Sizing of the expert-parallel layer's fixed-capacity buffers: factor x own routed rows, rounded up, clamped to
    the rows that exist; nonsense factors are refused before anything is allocated."""
    import pytest
    ep = importlib.import_module("triton-kernel-fused_b200.ep_p2p")
    assert ep.fixed_capacity_rows(8, 16384, 6, 1.5) == 147456
    assert ep.fixed_capacity_rows(8, 1000, 3, 1.0001) == 3001          # rounded up
    assert ep.fixed_capacity_rows(2, 1024, 4, 5.0) == 2 * 4096          # never more rows than exist
    assert ep.fixed_capacity_rows(4, 10, 2, 0.25) == 5
    for bad in (0, -1.0, float("nan")):
        with pytest.raises(ValueError):
            ep.fixed_capacity_rows(2, 8, 2, bad)
