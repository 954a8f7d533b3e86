"""Case table and input helpers shared by the golden generator and the tests (no reference import)."""
from oracle import moe_oracle as O

# name -> (T, H, E, I, k, seed, bias_std, cap)   cap: route only to experts < cap (empty experts)
CASES = {
    "cfg1": (512, 256, 8, 512, 2, 0, 0.01, None),          # benchmark config 1
    "situ_small": (512, 128, 6, 96, 2, 7, 0.0, None),      # parity_situ.py:12 shape
    "empty_experts": (512, 128, 6, 96, 2, 7, 0.0, 4),      # parity_situ.py:93 (experts 4,5 empty)
    "grouped_k4": (1024, 128, 16, 64, 4, 3, 0.01, None),   # top-4, more experts
}


def sub(t):
    """Sub-sample of a large (E, rows, cols) weight gradient kept in the fixture."""
    return t[:, ::8, ::8].contiguous()


def routing_for(inp, E, k, cap):
    """Routing fed to the reference's moe_eager when the fixture was made."""
    logits = inp["x"] @ inp["gate_weight"].t()
    if cap is not None:
        logits = logits.clone()
        logits[:, cap:] = -1e4                 # sigmoid -> 0: never picked while cap >= k
    idx, w, counts = O.router_epilogue_fwd(logits, inp["bias"], k)
    return idx, w


# PolyGLU cases after parity_situ.py:79-106 of the reference: name -> (codes, use act_params, cap, I)
POLY_N, POLY_H, POLY_K = 256, 128, 2
POLY_CASES = {
    "all_situ": ([5] * 6, True, None, 96),
    "all_situ_raw": ([5] * 6, False, None, 96),
    "mixed_raw": ([0, 1, 2, 5, 0, 5], False, None, 96),
    "all_relu2": ([1] * 6, True, None, 96),
    "all_normsilu": ([2] * 6, True, None, 96),
    "all_normrelu2": ([6] * 6, True, None, 96),
    "all_normsitu": ([7] * 6, True, None, 96),
    "mixed_0125": ([0, 1, 2, 5, 0, 5], True, None, 96),
    "mixed_126": ([1, 2, 6, 6, 2, 1], True, None, 96),
    "mixed_257": ([2, 5, 7, 7, 5, 2], True, None, 96),
    "normrelu2_specials": ([6, 2, 6, 5, 3, 4], True, None, 96),
    "normsitu_specials": ([7, 2, 7, 5, 3, 4], True, None, 96),
    "situ_specials": ([0, 5, 2, 5, 3, 4], True, None, 96),
    "empty_experts_poly": ([5, 5, 5, 5, 0, 2], True, 4, 96),
    "mixed_wide": ([0, 1, 2, 5, 0, 5], True, None, 1536),
    "situ_specials_wide": ([0, 5, 2, 5, 3, 4], True, None, 1536),
}


def poly_inputs(name):
    """Seeded inputs of a PolyGLU case, scaled like parity_situ.py:15-27 (hidden*0.5, weights*0.1,
    uniform-random top-k routing, act_params in [0.5, 1.5))."""
    import torch
    codes, use_ap, cap, I = POLY_CASES[name]
    E = len(codes)
    n_glu = sum(1 for c in codes if c not in (3, 4))
    g = torch.Generator().manual_seed(sum(map(ord, name)))
    hid = torch.randn(POLY_N, POLY_H, generator=g) * 0.5
    gup = torch.randn(n_glu, 2 * I, POLY_H, generator=g) * 0.1
    dwn = torch.randn(n_glu, POLY_H, I, generator=g) * 0.1
    scores = torch.rand(POLY_N, cap or E, generator=g)
    wt, idx = scores.topk(POLY_K, dim=-1)
    wt = wt / wt.sum(-1, keepdim=True)
    ap = torch.stack([torch.rand(E, generator=g) + 0.5, torch.rand(E, generator=g) + 0.5], dim=1) if use_ap else None
    gsig = torch.randn(POLY_N, POLY_H, generator=g) * 0.1
    return dict(codes=codes, hidden=hid, gate_up=gup, down=dwn, idx=idx, w=wt, act_params=ap, grad_out=gsig, I=I)


# ---- expert-stack optimizer (Muon) cases: name -> (shape, seed).  Wide, tall, square stacks and one plain matrix.
MUON_NS_CASES = {
    "wide": ((3, 64, 96), 11),
    "tall": ((3, 96, 64), 12),
    "square": ((2, 64, 64), 13),
    "matrix": ((48, 80), 14),
}
# name -> (shape, seed, scale_mode, nesterov, weight_decay, steps)
MUON_STEP_CASES = {
    "polar_tall": ((4, 96, 64), 21, "polar", True, 0.1, 3),
    "polar_wide_plain_momentum": ((4, 64, 96), 22, "polar", False, 0.0, 3),
    "aurora_tall": ((4, 96, 64), 23, "aurora", True, 0.1, 3),
    "aurora_wide": ((4, 64, 96), 24, "aurora", True, 0.0, 3),
}
MUON_LR, MUON_MOMENTUM = 0.02, 0.95


def muon_ns_input(name):
    import torch
    shape, seed = MUON_NS_CASES[name]
    return torch.randn(*shape, generator=torch.Generator().manual_seed(seed))


def muon_step_inputs(name):
    """(initial parameters, list of per-step gradients), fp32, seeded."""
    import torch
    shape, seed, _mode, _nest, _wd, steps = MUON_STEP_CASES[name]
    g = torch.Generator().manual_seed(seed)
    p0 = torch.randn(*shape, generator=g) * 0.02
    grads = [torch.randn(*shape, generator=g) for _ in range(steps)]
    return p0, grads
