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
    # stacks of the parameter-free codes 0 / 1 / 5 only: the CUDA path applies these inside the GEMM epilogues
    "fused_codes_015": ([0, 1, 5, 1, 5, 0], False, None, 96),
    "fused_codes_015_wide": ([5, 1, 0, 1, 5, 0], False, None, 1536),
    "fused_codes_015_empty": ([1, 5, 0, 5, 1, 0], False, 4, 256),
    "mixed_wide": ([0, 1, 2, 5, 0, 5], True, None, 1536),
    "normrelu2_wide": ([1, 2, 6, 6, 0, 6], True, None, 1536),        # parity_situ.py:96
    "normsitu_wide": ([2, 5, 7, 7, 0, 7], True, None, 1536),         # parity_situ.py:97
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
# the per-row scale modes and aurora with two passes: name -> (shape, seed, scale_mode, nesterov, weight_decay, steps, aurora_k)
MUON_MODE_CASES = {
    "normuon_tall": ((3, 96, 64), 31, "normuon", True, 0.1, 3, None),
    "normuon_wide": ((3, 64, 96), 32, "normuon", True, 0.0, 3, None),
    "aurora_ema_tall": ((3, 96, 64), 33, "aurora_ema", True, 0.1, 3, None),
    "aurora_ema_wide": ((3, 64, 96), 34, "aurora_ema", False, 0.0, 3, None),
    "aurora_ema_v2_tall": ((3, 96, 64), 35, "aurora_ema_v2", True, 0.1, 3, None),
    "aurora_k2_tall": ((3, 96, 64), 36, "aurora", True, 0.0, 3, 2),
    "aurora_k2_wide": ((3, 64, 96), 37, "aurora", True, 0.1, 3, 2),
}
MUON_LR, MUON_MOMENTUM = 0.02, 0.95


def muon_ns_input(name):
    import torch
    shape, seed = MUON_NS_CASES[name]
    return torch.randn(*shape, generator=torch.Generator().manual_seed(seed))


def muon_step_inputs(name):
    """(initial parameters, list of per-step gradients), fp32, seeded."""
    import torch
    shape, seed, _mode, _nest, _wd, steps = (MUON_STEP_CASES.get(name) or MUON_MODE_CASES[name])[:6]
    g = torch.Generator().manual_seed(seed)
    p0 = torch.randn(*shape, generator=g) * 0.02
    grads = [torch.randn(*shape, generator=g) for _ in range(steps)]
    return p0, grads


# ---- router cases pinned on the reference's own Triton kernels run under the Triton interpreter on CPU tensors.
# Epilogue cases: name -> (N, E, k, norm_topk, scale, use_bias, kind, seed)
#   kind "f32"  : tie-free fp32 logits ~ N(0,1)
#   kind "grid" : fp32 logits on a coarse grid (multiples of 1/4 in [-1, 1]): every row is full of exact ties
#   kind "bf16" : bf16 tensor of grid logits (ties survive the dtype)
ROUTER_EPI_CASES = {
    "f32_e8_k2": (300, 8, 2, True, 1.0, True, "f32", 31),
    "f32_e64_k6": (300, 64, 6, True, 1.0, False, "f32", 32),
    "f32_e64_k6_bias_scale": (300, 64, 6, True, 2.5, True, "f32", 33),
    "f32_e128_k8_nonorm": (260, 128, 8, False, 1.0, True, "f32", 34),
    "f32_e256_k8": (200, 256, 8, True, 0.5, True, "f32", 35),
    "f32_e11_k1": (140, 11, 1, True, 1.0, True, "f32", 36),
    "grid_e8_k2": (300, 8, 2, True, 1.0, False, "grid", 37),
    "grid_e64_k6_bias": (300, 64, 6, True, 1.0, True, "grid", 38),
    "grid_e256_k8": (150, 256, 8, True, 1.0, False, "grid", 39),
    "bf16_e64_k6": (300, 64, 6, True, 1.0, False, "bf16", 40),
    "bf16_e128_k8_bias": (200, 128, 8, True, 1.5, True, "bf16", 41),
}
# Whole linear / conv router cases: name -> (B, S, H, E, k, K (0 = linear router), norm, scale, use_bias, seed)
ROUTER_FULL_CASES = {
    "mlp_e8_k2": (2, 96, 64, 8, 2, 0, True, 1.0, True, 51),
    "mlp_e64_k6": (1, 200, 96, 64, 6, 0, True, 2.0, False, 52),
    "mlp_e16_k4_nonorm": (3, 50, 64, 16, 4, 0, False, 1.0, True, 53),
    "conv_e11_k2_K4": (2, 80, 64, 11, 2, 4, True, 1.0, True, 54),
    "conv_e16_k4_K3": (3, 40, 32, 16, 4, 3, True, 1.5, False, 55),
}


def router_epi_inputs(name):
    """(logits, bias or None, upstream gradient of the weights) of an epilogue case, seeded."""
    import torch
    N, E, k, _norm, _scale, use_bias, kind, seed = ROUTER_EPI_CASES[name]
    g = torch.Generator().manual_seed(seed)
    if kind == "f32":
        logits = torch.randn(N, E, generator=g)
    else:
        logits = torch.randint(-4, 5, (N, E), generator=g).float() * 0.25
        if kind == "bf16":
            logits = logits.to(torch.bfloat16)
    # a bias on the same coarse grid keeps sel = score + bias full of ties in the grid cases
    bias = None
    if use_bias:
        bias = (torch.randint(-2, 3, (E,), generator=g).float() * 0.125) if kind != "f32" else torch.randn(E, generator=g) * 0.01
    grad_w = torch.randn(N, k, generator=g)
    return logits, bias, grad_w


def router_full_inputs(name):
    """(x (B,S,H), weight (E,H) or (E,H,K), bias or None, upstream gradient of the weights (B*S,k)), fp32, seeded."""
    import torch
    B, S, H, E, k, K, _norm, _scale, use_bias, seed = ROUTER_FULL_CASES[name]
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(B, S, H, generator=g)
    w = torch.randn(*((E, H, K) if K else (E, H)), generator=g) * (0.1 if K else 0.2)
    bias = torch.randn(E, generator=g) * 0.01 if use_bias else None
    grad_w = torch.randn(B * S, k, generator=g)
    return x, w, bias, grad_w
