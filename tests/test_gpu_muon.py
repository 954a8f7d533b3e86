"""GPU: the expert-stack optimizer step (`newton_schulz`, `FusedMuon`) against the CPU oracle and against results
of the reference's own code (tests/golden/muon.npz).

The iteration runs in bf16 on the GPU.  Ten quintic steps with the default coefficients amplify rounding noise of
the small singular directions, so a bf16 run is compared (a) with the fp32 result at 3e-2 relative L2, (b) by the
reference's own stability gate for its low-precision iteration (bench.py:1054-1058: no NaN, mean singular value in
[0.8, 1.2]), and (c) exactly where the arithmetic is exact or rounds at the same places: momentum buffers, pad
rows, reruns."""
import os

import numpy as np
import pytest
import torch

from oracle import muon_oracle as MO
from tests.golden.cases import (MUON_LR, MUON_MODE_CASES, MUON_MOMENTUM, MUON_NS_CASES, MUON_STEP_CASES, muon_ns_input,
                                muon_step_inputs)

pytestmark = pytest.mark.gpu
DEV = "cuda"
NS_TOL = 3e-2       # bf16 iteration against the fp32 iteration, relative L2 (measured 6e-3 ... 7e-3)
STEP_TOL = 1e-1     # the same for the update p_new - p_old of a step


@pytest.fixture(scope="module")
def gold(golden_dir):
    return np.load(os.path.join(golden_dir, "muon.npz"))


def _sv_gate(Y):
    Y = Y.float()
    sv = torch.linalg.svdvals(Y if Y.dim() == 3 else Y[None])
    assert not Y.isnan().any()
    assert 0.8 <= sv.mean().item() <= 1.2, sv.mean().item()


@pytest.mark.parametrize("name", list(MUON_NS_CASES))
def test_newton_schulz_against_reference_golden(pkg, gold, name):
    G = muon_ns_input(name)
    got = pkg.newton_schulz(G.to(DEV)).cpu()
    torch.cuda.synchronize(); pkg.check_status()
    assert got.shape == G.shape and got.dtype == G.dtype
    assert MO.rel_l2(got, torch.from_numpy(gold[f"ns_{name}_f32"])) < NS_TOL
    assert MO.rel_l2(got, torch.from_numpy(gold[f"ns_{name}_bf16"])) < NS_TOL
    _sv_gate(got)


# the reference's stability shapes (bench.py:1054) and the layer's own expert stacks (headline: (E,2I,H), (E,H,I))
@pytest.mark.parametrize("shape", [(512, 512), (256, 512), (1536, 512), (9, 1536, 512), (9, 512, 768),
                                   (4, 2816, 2048), (4, 2048, 1408), (2, 1536, 2048)])
def test_newton_schulz_against_oracle(pkg, shape):
    G = torch.randn(*shape, generator=torch.Generator().manual_seed(sum(shape)))
    got = pkg.newton_schulz(G.to(DEV).to(torch.bfloat16)).float()
    torch.cuda.synchronize(); pkg.check_status()
    ref = MO.newton_schulz(G.to(torch.bfloat16).float().to(DEV), ns_dtype=torch.float32)   # oracle code, fp32
    assert MO.rel_l2(got, ref) < NS_TOL
    _sv_gate(got)
    again = pkg.newton_schulz(G.to(DEV).to(torch.bfloat16)).float()
    assert torch.equal(got, again)                      # no atomics anywhere: reruns are bit-identical


def test_zero_matrix_stays_zero_and_finite(pkg):
    G = torch.zeros(2, 64, 128, device=DEV, dtype=torch.bfloat16)
    out = pkg.newton_schulz(G)
    assert torch.equal(out, G)                          # norm clamps at eps (kernels/sm75/muon.py:78): 0 / eps = 0


@pytest.mark.parametrize("name", list(MUON_STEP_CASES))
@pytest.mark.parametrize("pdtype", [torch.float32, torch.bfloat16])
def test_step_against_reference_golden_and_oracle(pkg, gold, name, pdtype):
    _shape, _seed, mode, nesterov, wd, steps = MUON_STEP_CASES[name]
    p0, grads = muon_step_inputs(name)
    p = torch.nn.Parameter(p0.to(DEV).to(pdtype))
    opt = pkg.FusedMuon([p], lr=MUON_LR, momentum=MUON_MOMENTUM, nesterov=nesterov, weight_decay=wd, scale_mode=mode)
    po, mo = p0.to(pdtype).clone(), torch.zeros_like(p0, dtype=torch.bfloat16)
    for i in range(steps):
        p.grad = grads[i].to(DEV).to(pdtype)         # torch wants a gradient of the parameter's dtype
        opt.step()
        MO.muon_step(po, grads[i].to(pdtype), mo, MUON_LR, MUON_MOMENTUM, nesterov, wd, ns_dtype=torch.bfloat16, scale_mode=mode)
    torch.cuda.synchronize(); pkg.check_status()
    # momentum: the same bf16 roundings in the same order (a product that lands on a rounding tie may differ by one
    # unit in the last place between the host's and the GPU's multiply)
    mom = opt.state[p]["muon_mom"].cpu().view_as(mo).float()
    assert (mom != mo.float()).float().mean().item() < 1e-3 and MO.rel_l2(mom, mo.float()) < 1e-3
    start = p0.to(pdtype).float()
    moved = p.detach().float().cpu() - start
    ref_moved = torch.from_numpy(gold[f"step_{name}_p"]) - p0           # the reference, fp32 throughout
    tol = STEP_TOL if pdtype == torch.float32 else 2 * STEP_TOL         # bf16 parameters round every update
    assert MO.rel_l2(moved, ref_moved) < tol
    assert MO.rel_l2(moved, po.float() - start) < tol                   # oracle with a bf16 iteration


def test_layer_sized_stack_step_and_padding(pkg):
    # d_ff = 1408 is not a multiple of the 256-row tile: the iteration runs on 1536 padded rows
    E, H, I = 3, 512, 1408
    g = torch.Generator().manual_seed(5)
    p0 = torch.randn(E, H, I, generator=g) * 0.02
    grad = torch.randn(E, H, I, generator=g)
    p = torch.nn.Parameter(p0.to(DEV).to(torch.bfloat16))
    p.grad = grad.to(DEV).to(torch.bfloat16)
    opt = pkg.FusedMuon([p], lr=0.01, weight_decay=0.0, scale_mode="polar")
    opt.step()
    torch.cuda.synchronize(); pkg.check_status()
    po, mo = p0.to(torch.bfloat16).float(), torch.zeros(E, H, I)
    MO.muon_step(po, grad.to(torch.bfloat16).float(), mo, 0.01, weight_decay=0.0, ns_dtype=torch.float32,
                 scale_mode="polar")
    start = p0.to(torch.bfloat16).float()
    assert MO.rel_l2(p.detach().float().cpu() - start, po - start) < 2 * STEP_TOL


def test_rejected_options(pkg):
    p = torch.nn.Parameter(torch.zeros(2, 64, 64, device=DEV))
    for kw in (dict(scale_mode="no_such_mode"), dict(aurora_k=0), dict(ns_dtype=torch.float16),
               dict(xorth_post=0.1), dict(spectral_wd=0.1)):
        with pytest.raises(ValueError):
            pkg.FusedMuon([p], **kw)
    with pytest.raises(ValueError):
        pkg.newton_schulz(torch.zeros(4, 12, 64, device=DEV))          # 12 is not a multiple of 8


def test_a_shard_of_a_stack_steps_like_the_whole_stack(pkg):
    """Matrices of a stack are orthogonalised independently, so an expert-parallel rank that owns experts [e0, e1)
    steps its shard with no exchange: the shard's result equals the same matrices inside the full stack, bit for bit."""
    E, r, c = 8, 512, 320
    g = torch.Generator().manual_seed(9)
    p0 = (torch.randn(E, r, c, generator=g) * 0.02).to(torch.bfloat16)
    grad = torch.randn(E, r, c, generator=g).to(torch.bfloat16)

    def step(lo, hi):
        p = torch.nn.Parameter(p0[lo:hi].clone().to(DEV))
        p.grad = grad[lo:hi].clone().to(DEV)
        opt = pkg.FusedMuon([p], lr=0.01, weight_decay=0.1)
        opt.step(); opt.step()
        return p.detach().clone(), opt.state[p]["muon_mom"].clone()

    full_p, full_m = step(0, E)
    for lo, hi in ((0, 4), (4, 8), (2, 3)):
        sp, sm = step(lo, hi)
        assert torch.equal(sp, full_p[lo:hi]) and torch.equal(sm, full_m[lo:hi])
    torch.cuda.synchronize(); pkg.check_status()


def test_same_shape_parameters_step_as_one_stack(pkg):
    """2-D and 3-D parameters with the same matrix shape are orthogonalised in one batched stack (the reference's
    batched-state design); every parameter ends up exactly where it would stepping alone, also when the cap on the
    batch splits the stack into chunks."""
    g = torch.Generator().manual_seed(17)
    shapes = [(128, 192), (128, 192), (3, 128, 192), (192, 128), (128, 192)]
    init = [(torch.randn(*s, generator=g) * 0.02) for s in shapes]
    grads = [torch.randn(*s, generator=g) for s in shapes]

    def run(split, cap):
        ps = [torch.nn.Parameter(t.clone().to(DEV)) for t in init]
        opts = ([pkg.FusedMuon([p], lr=0.01, weight_decay=0.1) for p in ps] if split
                else [pkg.FusedMuon(ps, lr=0.01, weight_decay=0.1, ns_batch_elems=cap)])
        for _ in range(2):
            for p, gr in zip(ps, grads):
                p.grad = gr.to(DEV)
            for o in opts:
                o.step()
        torch.cuda.synchronize(); pkg.check_status()
        return [p.detach().clone() for p in ps]

    alone = run(True, None)
    for cap in (64 * 1024 * 1024, 2 * 128 * 192, 1):        # one stack of 6; chunks of at most 2 matrices; one by one
        for a, b in zip(alone, run(False, cap)):
            assert torch.equal(a, b)


def test_state_dict_round_trip_with_fp32_master_weights(pkg):
    """`load_state_dict` casts the bf16 momentum buffer to the parameter's dtype (fp32 masters).  The resumed
    optimizer must bring it back to bf16 instead of letting the kernel reinterpret fp32 memory: a run interrupted
    by state_dict / load_state_dict ends bit-identically to an uninterrupted one."""
    g = torch.Generator().manual_seed(23)
    p0 = torch.randn(3, 128, 192, generator=g) * 0.02
    grads = [torch.randn(3, 128, 192, generator=g) for _ in range(3)]

    def make():
        p = torch.nn.Parameter(p0.clone().to(DEV))           # fp32 master weights
        return p, pkg.FusedMuon([p], lr=0.01, weight_decay=0.1)

    p_a, opt_a = make()
    for gr in grads:
        p_a.grad = gr.to(DEV)
        opt_a.step()
    p_b, opt_b = make()
    for gr in grads[:2]:
        p_b.grad = gr.to(DEV)
        opt_b.step()
    saved = opt_b.state_dict()
    p_c = torch.nn.Parameter(p_b.detach().clone())
    opt_c = pkg.FusedMuon([p_c], lr=0.01, weight_decay=0.1)
    opt_c.load_state_dict(saved)
    assert opt_c.state[p_c]["muon_mom"].dtype == torch.float32      # what torch's loader did to it
    p_c.grad = grads[2].to(DEV)
    opt_c.step()
    torch.cuda.synchronize(); pkg.check_status()
    assert opt_c.state[p_c]["muon_mom"].dtype == torch.bfloat16
    assert torch.equal(p_c.detach(), p_a.detach())
    assert torch.equal(opt_c.state[p_c]["muon_mom"], opt_a.state[p_a]["muon_mom"])
    # a buffer of the wrong size is refused, not read out of bounds
    opt_c.state[p_c]["muon_mom"] = torch.zeros(2, 128, 192, dtype=torch.bfloat16, device=DEV)
    p_c.grad = grads[0].to(DEV)
    with pytest.raises(ValueError):
        opt_c.step()


@pytest.mark.parametrize("name", list(MUON_MODE_CASES))
@pytest.mark.parametrize("pdtype", [torch.float32, torch.bfloat16])
def test_per_row_modes_and_two_pass_aurora_against_reference_golden(pkg, gold, name, pdtype):
    """normuon, aurora_ema, aurora_ema_v2 and aurora with two passes: three steps against the reference's own
    FusedMuon (fp32 iteration) and against the oracle with a bf16 iteration; the per-row EMA state against both."""
    shape, _seed, mode, nesterov, wd, steps, k = MUON_MODE_CASES[name]
    p0, grads = muon_step_inputs(name)
    p = torch.nn.Parameter(p0.to(DEV).to(pdtype))
    opt = pkg.FusedMuon([p], lr=MUON_LR, momentum=MUON_MOMENTUM, nesterov=nesterov, weight_decay=wd, scale_mode=mode,
                        aurora_k=k)
    po, mo, vo = p0.to(pdtype).clone(), torch.zeros_like(p0, dtype=torch.bfloat16), torch.zeros(shape[0], shape[1])
    for i in range(steps):
        p.grad = grads[i].to(DEV).to(pdtype)
        opt.step()
        MO.muon_step(po, grads[i].to(pdtype), mo, MUON_LR, MUON_MOMENTUM, nesterov, wd, ns_dtype=torch.bfloat16,
                     scale_mode=mode, aurora_k=k or 1, scale_v=vo)
    torch.cuda.synchronize(); pkg.check_status()
    start = p0.to(pdtype).float()
    moved = p.detach().float().cpu() - start
    ref_moved = torch.from_numpy(gold[f"step_{name}_p"]) - p0
    tol = STEP_TOL if pdtype == torch.float32 else 2 * STEP_TOL
    assert MO.rel_l2(moved, ref_moved) < tol
    assert MO.rel_l2(moved, po.float() - start) < tol
    if f"step_{name}_v" in gold.files:
        v = opt.state[p]["scale_v"].cpu()
        assert v.dtype == torch.float32 and v.shape == (shape[0], shape[1])
        assert MO.rel_l2(v, torch.from_numpy(gold[f"step_{name}_v"])) < 5e-2
        assert MO.rel_l2(v, vo) < 5e-2


@pytest.mark.parametrize("mode", ["polar", "aurora", "normuon", "aurora_ema"])
def test_graph_mode_replays_the_eager_step_bit_for_bit(pkg, mode):
    """use_graph: gradients are staged eagerly, the rest of the step is captured after the warm-up steps and replayed;
    parameters and state end exactly where the eager optimizer puts them, also when the gradient tensors are new
    objects every step."""
    g = torch.Generator().manual_seed(29)
    shapes = [(3, 128, 192), (192, 128), (3, 128, 192)]
    init = [torch.randn(*s, generator=g) * 0.02 for s in shapes]
    grads = [[torch.randn(*s, generator=g) for s in shapes] for _ in range(6)]

    def run(use_graph):
        ps = [torch.nn.Parameter(t.clone().to(DEV)) for t in init]
        opt = pkg.FusedMuon(ps, lr=0.01, weight_decay=0.1, scale_mode=mode, use_graph=use_graph, graph_warmup=2)
        for step_grads in grads:
            for p, gr in zip(ps, step_grads):
                p.grad = gr.to(DEV)                 # a new tensor every step, as after zero_grad(set_to_none=True)
            opt.step()
        torch.cuda.synchronize(); pkg.check_status()
        return opt, [p.detach().clone() for p in ps], [opt.state[p]["muon_mom"].clone() for p in ps]

    opt_g, pg, mg = run(True)
    _, pe, me = run(False)
    assert opt_g._graph is not None and not opt_g._graph_failed          # it did capture
    for a, b in zip(pg + mg, pe + me):
        assert torch.equal(a, b)


def test_distributed_muon_on_one_rank_equals_fused_muon(pkg):
    """With a process group of one rank DistributedMuon owns every parameter: momentum, update and apply go through
    its own code path (update materialised, broadcast, row-update kernel) and must land where FusedMuon lands."""
    import torch.distributed as dist
    import socket
    if not dist.is_initialized():
        s = socket.socket(); s.bind(("127.0.0.1", 0)); port = s.getsockname()[1]; s.close()
        dist.init_process_group("nccl", init_method=f"tcp://127.0.0.1:{port}", rank=0, world_size=1,
                                device_id=torch.device("cuda", 0))
    try:
        g = torch.Generator().manual_seed(31)
        shapes = [(2, 128, 192), (192, 128), (64, 64)]
        init = [torch.randn(*s, generator=g) * 0.02 for s in shapes]
        grads = [[torch.randn(*s, generator=g) for s in shapes] for _ in range(3)]
        for mode in ("polar", "aurora", "normuon"):
            outs = []
            for cls in (pkg.FusedMuon, pkg.DistributedMuon):
                ps = [torch.nn.Parameter(t.clone().to(DEV)) for t in init]
                opt = cls(ps, lr=0.01, weight_decay=0.1, scale_mode=mode)
                for step_grads in grads:
                    for p, gr in zip(ps, step_grads):
                        p.grad = gr.to(DEV)
                    opt.step()
                torch.cuda.synchronize(); pkg.check_status()
                outs.append([p.detach().clone() for p in ps])
            for a, b, t0 in zip(outs[0], outs[1], init):
                # same kernels, same roundings; the decay-and-add is one fused expression in both paths
                assert MO.rel_l2((b.cpu() - t0), (a.cpu() - t0)) < 1e-3, mode
        with pytest.raises(NotImplementedError):
            pkg.DistributedMuon([torch.nn.Parameter(init[0].to(DEV))], scale_mode="aurora_ema")
    finally:
        dist.destroy_process_group()
