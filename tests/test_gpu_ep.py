"""GPU, 2 ranks over NCCL: the expert-parallel layer equals the single-GPU layer on the
concatenated batch (bit-exact routing, values within the bf16 gate).  Needs two GPUs."""
import os
import socket

import pytest
import torch

pytestmark = pytest.mark.gpu


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, cfg, transport, q):
    import importlib
    import torch.distributed as dist
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        pkg = importlib.import_module("triton-kernel-fused_b200")
        from oracle import moe_oracle as O
        T, H, E, I, k = cfg
        inp = O.make_inputs(T, H, E, I, k, seed=41, bias_std=0.01, dtype=torch.bfloat16)
        Tl, El = T // world, E // world
        sl = slice(rank * Tl, (rank + 1) * Tl)
        # "p2p" = push exchange, "p2p-pull" = pull exchange, "p2p-pull+24" = pull with the last backward pull
        # overlapped on 24 SMs
        # "p2p/3" = push exchange with the local experts pipelined in 3 groups; "p2p@1.5" = buffers of a fixed
        # capacity (1.5 x a rank's own routed rows), no host wait in the forward
        transport, _, cap = transport.partition("@")
        transport, _, groups = transport.partition("/")
        transport, _, sms = transport.partition("+")
        transport, _, exch = transport.partition("-")
        layer = pkg.ExpertParallelMoELayer(H, I, E, top_k=k, transport=transport, reserved_sms=int(sms or 0),
                                           exchange=exch or "push", expert_groups=int(groups or 1),
                                           capacity_factor=float(cap) if cap else None).to(dev).to(torch.bfloat16)
        with torch.no_grad():
            layer.gate.weight.copy_(inp["gate_weight"])
            layer.gate_up_proj.copy_(inp["gate_up"][rank * El:(rank + 1) * El])
            layer.down_proj.copy_(inp["down"][rank * El:(rank + 1) * El])
            layer.bias.copy_(inp["bias"])
        x = inp["x"][sl].to(dev).requires_grad_(True)
        out = layer(x)
        (out.float() * inp["grad_out"][sl].to(dev).float()).sum().backward()
        torch.cuda.synchronize()
        pkg.check_status()
        gw = layer.gate.weight.grad.clone()
        dist.all_reduce(gw)                      # replicated router weight: sum of the local grads
        layer.update_bias(0.001)
        q.put((rank, out.detach().cpu(), x.grad.cpu(), layer.gate_up_proj.grad.cpu(), layer.down_proj.grad.cpu(),
               gw.cpu(), layer.bias.cpu()))
    except BaseException as exc:                 # reported at once: the parent must not sit out its queue timeout
        q.put((rank, "error", repr(exc)[:500]))
        raise
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("transport", ["nccl", "p2p", "p2p-pull", "p2p-pull+24", "p2p/2", "p2p+24/3", "p2p@1.5"])
@pytest.mark.parametrize("cfg", [(2048, 512, 16, 256, 4), (1024, 256, 64, 128, 8)])
def test_expert_parallel_equals_single_gpu(pkg, cfg, transport):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    import torch.multiprocessing as mp
    from oracle import moe_oracle as O
    world = 2
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, cfg, transport, q)) for r in range(world)]
    for p in procs:
        p.start()
    res = {}
    try:
        for _ in range(world):
            r = q.get(timeout=300)
            assert r[1] != "error" if isinstance(r[1], str) else True, f"rank {r[0]} failed: {r[2]}"
            res[r[0]] = r[1:]
    except BaseException:
        for p in procs:                          # a rank that failed leaves its peer waiting: end both
            p.join(timeout=5)
            if p.is_alive():
                p.kill()
        raise
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    T, H, E, I, k = cfg
    inp = O.make_inputs(T, H, E, I, k, seed=41, bias_std=0.01, dtype=torch.bfloat16)
    dev = "cuda"
    layer = pkg.MoELayer(H, I, E, top_k=k).to(dev).to(torch.bfloat16)
    with torch.no_grad():
        layer.gate.weight.copy_(inp["gate_weight"])
        layer.gate_up_proj.copy_(inp["gate_up"])
        layer.down_proj.copy_(inp["down"])
        layer.bias.copy_(inp["bias"])
    x = inp["x"].to(dev).requires_grad_(True)
    out = layer(x)
    (out.float() * inp["grad_out"].to(dev).float()).sum().backward()
    layer.update_bias(0.001)
    cat = lambda i: torch.cat([res[r][i] for r in range(world)])
    tol = 1e-2      # same bf16 kernels on both sides; only tile composition / summation order differ
    assert O.rel_l2(cat(0), out.detach().cpu()) < tol
    assert O.rel_l2(cat(1), x.grad.cpu()) < tol
    assert O.rel_l2(cat(2), layer.gate_up_proj.grad.cpu()) < tol
    assert O.rel_l2(cat(3), layer.down_proj.grad.cpu()) < tol
    assert O.rel_l2(res[0][4], layer.gate.weight.grad.cpu()) < 2e-2
    assert torch.equal(res[0][5], layer.bias.cpu()) and torch.equal(res[1][5], layer.bias.cpu())


def _overflow_worker(rank, world, port, q):
    import importlib
    import torch.distributed as dist
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        pkg = importlib.import_module("triton-kernel-fused_b200")
        T, H, E, I, k = 512, 256, 8, 128, 2
        torch.manual_seed(3)
        layer = pkg.ExpertParallelMoELayer(H, I, E, top_k=k, transport="p2p", capacity_factor=0.25).to(dev).to(torch.bfloat16)
        x = torch.randn(T, H, device=dev, dtype=torch.bfloat16, requires_grad=True)
        out = layer(x)
        out.float().sum().backward()
        torch.cuda.synchronize()
        try:
            pkg.check_status()
            q.put((rank, "no error raised"))
        except RuntimeError as exc:
            q.put((rank, "raised" if "fixed-capacity" in str(exc) else f"other: {exc}"))
        # the status word was cleared by the read: the context and the layer's workspace stay usable
        torch.cuda.synchronize()
        pkg.check_status()
    except BaseException as exc:
        q.put((rank, "error: " + repr(exc)[:300]))
        raise
    finally:
        dist.destroy_process_group()


def test_fixed_capacity_overflow_is_reported_not_truncated(pkg):
    """Buffers sized for a quarter of the rows that will arrive: every rank's plan kernel refuses the step (status 8),
    nothing is computed or written out of bounds, and the error reaches the caller as a RuntimeError."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    import torch.multiprocessing as mp
    world = 2
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_overflow_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    got = {}
    try:
        for _ in range(world):
            r = q.get(timeout=300)
            got[r[0]] = r[1]
    finally:
        for p in procs:
            p.join(timeout=60)
            if p.is_alive():
                p.kill()
    assert got == {0: "raised", 1: "raised"}, got
