"""GPU, 2 ranks over NCCL: DistributedMuon (round-robin ownership, one broadcast per source rank) leaves every rank
with the parameters the replicated FusedMuon produces.  Needs two GPUs."""
import os
import socket

import pytest
import torch

pytestmark = pytest.mark.gpu

SHAPES = [(2, 128, 192), (192, 128), (64, 64), (3, 64, 128), (128, 192)]


def _inputs():
    g = torch.Generator().manual_seed(37)
    init = [torch.randn(*s, generator=g) * 0.02 for s in SHAPES]
    grads = [[torch.randn(*s, generator=g) for s in SHAPES] for _ in range(3)]
    return init, grads


def _worker(rank, world, port, mode, q):
    import importlib
    import torch.distributed as dist
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        pkg = importlib.import_module("triton-kernel-fused_b200")
        init, grads = _inputs()
        ps = [torch.nn.Parameter(t.clone().to(dev)) for t in init]
        opt = pkg.DistributedMuon(ps, lr=0.01, weight_decay=0.1, scale_mode=mode)
        for step_grads in grads:
            for p, gr in zip(ps, step_grads):
                p.grad = gr.to(dev)               # equal on both ranks, as after DDP's all-reduce
            opt.step()
        torch.cuda.synchronize()
        pkg.check_status()
        owned = [i for i, o in enumerate(opt._owner) if o == rank]
        has_mom = [i for i, p in enumerate(ps) if "muon_mom" in opt.state[p]]
        q.put((rank, [p.detach().cpu() for p in ps], owned, has_mom))
    except BaseException as exc:
        q.put((rank, "error", repr(exc)[:500]))
        raise
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("mode", ["polar", "aurora", "normuon"])
def test_distributed_muon_equals_replicated_fused_muon(pkg, mode):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    import torch.multiprocessing as mp
    from oracle import muon_oracle as MO
    world = 2
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    s = socket.socket(); s.bind(("127.0.0.1", 0)); port = s.getsockname()[1]; s.close()
    procs = [ctx.Process(target=_worker, args=(r, world, port, mode, q)) for r in range(world)]
    for p in procs:
        p.start()
    res = {}
    try:
        for _ in range(world):
            r = q.get(timeout=300)
            assert not isinstance(r[1], str), f"rank {r[0]} failed: {r[2]}"
            res[r[0]] = r[1:]
    finally:
        for p in procs:
            p.join(timeout=30)
            if p.is_alive():
                p.kill()
    # both ranks hold the same parameters, bit for bit
    for a, b in zip(res[0][0], res[1][0]):
        assert torch.equal(a, b)
    # every parameter has exactly one owner and momentum lives only there
    assert sorted(res[0][1] + res[1][1]) == list(range(len(SHAPES)))
    assert res[0][2] == res[0][1] and res[1][2] == res[1][1]
    # and they are where the replicated optimizer ends
    init, grads = _inputs()
    ps = [torch.nn.Parameter(t.clone().cuda()) for t in init]
    opt = pkg.FusedMuon(ps, lr=0.01, weight_decay=0.1, scale_mode=mode)
    for step_grads in grads:
        for p, gr in zip(ps, step_grads):
            p.grad = gr.cuda()
        opt.step()
    for got, p, t0 in zip(res[0][0], ps, init):
        assert MO.rel_l2(got - t0, p.detach().cpu() - t0) < 1e-3
