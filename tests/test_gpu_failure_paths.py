"""GPU: failure paths end in a status code or a Python exception, never in a hung or faulted GPU."""
import time

import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda"


def test_bounded_wait_runs_out_and_reports_status(pkg):
    """A wait on a barrier that nothing completes gives up after its limit (2e6 clocks, about 1 ms);
    the kernel returns normally and the context stays usable."""
    import importlib
    L = importlib.import_module(pkg.__name__ + "._lib")
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    t0 = time.perf_counter()
    L.check(pkg.lib().b200moe_selftest_bounded_wait(status.data_ptr(), 2_000_000, torch.cuda.current_stream().cuda_stream))
    torch.cuda.synchronize()
    assert time.perf_counter() - t0 < 1.0
    assert int(status.item()) == 6
    assert b"expected" in pkg.lib().b200moe_status_string(6)
    # the context is alive: a normal kernel still runs and verifies
    a = torch.randn(256, 128, device=DEV).to(torch.bfloat16)
    d = pkg.ops.gemm_nt(a, a)
    assert torch.isfinite(d).all()
    pkg.check_status()


def test_layer_forward_backward_in_a_cuda_graph(pkg):
    """The single-GPU layer has no host synchronisation, so forward + backward capture into one CUDA
    graph; replays on new inputs reproduce the eager result bit for bit."""
    T, H, E, I, k = 1024, 256, 8, 256, 2
    torch.manual_seed(0)
    layer = pkg.MoELayer(H, I, E, top_k=k).to(DEV).to(torch.bfloat16)
    x_static = torch.randn(T, H, device=DEV).to(torch.bfloat16).requires_grad_(True)
    go = torch.randn(T, H, device=DEV).to(torch.bfloat16)
    s = torch.cuda.Stream()
    s.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(s):                 # warm-up outside the capture (lazy one-time set-up)
        for _ in range(2):
            layer.zero_grad(set_to_none=True)
            x_static.grad = None
            layer(x_static).backward(go)
    torch.cuda.current_stream().wait_stream(s)
    layer.zero_grad(set_to_none=True)
    x_static.grad = None
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        out_static = layer(x_static)
        out_static.backward(go)
    x_new = torch.randn(T, H, device=DEV).to(torch.bfloat16)
    with torch.no_grad():
        x_static.copy_(x_new)
    g.replay()
    torch.cuda.synchronize()
    out_graph, gx_graph = out_static.clone(), x_static.grad.clone()
    gw_graph = layer.down_proj.grad.clone()
    layer.zero_grad(set_to_none=True)
    xe = x_new.clone().requires_grad_(True)
    out_e = layer(xe)
    out_e.backward(go)
    pkg.check_status()
    assert torch.equal(out_graph, out_e) and torch.equal(gx_graph, xe.grad)
    assert torch.equal(gw_graph, layer.down_proj.grad)


def test_expert_index_out_of_range_is_reported_and_skipped(pkg):
    """Routing indices outside [0, E) raise the status word; the slot gets no row (slot_row = slot_pos = -1), every
    consumer of the tables skips it, and the rest of the batch is computed as if the slot were absent."""
    T, H, E, I, k = 512, 128, 8, 64, 2
    g = torch.Generator().manual_seed(0)
    x = torch.randn(T, H, generator=g).to(torch.bfloat16).to(DEV).requires_grad_(True)
    gu = (torch.randn(E, 2 * I, H, generator=g) * 0.05).to(torch.bfloat16).to(DEV).requires_grad_(True)
    dn = (torch.randn(E, H, I, generator=g) * 0.05).to(torch.bfloat16).to(DEV).requires_grad_(True)
    idx = torch.randint(0, E, (T, k), generator=g)
    w = torch.rand(T, k, generator=g)
    bad = idx.clone()
    bad[3, 1] = E            # one past the last expert
    bad[7, 0] = -1
    bad[9, 1] = 1 << 40      # does not even fit an int
    codes = torch.zeros(E, dtype=torch.int32, device=DEV)
    perm = pkg.ops.permute_build(bad.to(DEV), E, want_order=True)
    torch.cuda.synchronize()
    slots = [3 * k + 1, 7 * k, 9 * k + 1]
    assert perm.slot_row.cpu()[slots].tolist() == [-1, -1, -1]
    assert perm.slot_pos.cpu()[slots].tolist() == [-1, -1, -1]
    assert int(perm.counts.sum()) == T * k - 3
    with pytest.raises(RuntimeError):
        pkg.check_status()                                   # ST_BAD_EXPERT_INDEX; reading it clears it
    out = pkg.moe(x, bad.to(DEV), w.to(DEV), gu, dn, codes)
    out.float().sum().backward()
    torch.cuda.synchronize()
    with pytest.raises(RuntimeError):
        pkg.check_status()
    assert torch.isfinite(out).all() and torch.isfinite(x.grad).all() and torch.isfinite(gu.grad).all()
    # the other tokens are untouched by the bad slots: same rows as a run in which those slots carry weight zero
    good = idx.clone()
    w0 = w.clone()
    for t, j in ((3, 1), (7, 0), (9, 1)):
        w0[t, j] = 0.0
    ref = pkg.moe(x.detach(), good.to(DEV), w0.to(DEV), gu.detach(), dn.detach(), codes)
    pkg.check_status()
    assert torch.equal(out.detach(), ref)


def test_cross_rank_barrier_is_bounded(pkg):
    """The expert-parallel barrier on ONE GPU: with every flag word already at the generation it passes at once;
    when a peer's word never arrives (nothing sets it) the wait runs out after its limit (2e6 clocks, about 1 ms),
    the status word receives 7 and the kernel returns normally with the context intact."""
    import importlib
    L = importlib.import_module(pkg.__name__ + "._lib")
    lib = pkg.lib()
    st = torch.cuda.current_stream().cuda_stream
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    mine = torch.zeros(16, dtype=torch.int32, device=DEV)       # this rank's flag array
    peer = torch.zeros(16, dtype=torch.int32, device=DEV)       # stands in for the peer's array (never read here)
    table = L.ptr_table([mine.data_ptr(), peer.data_ptr()])
    # world of one: the rank announces itself and sees it
    L.check(lib.b200moe_ep_barrier(L.ptr_table([mine.data_ptr()]), 1, 0, 1, 2_000_000, status.data_ptr(), st))
    torch.cuda.synchronize()
    assert int(status.item()) == 0 and int(mine[0]) == 1
    # world of two, the peer's arrival (word 1 of this rank's array) is already there: passes, and announces itself
    mine[1] = 5
    L.check(lib.b200moe_ep_barrier(table, 2, 0, 5, 2_000_000, status.data_ptr(), st))
    torch.cuda.synchronize()
    assert int(status.item()) == 0 and int(mine[0]) == 5 and int(peer[0]) == 5
    # the next generation never arrives from the peer
    t0 = time.perf_counter()
    L.check(lib.b200moe_ep_barrier(table, 2, 0, 6, 2_000_000, status.data_ptr(), st))
    torch.cuda.synchronize()
    assert time.perf_counter() - t0 < 1.0
    assert int(status.item()) == 7
    with pytest.raises(RuntimeError, match="peer rank"):
        L.raise_for_status(int(status.item()))
    a = torch.randn(256, 128, device=DEV).to(torch.bfloat16)    # the context is alive
    assert torch.isfinite(pkg.ops.gemm_nt(a, a)).all()
    pkg.check_status()
