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
