"""GPU: b200moe_permute_build_static — the permutation entry point that allocates nothing.

Some users of the library cannot call cudaMalloc where they route tokens (a plugin inside a framework
that owns all free device memory, a latency-bound serving loop), so this entry point keeps its
histogram scratch in a fixed 1 MiB array inside the library.  The test calls it through the C ABI
twice in a row on different routings (the array keeps the previous call's contents) and checks every
output table bit for bit against b200moe_permute_build, which takes a caller-allocated workspace.
The file name sorts last so that pytest collects it after every other test: a run that stops at the
first failure (-x) has then already exercised the whole main path before this side entry point can end
it.  Nothing here depends on the other tests; it passes on its own in a fresh process as well.
"""
import importlib

import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _tables(E, M, cap):
    i32 = dict(dtype=torch.int32, device=DEV)
    names = ("counts", "offs", "poffs", "slot_row", "row_slot", "tile_expert", "order", "slot_pos")
    sizes = (E, E + 1, E + 1, M, cap, cap // 256, M, M)
    return {n: torch.full((s,), -7, **i32) for n, s in zip(names, sizes)}


def _call(fn, idx, E, tabs, status, extra=()):
    T, k = idx.shape
    ptrs = [tabs[n].data_ptr() for n in ("counts", "offs", "poffs", "slot_row", "row_slot", "tile_expert",
                                         "order", "slot_pos")]
    return fn(idx.data_ptr(), T, k, E, *ptrs, *extra, status.data_ptr(), torch.cuda.current_stream().cuda_stream)


@pytest.mark.parametrize("shapes", [[(4099, 64, 6), (3000, 128, 8)], [(512, 8, 2), (20000, 64, 6)]])
def test_static_scratch_matches_workspace_version_twice_in_a_row(pkg, shapes):
    L = importlib.import_module(pkg.__name__ + "._lib")
    lib = pkg.lib()
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    for call_no, (T, E, k) in enumerate(shapes):          # two calls in a row, different sizes
        g = torch.Generator().manual_seed(100 + call_no)
        idx = torch.topk(torch.randn(T, E, generator=g), k, dim=1).indices.to(DEV)
        M = T * k
        cap = L.padded_rows_cap(M, E)
        ref, got = _tables(E, M, cap), _tables(E, M, cap)
        ws_bytes = int(lib.b200moe_permute_ws_bytes(M, E))
        ws = torch.empty(ws_bytes, dtype=torch.uint8, device=DEV)
        L.check(_call(lib.b200moe_permute_build, idx, E, ref, status, extra=(ws.data_ptr(), ws_bytes)))
        L.check(_call(lib.b200moe_permute_build_static, idx, E, got, status))
        torch.cuda.synchronize()
        assert int(status.item()) == 0
        total = int(ref["poffs"][-1])
        for name in ref:                                   # integer tables: bit-exact
            n = total if name == "row_slot" else (total // 256 if name == "tile_expert" else ref[name].numel())
            assert torch.equal(got[name][:n], ref[name][:n]), (call_no, name)


def test_static_scratch_rejects_oversized_problem(pkg):
    L = importlib.import_module(pkg.__name__ + "._lib")
    lib = pkg.lib()
    T, k, E = 1 << 20, 8, 256                               # needs 16 MiB of histogram scratch
    rc = lib.b200moe_permute_build_static(1, T, k, E, 1, 1, 1, 1, 1, 1, None, None, 1, None)
    assert rc == -4
    with pytest.raises(ValueError, match="built-in array holds 1048576"):
        L.check(rc)
