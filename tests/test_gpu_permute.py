"""GPU: the device-side counting sort against the stable-sort oracle, bit-exact."""
import pytest
import torch

from oracle import moe_oracle as O

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _routing(T, E, k, seed, skew=None, cap=None):
    g = torch.Generator().manual_seed(seed)
    logits = torch.randn(T, E, generator=g)
    if skew is not None:
        logits = logits + torch.log(torch.arange(1, E + 1).float().pow(-skew))[None, :] * 3
    if cap is not None:
        logits[:, cap:] = -1e4
    return torch.topk(logits, k, dim=1).indices


@pytest.mark.parametrize("T,E,k,skew,cap", [(512, 8, 2, None, None), (4099, 64, 6, None, None),
                                            (3000, 128, 8, 1.1, None), (1024, 256, 8, None, None),
                                            (777, 6, 2, None, 4), (1, 4, 1, None, None),
                                            (20000, 64, 6, 2.0, None)])
def test_tables_bit_exact(pkg, T, E, k, skew, cap):
    idx = _routing(T, E, k, 5 + T, skew, cap)
    tb = O.permutation_tables(idx, E)
    perm = pkg.ops.permute_build(idx.to(DEV), E, want_order=True)
    pkg.check_status()
    total = int(tb["poffs"][-1])
    assert torch.equal(perm.counts.cpu(), tb["counts"])
    assert torch.equal(perm.offs.cpu(), tb["offs"])
    assert torch.equal(perm.poffs.cpu(), tb["poffs"])
    assert torch.equal(perm.order.cpu().long(), tb["order"])     # == torch.sort(stable=True)
    inv = torch.empty_like(tb["order"])
    inv[tb["order"]] = torch.arange(tb["order"].numel())
    assert torch.equal(perm.slot_pos.cpu().long(), inv)
    assert torch.equal(perm.slot_row.cpu(), tb["slot_row"])
    assert torch.equal(perm.row_slot.cpu()[:total], tb["row_slot"])
    assert torch.equal(perm.tile_expert.cpu()[: total // 256], tb["tile_expert"])
    assert perm.cap >= total
    if cap is not None:
        assert perm.counts.cpu()[cap:].sum() == 0


def test_gather_rows_and_pad_rows_are_zero(pkg):
    T, E, k, H = 1000, 16, 4, 256
    idx = _routing(T, E, k, 1)
    x = torch.randn(T, H, generator=torch.Generator().manual_seed(2)).to(torch.bfloat16)
    perm = pkg.ops.permute_build(idx.to(DEV), E)
    x_s = pkg.ops.gather_rows(x.to(DEV), perm).cpu()
    tb = O.permutation_tables(idx, E)
    rs = tb["row_slot"]
    live = rs >= 0
    assert torch.equal(x_s[: rs.numel()][live], x[(rs[live] // k).long()])
    assert (x_s[: rs.numel()][~live] == 0).all()


def test_bad_expert_index_raises_status(pkg):
    idx = torch.tensor([[0, 9]], device=DEV)
    pkg.ops.permute_build(idx, 4)
    with pytest.raises(RuntimeError, match="expert index"):
        pkg.check_status()
    pkg.check_status()      # cleared
