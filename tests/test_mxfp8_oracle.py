"""CPU: the MXFP8 quantise oracle follows the stated MX convention (known answers)."""
import torch

from oracle import mxfp8_oracle as Q


def test_known_scales_and_saturation():
    x = torch.zeros(4, 32)
    x[0, 0] = 1.0        # amax 1   -> exponent 0-8  -> byte 119, code for 256
    x[1, 0] = 448.0      # amax 448 -> exponent 8-8  -> byte 127
    x[2, 0] = 500.0      # amax 500 -> exponent 0, 500 saturates to 448
    codes, sb = Q.quantise(x)
    assert sb.flatten().tolist() == [119, 127, 127, 0]
    d = Q.dequantise(codes, sb)
    assert d[0, 0] == 1.0 and d[1, 0] == 448.0 and d[2, 0] == 448.0 and (d[3] == 0).all()


def test_round_to_nearest_even_on_the_e4m3_grid():
    # with scale 2^0 the grid between 16 and 32 has step 2: 17 -> 16 (tie to even), 19 -> 20
    x = torch.zeros(1, 32)
    x[0, :4] = torch.tensor([256.0, 17.0, 19.0, 18.0])
    assert Q.qdq(x)[0, :4].tolist() == [256.0, 16.0, 20.0, 18.0]


def test_relative_error_bound_and_atom_layout():
    g = torch.Generator().manual_seed(0)
    x = torch.randn(256, 256, generator=g)
    d = Q.qdq(x)
    amax = x.view(256, 8, 32).abs().amax(-1, keepdim=True).expand(256, 8, 32).reshape(256, 256)
    assert ((d - x).abs() <= amax * 0.126).all()           # saturation corner: at most 1/8 of amax
    _, sb = Q.quantise(x)
    atoms = Q.sf_atoms(sb)
    assert atoms.numel() == 2 * 2 * 512
    r, kb = 200, 5                                         # row-block 1, k-chunk 1
    off = ((r // 128) * 2 + kb // 4) * 512 + (r % 32) * 16 + ((r % 128) // 32) * 4 + kb % 4
    assert int(atoms[off]) == int(sb[r, kb])


def test_mx_matmul_backward_quantises_along_each_reduction():
    g = torch.Generator().manual_seed(1)
    a = torch.randn(64, 96, generator=g, requires_grad=True)
    b = torch.randn(32, 96, generator=g, requires_grad=True)
    go = torch.randn(64, 32, generator=g)
    Q.mx_matmul_nt(a, b).backward(go)
    assert torch.allclose(a.grad, Q.qdq(go) @ Q.qdq(b.detach().t().contiguous()).t())
    assert torch.allclose(b.grad, Q.qdq(go.t().contiguous()) @ Q.qdq(a.detach().t().contiguous()).t())
