"""GPU: the tcgen05 GEMM in its dense modes (every operand-major combination, tails, split-K)."""
import pytest
import torch

from oracle import moe_oracle as O

pytestmark = pytest.mark.gpu
DEV = "cuda"
TOL = 4e-3       # bf16 output rounding (2^-9 per element) on fp32-accumulated sums


def _rand(*shape, seed):
    return torch.randn(*shape, generator=torch.Generator().manual_seed(seed)).to(torch.bfloat16)


@pytest.mark.parametrize("M,N,K", [(128, 256, 64), (256, 256, 128), (300, 64, 256), (1000, 128, 2048),
                                   (512, 1408, 512), (129, 2048, 1408), (4096, 72, 200)])
def test_gemm_nt(pkg, M, N, K):
    a, b = _rand(M, K, seed=1), _rand(N, K, seed=2)
    d = pkg.ops.gemm_nt(a.to(DEV), b.to(DEV))
    pkg.check_status()
    ref = a.float() @ b.float().t()
    assert O.rel_l2(d.float().cpu(), ref) < TOL


@pytest.mark.parametrize("M,N,K", [(128, 256, 64), (300, 128, 256), (1000, 2048, 64), (512, 1408, 512),
                                   (256, 64, 128)])
def test_gemm_nn(pkg, M, N, K):
    a, b = _rand(M, K, seed=3), _rand(K, N, seed=4)
    d = pkg.ops.gemm_nn(a.to(DEV), b.to(DEV))
    pkg.check_status()
    ref = a.float() @ b.float()
    assert O.rel_l2(d.float().cpu(), ref) < TOL


@pytest.mark.parametrize("M,N,K", [(128, 256, 128), (64, 2048, 4096), (256, 512, 1000), (1408, 2048, 300)])
def test_gemm_tn_splitk(pkg, M, N, K):
    a, b = _rand(K, M, seed=5), _rand(K, N, seed=6)
    d = pkg.ops.gemm_tn(a.to(DEV), b.to(DEV))
    pkg.check_status()
    ref = a.float().t() @ b.float()
    assert O.rel_l2(d.float().cpu(), ref) < TOL


@pytest.mark.parametrize("T,E,k,N,K,w_kn", [(1500, 8, 2, 2048, 1408, False), (900, 6, 3, 320, 256, False),
                                            (1200, 4, 2, 512, 704, True), (700, 16, 4, 64, 128, True)])
def test_expert_linear_push_equals_store_then_scatter(pkg, T, E, k, N, K, w_kn):
    """The pushing epilogue (one bulk copy per 128-byte row piece to base[rank] + slot * N) against the storing
    GEMM followed by a scatter; the receive buffer is local here (one rank), some rows are dropped (rank -1)."""
    ops = pkg.ops
    g = torch.Generator().manual_seed(11)
    idx = torch.stack([torch.randperm(E, generator=g)[:k] for _ in range(T)])
    perm = ops.permute_build(idx.to(DEV), E)
    a = _rand(T, K, seed=12).to(DEV)
    a_s = ops.gather_rows(a, perm)
    w = (_rand(E, K, N, seed=13) if w_kn else _rand(E, N, K, seed=13)).to(DEV) * 0.05
    w = w.contiguous()
    ref_rows = (ops.expert_linear_t if w_kn else ops.expert_linear)(a_s, w, perm)
    # every live row gets a distinct slot; every seventh one is dropped
    row_slot_src = perm.row_slot.clone()
    total = int(perm.poffs[-1])                 # rows past the padded total are not part of the permutation
    live = (row_slot_src >= 0) & (torch.arange(row_slot_src.numel(), device=DEV) < total)
    slots = torch.full_like(row_slot_src, 0)
    slots[live] = torch.randperm(int(live.sum()), generator=g).to(torch.int32).to(DEV)
    rank = torch.where(live, torch.zeros_like(slots), torch.full_like(slots, -1))
    drop = (torch.arange(rank.numel(), device=DEV) % 7 == 3) & live
    rank[drop] = -1
    recv = torch.full((int(live.sum()), N), 7.0, dtype=torch.bfloat16, device=DEV)
    base = torch.tensor([recv.data_ptr()], dtype=torch.int64, device=DEV)
    ops.expert_linear_push(a_s, w, perm, rank, slots, base, w_kn=w_kn)
    torch.cuda.synchronize()
    pkg.check_status()
    expect = torch.full_like(recv, 7.0)
    keep = live & ~drop
    expect[slots[keep].long()] = ref_rows[keep]
    assert torch.equal(recv, expect)


@pytest.mark.parametrize("E,R,K", [(3, 256, 96), (2, 512, 512), (5, 1536, 264)])
def test_expert_linear_axpby_epilogue(pkg, E, R, K):
    """alpha * (a @ W[e]^T) + beta * c + diag * I on uniform row segments against the plain grouped GEMM followed
    by the same arithmetic in fp32 (the fused epilogue rounds once, so it is compared with the fp32 result)."""
    seg = pkg.muon._uniform_segments(E, R, DEV)
    a = _rand(E * R, K, seed=21).to(DEV) * 0.1
    w = _rand(E, R, K, seed=22).to(DEV) * 0.1
    c = _rand(E * R, R, seed=23).to(DEV)
    alpha, beta, diag = 2.0315, -4.775, 3.4445
    out = torch.full((E * R, R), 9.0, dtype=torch.bfloat16, device=DEV)
    pkg.ops.expert_linear_axpby(a, w, c, alpha, beta, diag, seg, out)
    torch.cuda.synchronize()
    pkg.check_status()
    prod = torch.bmm(a.float().view(E, R, K), w.float().transpose(1, 2))
    ref = alpha * prod + beta * c.float().view(E, R, R) + diag * torch.eye(R, device=DEV)
    assert O.rel_l2(out.float().view(E, R, R).cpu(), ref.cpu()) < TOL
    plain = pkg.ops.expert_linear(a, w, seg).float().view(E, R, R)      # and the unfused product is what it scales
    assert O.rel_l2(plain.cpu(), prod.cpu()) < TOL


@pytest.mark.parametrize("E,R,K", [(3, 256, 96), (2, 768, 512), (4, 1536, 264), (1, 2048, 128)])
def test_symmetric_products_equal_the_full_ones_bit_for_bit(pkg, E, R, K):
    """x x^T and alpha * (A A^T) + beta * A + diag * I computed over the upper tiles and mirrored against the same
    products computed in full: element (i,j) and (j,i) sum the same products in the same order, so the bits agree."""
    ops = pkg.ops
    seg = pkg.muon._uniform_segments(E, R, DEV)
    x = _rand(E * R, K, seed=31).to(DEV) * 0.1
    full = ops.expert_linear(x, x.view(E, R, K), seg)
    sym = torch.full((E * R, R), 9.0, dtype=torch.bfloat16, device=DEV)
    ops.mirror_upper(ops.expert_gram(x, seg, sym, mirror=False), E, R)      # upper tiles, then the mirroring copy
    sym2 = torch.full((E * R, R), 9.0, dtype=torch.bfloat16, device=DEV)
    ops.expert_gram(x, seg, sym2)                                            # transposed chunks from the epilogue
    torch.cuda.synchronize(); pkg.check_status()
    assert torch.equal(sym, full) and torch.equal(sym2, full)
    assert torch.equal(full.view(E, R, R), full.view(E, R, R).transpose(1, 2))
    A = full
    out_full = torch.empty_like(A)
    ops.expert_linear_axpby(A, A.view(E, R, R), A, 2.0315, -4.775, 3.4445, seg, out_full)
    out_sym = torch.full_like(A, 9.0)
    ops.mirror_upper(ops.expert_linear_axpby(A, A.view(E, R, R), A, 2.0315, -4.775, 3.4445, seg, out_sym,
                                             symmetric=1), E, R)
    out_sym2 = torch.full_like(A, 9.0)
    ops.expert_linear_axpby(A, A.view(E, R, R), A, 2.0315, -4.775, 3.4445, seg, out_sym2, symmetric=2)
    torch.cuda.synchronize(); pkg.check_status()
    assert torch.equal(out_sym, out_full) and torch.equal(out_sym2, out_full)
