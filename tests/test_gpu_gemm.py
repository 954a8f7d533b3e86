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
