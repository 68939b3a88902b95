"""The CTA-pair (tcgen05 cta_group::2, 256 x 256 tile) GEMM against a PyTorch fp32 reference."""
import math

import pytest
import torch
import torch.nn.functional as F

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _rel_err(a, b):
    a, b = a.float(), b.float()
    return ((a - b).norm() / (b.norm() + 1e-12)).item()


@pytest.fixture(autouse=True)
def _status_clean():
    yield
    from necklace_b200.ops import check_status
    check_status()


@pytest.mark.parametrize("a_mn,b_mn", [(False, False), (False, True), (True, False), (True, True)])
@pytest.mark.parametrize("M,N,K", [(256, 256, 64), (512, 768, 256), (8192, 1024, 1024),
                                   (1000, 520, 136), (300, 264, 72), (2048, 4096, 512)])
def test_pair_layouts(a_mn, b_mn, M, N, K):
    from necklace_b200.ops import gemm
    torch.manual_seed(0)
    A = torch.randn(M, K, device=DEV).bfloat16()
    B = torch.randn(N, K, device=DEV).bfloat16()
    out = gemm(A.t().contiguous() if a_mn else A, B.t().contiguous() if b_mn else B,
               a_mn=a_mn, b_mn=b_mn, bn=512)
    ref = A.float() @ B.float().t()
    assert _rel_err(out, ref) < 1e-2
    assert (out.float() - ref).abs().max().item() < 0.05 * math.sqrt(K) + 0.5


def test_pair_epilogues():
    from necklace_b200.ops import gemm, EPI_GELU_FWD, EPI_GELU_BWD
    torch.manual_seed(1)
    M, N, K = 768, 1024, 320
    A = (torch.randn(M, K, device=DEV) * 0.5).bfloat16()
    B = (torch.randn(N, K, device=DEV) * 0.1).bfloat16()
    bias = torch.randn(N, device=DEV).bfloat16()
    res = torch.randn(M, N, device=DEV).bfloat16()
    base = A.float() @ B.float().t()
    out = gemm(A, B, bias=bias, res=res, bn=512)
    assert _rel_err(out, base + bias.float() + res.float()) < 1e-2
    aux = torch.empty(M, N, device=DEV, dtype=torch.bfloat16)
    out = gemm(A, B, bias=bias, epi=EPI_GELU_FWD, aux=aux, bn=512)
    z = base + bias.float()
    assert _rel_err(aux, z) < 1e-2 and _rel_err(out, F.gelu(z, approximate="tanh")) < 1e-2
    zz = aux.float().requires_grad_(True)
    F.gelu(zz, approximate="tanh").backward(torch.ones_like(zz))
    out = gemm(A, B, epi=EPI_GELU_BWD, aux=aux, bn=512)
    assert _rel_err(out, base * zz.grad) < 2e-2
    C = torch.randn(M, N, device=DEV)
    C0 = C.clone()
    gemm(A, B, out=C, accumulate=True, alpha=0.5, bn=512)
    assert _rel_err(C, C0 + 0.5 * base) < 1e-2


@pytest.mark.parametrize("bn", [0, 256, 512])
@pytest.mark.parametrize("M,N,K,acc", [(1024, 1024, 8192, False), (3072, 1024, 4096, True),
                                       (256, 512, 2048, False), (1024, 4096, 8192, False)])
def test_split_k_weight_gradient_shapes(bn, M, N, K, acc):
    """Few output tiles and a long K: the split-K path (slices + reduce kernel)."""
    from necklace_b200.ops import gemm
    torch.manual_seed(2)
    At = (torch.randn(K, M, device=DEV) * 0.1).bfloat16()   # MN-major operands (wgrad layout)
    Bt = (torch.randn(K, N, device=DEV) * 0.1).bfloat16()
    ref = At.float().t() @ Bt.float()
    out = torch.randn(M, N, device=DEV).bfloat16() if acc else None
    base = out.float().clone() if acc else 0
    got = gemm(At, Bt, a_mn=True, b_mn=True, out=out, accumulate=acc, alpha=0.5, bn=bn)
    assert _rel_err(got, base + 0.5 * ref) < 1e-2
    c32 = torch.zeros(M, N, device=DEV)
    gemm(At, Bt, a_mn=True, b_mn=True, out=c32, bn=bn)
    assert _rel_err(c32, ref) < 5e-3
