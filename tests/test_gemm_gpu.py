"""tcgen05 bf16 GEMM kernels (single CTA per tile, and CTA pair per tile) against an fp32 matmul."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _rel(a, b):
    return ((a.float() - b.float()).norm() / b.float().norm().clamp_min(1e-9)).item()


@pytest.mark.parametrize("M,N,K", [(128, 256, 64), (384, 512, 320), (1000, 264, 192), (2048, 2048, 1024)])
def test_gemm_single_cta(M, N, K):
    from umdk_b200.ops.gemm import gemm_bf16
    g = torch.Generator(device="cuda").manual_seed(M + N)
    a = torch.randn(M, K, device="cuda", generator=g).to(torch.bfloat16)
    b = torch.randn(N, K, device="cuda", generator=g).to(torch.bfloat16)
    c = gemm_bf16(a, b, impl="1sm")
    torch.cuda.synchronize()
    assert _rel(c, a.float() @ b.float().t()) < 5e-3


@pytest.mark.parametrize("M,N,K", [(256, 256, 64), (512, 768, 320), (2048, 1024, 1024), (4096, 4096, 512)])
def test_gemm_cta_pair(M, N, K):
    from umdk_b200.ops.gemm import gemm_bf16
    g = torch.Generator(device="cuda").manual_seed(M + N + 1)
    a = torch.randn(M, K, device="cuda", generator=g).to(torch.bfloat16)
    b = torch.randn(N, K, device="cuda", generator=g).to(torch.bfloat16)
    want = a.float() @ b.float().t()
    for _ in range(2):   # twice: barriers and TMEM are handed back cleanly
        c = gemm_bf16(a, b, impl="2sm")
        torch.cuda.synchronize()
        assert _rel(c, want) < 5e-3
