"""The tensor-core engine in isolation (xmc_test_gemm of the C ABI) against torch fp32 matmul."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _rand(shape, dtype, gen, scale=1.0):
    return (torch.randn(*shape, generator=gen) * scale).to(dtype).cuda()


@pytest.mark.parametrize("m,n,k", [(128, 256, 64), (128, 256, 256), (200, 300, 192), (384, 768, 520),
                                   (1000, 48, 768), (64, 16, 72)])
def test_kmajor_bf16(m, n, k):
    from elmo_b200.handle import test_gemm
    g = torch.Generator().manual_seed(m + n + k)
    a = _rand((m, k), torch.bfloat16, g); b = _rand((n, k), torch.bfloat16, g)
    d = test_gemm(a, b, 0)
    ref = a.float() @ b.float().t()
    assert torch.allclose(d, ref, rtol=1e-4, atol=1e-3), float((d - ref).abs().max())


@pytest.mark.parametrize("m,n,k", [(128, 256, 128), (256, 512, 768), (300, 80, 400), (130, 272, 1040)])
def test_kmajor_e4m3(m, n, k):
    from elmo_b200.handle import test_gemm
    g = torch.Generator().manual_seed(m * 3 + n + k)
    a = _rand((m, k), torch.float8_e4m3fn, g); b = _rand((n, k), torch.float8_e4m3fn, g)
    d = test_gemm(a, b, 0)
    ref = a.float() @ b.float().t()
    assert torch.allclose(d, ref, rtol=1e-4, atol=1e-3), float((d - ref).abs().max())


@pytest.mark.parametrize("m,n,k", [(128, 256, 64), (128, 256, 256), (512, 768, 1000), (48, 128, 130),
                                   (200, 320, 4096)])
def test_mnmajor_bf16(m, n, k):
    from elmo_b200.handle import test_gemm
    g = torch.Generator().manual_seed(m + 7 * n + k)
    a = _rand((k, m), torch.bfloat16, g); b = _rand((k, n), torch.bfloat16, g)
    d = test_gemm(a, b, 1)
    ref = a.float().t() @ b.float()
    assert torch.allclose(d, ref, rtol=1e-4, atol=2e-3), float((d - ref).abs().max())
