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


def test_a_wait_that_runs_out_is_reported_and_the_context_survives():
    """Failure handling without a fault: the self-test leaves out one operand load and shortens the wait
    limit to about a millisecond.  The wait for the missing load gives up, the CTA unwinds (tensor memory
    freed), the call reports XMC_ERR_DEVICE_FLAG with the wait's site, and the next call works."""
    from elmo_b200._lib import XmcError
    from elmo_b200.handle import test_gemm
    g = torch.Generator().manual_seed(5)
    a = _rand((256, 512), torch.bfloat16, g); b = _rand((256, 512), torch.bfloat16, g)
    # whichever wait of the chain behind the missing load started first reports: the MMA issuer's wait for
    # the operand stage (sites 300-303) or the epilogue's wait for the accumulator (400, 401)
    with pytest.raises(XmcError, match=r"device status 1 .*site (30[0-3]|40[01])") as exc:
        test_gemm(a, b, 8)
    assert exc.value.code == 4                                   # XMC_ERR_DEVICE_FLAG
    d = test_gemm(a, b, 0)                                       # the context is intact
    assert torch.allclose(d, a.float() @ b.float().t(), rtol=1e-4, atol=1e-3)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float8_e4m3fn])
@pytest.mark.parametrize("m,n,k", [(256, 256, 128), (512, 768, 1024), (300, 80, 400), (1000, 528, 768),
                                   (64, 16, 128), (128 * 75, 256, 512), (40000, 768, 512)])
def test_kmajor_cta_pairs(m, n, k, dtype):
    """The same contraction on CTA pairs (cluster of two, cta_group::2): 256-row tiles, each CTA of a pair
    stages its own 128 rows of A and half of the B rows.  Covers an odd number of 128-row tiles (the second
    CTA of the last pair has nothing to do) and more tiles than pairs (several tiles per pair)."""
    from elmo_b200.handle import test_gemm
    g = torch.Generator().manual_seed(m + n + k)
    a = _rand((m, k), dtype, g); b = _rand((n, k), dtype, g)
    d = test_gemm(a, b, 4)
    ref = a.float() @ b.float().t()
    assert torch.allclose(d, ref, rtol=1e-4, atol=2e-3), float((d - ref).abs().max())


def test_a_wait_that_runs_out_on_a_cta_pair_is_reported_and_the_context_survives():
    """The same failure handling on a CTA pair: both CTAs leave out the load, every wait behind it gives
    up after about a millisecond, both CTAs meet at the closing cluster barrier and free their tensor memory."""
    from elmo_b200._lib import XmcError
    from elmo_b200.handle import test_gemm
    g = torch.Generator().manual_seed(6)
    a = _rand((512, 512), torch.bfloat16, g); b = _rand((256, 512), torch.bfloat16, g)
    with pytest.raises(XmcError, match=r"device status 1 .*site (10[0-7]|20[01]|30[0-7]|40[01])") as exc:
        test_gemm(a, b, 4 | 8)
    assert exc.value.code == 4
    d = test_gemm(a, b, 4)
    assert torch.allclose(d, a.float() @ b.float().t(), rtol=1e-4, atol=1e-3)
