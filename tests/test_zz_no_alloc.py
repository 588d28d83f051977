"""The allocation-free contraction entry point (xmc_large_k_matmul_noalloc) against the existing
tensor-core entry point that computes the same product with cudaMalloc'd scratch (xmc_test_gemm,
MN-major layout).  Some callers -- code under a device-owning memory pool, allocation-free serving
loops, hosted plug-ins -- cannot allocate where they call the library; this path must give them
the same numbers.  Collected last on purpose: a failure here must not hide the other tests."""
import ctypes as C

import pytest
import torch

pytestmark = pytest.mark.gpu


def _noalloc(a, b):
    from elmo_b200 import _lib
    lib = _lib.load()
    k, m = a.shape
    n = b.shape[1]
    out = torch.full((m, n), float("nan"), dtype=torch.float32, device=a.device)
    dt = _lib.DT_E4M3 if b.dtype == torch.float8_e4m3fn else _lib.DT_BF16
    stream = C.c_void_p(torch.cuda.current_stream(a.device).cuda_stream)
    _lib.check(lib.xmc_large_k_matmul_noalloc(a.device.index or 0, C.c_void_p(a.data_ptr()),
                                              C.c_void_p(b.data_ptr()), dt, k, m, n,
                                              C.c_void_p(out.data_ptr()), stream))
    _lib.check(lib.xmc_noalloc_check(a.device.index or 0, stream))     # synchronises; no wait gave up
    return out


def test_noalloc_matches_allocating_entry_point_twice_in_a_row():
    from elmo_b200.handle import test_gemm
    dev = torch.device("cuda", 0)
    g = torch.Generator().manual_seed(42)
    for k, m, n in [(5000, 512, 768), (777, 192, 320)]:          # two calls in a row share the scratch
        a = torch.randn(k, m, generator=g).to(torch.bfloat16).to(dev)
        b = torch.randn(k, n, generator=g).to(torch.bfloat16).to(dev)
        want = test_gemm(a, b, 1)                                # existing entry point
        got = _noalloc(a, b)
        assert torch.allclose(got, want, rtol=1e-4, atol=2e-3), float((got - want).abs().max())
    # same shape again: stale partial sums of the previous call must not leak into the result
    a2 = torch.randn(777, 192, generator=g).to(torch.bfloat16).to(dev)
    b2 = torch.randn(777, 320, generator=g).to(torch.bfloat16).to(dev)
    assert torch.allclose(_noalloc(a2, b2), test_gemm(a2, b2, 1), rtol=1e-4, atol=2e-3)


@pytest.mark.parametrize("k,m,n", [(20, 64, 64), (100, 128, 16384), (4000, 128, 256), (33, 2048, 1024)])
def test_noalloc_edge_shapes_against_fp32(k, m, n):
    """One accumulator (m <= 128), fewer k-steps than splits, and m * n at the 2 097 152 limit; bf16
    operands against torch in fp32."""
    dev = torch.device("cuda", 0)
    g = torch.Generator().manual_seed(k + m + n)
    a = torch.randn(k, m, generator=g).to(torch.bfloat16).to(dev)
    b = torch.randn(k, n, generator=g).to(torch.bfloat16).to(dev)
    want = a.float().t() @ b.float()
    got = _noalloc(a, b)
    assert torch.allclose(got, want, rtol=1e-4, atol=2e-3), float((got - want).abs().max())


def test_noalloc_allocates_nothing():
    """After the first call on the device, a call leaves the amount of free device memory unchanged."""
    dev = torch.device("cuda", 0)
    g = torch.Generator().manual_seed(1)
    a = torch.randn(1000, 256, generator=g).to(torch.bfloat16).to(dev)
    b = torch.randn(1000, 512, generator=g).to(torch.bfloat16).to(dev)
    _noalloc(a, b)                                              # set-up call
    out = torch.empty(256, 512, dtype=torch.float32, device=dev)
    from elmo_b200 import _lib
    lib = _lib.load()
    torch.cuda.synchronize(dev)
    free0, _ = torch.cuda.mem_get_info(dev)
    for _ in range(3):
        _lib.check(lib.xmc_large_k_matmul_noalloc(0, C.c_void_p(a.data_ptr()), C.c_void_p(b.data_ptr()), _lib.DT_BF16,
                                                  1000, 256, 512, C.c_void_p(out.data_ptr()), C.c_void_p(0)))
    _lib.check(lib.xmc_noalloc_check(0, C.c_void_p(0)))
    free1, _ = torch.cuda.mem_get_info(dev)
    assert free1 == free0
    assert torch.allclose(out, a.float().t() @ b.float(), rtol=1e-4, atol=2e-3)


def test_noalloc_e4m3_operand_and_size_limit():
    from elmo_b200._lib import XmcError
    dev = torch.device("cuda", 0)
    g = torch.Generator().manual_seed(7)
    a = torch.randn(3000, 256, generator=g).to(torch.bfloat16).to(dev)
    b8 = (torch.randn(3000, 256, generator=g) * 0.25).to(torch.float8_e4m3fn).to(dev)
    want = a.float().t() @ b8.float()
    got = _noalloc(a, b8)
    assert torch.allclose(got, want, rtol=1e-4, atol=2e-3)
    big_a = torch.zeros(64, 4096, dtype=torch.bfloat16, device=dev)
    big_b = torch.zeros(64, 1024, dtype=torch.bfloat16, device=dev)
    with pytest.raises(XmcError, match="exceeds the built-in scratch"):
        _noalloc(big_a, big_b)
