"""Head-Kahan variant (chunked_head_kahan_fp8xmc_clf.py, fuse_kernel.py:202-287) against the oracle."""
from types import SimpleNamespace as NS

import pytest
import torch

from tests._util import e4m3_ulp_distance, frac_equal_bits, rel_inf

pytestmark = pytest.mark.gpu


def _cfg(L, d, B, nc, fp8_kahan, ratio, rounding):
    return NS(environment=NS(device="cuda:0"),
              model=NS(xmc=NS(dtype="bfloat16", num_chunks=nc, input_features=d, sched_labels=512)),
              training=NS(precision=NS(mode="mixed", purelp_dtype="bfloat16"),
                          xmc=NS(momentum=0, wd=0.0, simulated_fp8=False, rounding=rounding),
                          FP8=NS(using_head_kahan=True, fp8_head_kahan=fp8_kahan, head_ratio=ratio)),
              data=NS(num_labels=L, batch_size=B))


@pytest.mark.parametrize("fp8_kahan", [False, True])
@pytest.mark.parametrize("rounding", ["rn", "sr"])
def test_kahan_head_matches_oracle(fp8_kahan, rounding):
    from elmo_b200.xmc_classifiers import Fp8XMCBCEChunkedHeadKahanLayer
    from oracle import xmc_oracle as O
    L, d, B, nc = 3000, 128, 64, 2
    layer = Fp8XMCBCEChunkedHeadKahanLayer(_cfg(L, d, B, nc, fp8_kahan, 0.23, rounding))
    nh = layer.num_head
    assert nh == int(0.23 * layer.num_labels) and nh % 128 != 0 and nh > 512      # crosses tiles and chunks
    gen = torch.Generator().manual_seed(11)
    ws = []
    for p in layer.xfc_weight:
        w = (torch.randn(p.shape, generator=gen) * 0.25).to(torch.float8_e4m3fn)
        p.data.copy_(w); ws.append(w)
    kah = torch.zeros(nh, d, dtype=layer.head_kahan.dtype)
    for it in range(3):                                        # the buffer matters from step 2 on
        x = (torch.randn(B, d, generator=gen) / d ** 0.5).to(torch.bfloat16)
        cols = torch.randint(0, L, (300,), generator=gen)
        cols = torch.where(torch.rand(300, generator=gen) < 0.5, cols % 40, cols)   # head labels are hot
        lab = torch.stack([torch.randint(0, B, (300,), generator=gen), cols], 1).to(torch.int32)
        layer.xfc_forward_backward(x.cuda(), lab.cuda(), [0.3])
        ws, gx, _ = O.fp8_chunked_step(ws, x, lab, 0.3, rounding=rounding, seed=layer.base_seed, step=it,
                                       kahan=kah)
        assert rel_inf(layer.grad_input.float().cpu(), gx) < 1e-2
    layer._handle.check()
    for p, w in zip(layer.xfc_weight, ws):
        got = p.data.cpu()
        assert frac_equal_bits(got, w) >= 0.995
        assert e4m3_ulp_distance(got, w) <= 1
    got_k = layer.head_kahan.float().cpu()
    want_k = kah.float()
    assert float((got_k != 0).float().mean()) > 0.3            # the compensation is actually in use
    close = ((got_k - want_k).abs() <= 0.26 * want_k.abs().clamp_min(2.0 ** -12)).float().mean()
    assert close >= 0.99, close
