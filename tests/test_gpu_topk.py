"""Fused logits + top-k (xfc_forward followed by torch.topk in the reference's evaluator,
evaluate.py:158-159,235-236) against the oracle; the logits are never materialised on the GPU."""
from types import SimpleNamespace as NS

import pytest
import torch

pytestmark = pytest.mark.gpu


def _cfg(L, d, B, nc, sim=False, sched=0):
    return NS(environment=NS(device="cuda:0"),
              model=NS(xmc=NS(dtype="bfloat16", num_chunks=nc, input_features=d, sched_labels=sched)),
              training=NS(precision=NS(mode="mixed", purelp_dtype="bfloat16"),
                          xmc=NS(momentum=0, wd=0.0, simulated_fp8=sim)),
              data=NS(num_labels=L, batch_size=B))


@pytest.mark.parametrize("k", [5, 20, 100])
@pytest.mark.parametrize("L,d,B,nc,sched", [(70001, 256, 200, 3, 0), (5000, 128, 300, 2, 1024)])
def test_topk_matches_oracle(L, d, B, nc, sched, k):
    from elmo_b200.xmc_classifiers import Fp8XMCBCEChunkedLayer
    from oracle import xmc_oracle as O
    layer = Fp8XMCBCEChunkedLayer(_cfg(L, d, B, nc, sched=sched))
    gen = torch.Generator().manual_seed(k + L)
    ws = []
    for p in layer.xfc_weight:
        w = (torch.randn(p.shape, generator=gen) * 0.25).to(torch.float8_e4m3fn)
        p.data.copy_(w); ws.append(w)
    x = (torch.randn(B - 3, d, generator=gen) / d ** 0.5).to(torch.bfloat16)
    vals, idx = layer.xfc_topk(x.cuda(), k)
    layer._handle.check()
    vals, idx = vals.cpu(), idx.cpu().long()
    assert vals.shape == idx.shape == (B - 3, k)
    z = O.forward_logits(ws, x, num_labels=L).to(torch.float32)           # [B, L] bf16-valued
    want_v, _ = O.topk_logits(ws, x, k, num_labels=L)
    assert int(idx.min()) >= 0 and int(idx.max()) < L                      # padding rows never show up
    assert all(len(set(r.tolist())) == k for r in idx)                     # no duplicates
    assert bool((vals[:, 1:] <= vals[:, :-1]).all())                       # descending
    ulp = z.abs().max() * 2.0 ** -7
    assert float((vals - torch.gather(z, 1, idx)).abs().max()) <= ulp      # reported value = that label's logit
    assert float((vals - want_v).abs().max()) <= ulp                       # and it is the k best, rank by rank


def test_topk_ties_take_lower_id_and_bf16_class():
    from elmo_b200.xmc_classifiers import XMCBCECHUNKEDLayer
    L, d, B = 1000, 64, 16
    cfg = _cfg(L, d, B, 1)
    layer = XMCBCECHUNKEDLayer(cfg)
    w = torch.zeros(L, d, dtype=torch.bfloat16)
    w[[7, 300, 999], 0] = 2.0                                              # three exact ties
    w[500, 0] = 3.0
    layer.xfc_weight.copy_(w)
    x = torch.zeros(B, d, dtype=torch.bfloat16); x[:, 0] = 1.0
    layer._handle.bind([layer.xfc_weight])
    vals, idx = layer._handle.forward_topk(x.cuda(), 4, L)
    layer._handle.check()
    assert idx.cpu().tolist() == [[500, 7, 300, 999]] * B
    assert vals.cpu().tolist() == [[3.0, 2.0, 2.0, 2.0]] * B


@pytest.mark.parametrize("k", [5, 40])
def test_topk_all_logits_equal_keeps_the_lowest_ids(k):
    """Every label ties with every other one across all CTAs, lists and launches: the published row
    threshold must not drop a lower id that arrives in another list."""
    from elmo_b200.handle import XmcHandle
    L, d, B = 40000, 64, 130
    dev = torch.device("cuda", 0)
    w = torch.zeros(L, d, dtype=torch.bfloat16)
    w[:, 0] = 1.5
    w[L // 2 + 11, 0] = 2.5                                                # one clear winner in the second chunk
    chunks = [w[:L // 2].contiguous().to(dev), w[L // 2:].contiguous().to(dev)]
    x = torch.zeros(B, d, dtype=torch.bfloat16)
    x[:, 0] = 1.0
    h = XmcHandle(dev, d, B, "bf16", sched_labels=4096)
    h.bind(chunks)
    vals, idx = h.forward_topk(x.to(dev), k, L)
    h.check()
    want = [L // 2 + 11] + list(range(k - 1))
    assert idx.cpu().tolist() == [want] * B
    assert vals.cpu()[:, 0].tolist() == [2.5] * B and bool((vals.cpu()[:, 1:] == 1.5).all())
    h.close()
