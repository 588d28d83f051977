"""Per-tensor scale bookkeeping on the GPU: statistics pass, power-of-two rescale, and a layer that starts
where the reference starts (everything below e4m3's normal range) and lets the keeper lift the weights."""
from types import SimpleNamespace as NS

import pytest
import torch

from tests._util import frac_equal_bits, rel_inf

pytestmark = pytest.mark.gpu
E4M3 = torch.float8_e4m3fn


def _handle(w, scale=1.0):
    from elmo_b200.handle import XmcHandle
    dev = torch.device("cuda", 0)
    h = XmcHandle(dev, w.shape[1], 64, "fp8", w_scale=scale)
    wd = [w.clone().to(dev)]
    h.bind(wd)
    return h, wd


def test_weight_stats_match_torch():
    g = torch.Generator().manual_seed(2)
    w = (torch.randn(3000, 128, generator=g) * torch.exp2(torch.randint(-12, 9, (3000, 1), generator=g).float()))
    w = w.clamp(-448, 448).to(E4M3)                             # torch's cast turns values beyond 464 into NaN
    w.view(torch.uint8)[5, 5] = 0x7F
    h, _ = _handle(w)
    st = h.weight_stats()
    f = w.float()
    fin = ~torch.isnan(f)
    assert st["nan"] == int((~fin).sum()) == 1 and st["elements"] == w.numel()
    assert st["zeros"] == int((f == 0).sum())
    assert st["subnormal"] == int(((f != 0) & (f.abs() < 2.0 ** -6)).sum())
    assert st["saturated"] == int((f.abs() == 448).sum())
    assert st["amax_stored"] == float(f[fin].abs().max())
    h.close()


def test_rescale_keeps_real_values():
    g = torch.Generator().manual_seed(3)
    w = (torch.randn(2048, 64, generator=g) * 0.5).to(E4M3)
    h, wd = _handle(w)
    h.rescale(-2, stochastic=False)                             # stored x 4, exact (nothing near 448 / 4)
    assert h.w_scale == 0.25
    assert torch.equal(wd[0].float().cpu(), w.float() * 4)
    h.rescale(2, stochastic=False)                              # and back: bit identical
    assert h.w_scale == 1.0 and torch.equal(wd[0].cpu().view(torch.uint8), w.view(torch.uint8))
    # shrinking by 2^5 pushes most values below the normal range: stochastic rounding keeps the mean
    h.rescale(5, stochastic=True, seed=11, step=3)
    real = wd[0].float().cpu() * h.w_scale
    assert h.w_scale == 32.0
    err = (real - w.float())
    assert abs(float(err.mean())) < 4 * float(err.std()) / err.numel() ** 0.5
    assert float(err.abs().max()) <= 32 * 2.0 ** -9 + 1e-9       # one grid step of the new scale
    h.close()


def test_step_after_rescale_matches_oracle_with_the_new_scale():
    from oracle import xmc_oracle as O
    g = torch.Generator().manual_seed(4)
    L, d, B = 1024, 128, 64
    w = ((torch.rand(L, d, generator=g) * 2 - 1) * 3e-3).to(E4M3)      # the reference's start: sub-normal weights
    x = (torch.randn(B, d, generator=g) / d ** 0.5).to(torch.bfloat16)
    lab = torch.stack([torch.randint(0, B, (200,), generator=g), torch.randint(0, L, (200,), generator=g)], 1).to(torch.int32)
    h, wd = _handle(w)
    h.rescale(-8, stochastic=False)                             # lift by 2^8: exact
    assert h.w_scale == 2.0 ** -8
    lifted = wd[0].cpu().clone()
    assert torch.equal(lifted.float(), w.float() * 256)
    dev = wd[0].device
    g32 = torch.zeros(B, d, dtype=torch.float32, device=dev)
    h.step(x.to(dev), lab.to(dev), 0.05, seed=5, step=1, stochastic=True, grad_f32=g32)
    h.check()
    want, gx, _ = O.fp8_chunked_step([lifted], x, lab, 0.05, rounding="sr", seed=5, step=1, w_scale=2.0 ** -8)
    assert frac_equal_bits(wd[0].cpu(), want[0]) >= 0.999
    assert rel_inf(g32.cpu(), gx) < 1e-2
    h.close()


def test_layer_with_auto_scale_and_keeper():
    """'auto' puts the Xavier bound at 16..32 stored; a layer started at scale 1 (the reference's start)
    with the keeper on lifts itself out of the sub-normal range within a few checks."""
    from elmo_b200.xmc_classifiers import Fp8XMCBCEChunkedLayer

    def cfg(w_scale, interval):
        return NS(environment=NS(device="cuda:0"),
                  model=NS(xmc=NS(dtype="bfloat16", num_chunks=2, input_features=128)),
                  training=NS(precision=NS(mode="mixed", purelp_dtype="bfloat16"),
                              xmc=NS(momentum=0, wd=0.0, simulated_fp8=False, rounding="sr", w_scale=w_scale,
                                     scale_interval=interval),
                              FP8=NS(using_head_kahan=False, fp8_head_kahan=False, head_ratio=0.0)),
                  data=NS(num_labels=300000, batch_size=32))

    torch.manual_seed(0)
    auto = Fp8XMCBCEChunkedLayer(cfg("auto", 0))
    auto._handle.bind(auto._weights())
    s = auto._handle.weight_stats()
    assert 8.0 <= s["amax_stored"] <= 32.0 and s["frac_subnormal"] + s["frac_zero"] < 0.01

    ref = Fp8XMCBCEChunkedLayer(cfg(1.0, 2))
    ref._handle.bind(ref._weights())
    s0 = ref._handle.weight_stats()
    assert s0["frac_subnormal"] + s0["frac_zero"] > 0.9          # chunked_fp8xmc_clf.py:29-32 at scale 1
    g = torch.Generator().manual_seed(1)
    for it in range(12):
        x = (torch.randn(32, 128, generator=g) / 128 ** 0.5).to(torch.bfloat16).cuda()
        lab = torch.stack([torch.randint(0, 32, (100,), generator=g), torch.randint(0, 300000, (100,), generator=g)], 1)
        ref.xfc_forward_backward(x, lab.to(torch.int32).cuda(), [0.01])
    assert ref.w_scale < 1.0 and ref.w_scale == ref._handle.w_scale
    assert len(ref.scale_keeper.history) == 6 and ref.scale_keeper.history[0]["shift"] == -1
    # the extra state carries the moved scale; a fresh layer adopts it
    sd = ref.state_dict()
    twin = Fp8XMCBCEChunkedLayer(cfg(1.0, 0))
    twin.load_state_dict(sd)
    assert twin.w_scale == ref.w_scale and twin._handle.w_scale == ref.w_scale
