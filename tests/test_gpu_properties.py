"""Size-independent properties at the benchmark's full size (670 091 x 768, batch 512), where the
CPU oracle would take minutes, and the statistical test of the stochastic rounding:
  * a step with lr = 0 leaves every weight value untouched (RN and SR; only the sign of a zero may
    change) and still produces grad_X;
  * the step does not depend on how label rows are split into handles (sharding invariance):
    W' bit-identical, grad_X parts add up;
  * stochastic rounding is unbiased: mean error within 3 sigma of zero over > 10^7 draws,
    stratified over normal and subnormal e4m3 magnitudes."""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu
E4M3 = torch.float8_e4m3fn


def _handle(mode, d, B, offset=0, sched=0):
    from elmo_b200.handle import XmcHandle
    return XmcHandle(torch.device("cuda", 0), d, B, mode, label_offset=offset, sched_labels=sched)


def test_full_size_lr_zero_and_sharding_invariance():
    from elmo_b200 import synth
    wl = synth.WORKLOADS["cfg2"]
    L, d, B = 670208, wl.dim, wl.batch                       # padded label count of the FP8 class at nc = 11
    dev = torch.device("cuda", 0)
    gen = torch.Generator().manual_seed(0)
    w = torch.empty(L, d, dtype=E4M3, device=dev)
    for s0 in range(0, L, 65536):
        blk = w[s0:s0 + 65536]
        blk.copy_(synth.make_weights_f32(blk.shape[0], d, gen).to(E4M3))
    x, lab = synth.make_step_inputs(wl, seed=3)
    x, lab = x.to(dev), lab.to(dev)

    # (1) lr = 0: weights untouched bit for bit, grad_X finite and non-trivial
    chunks = list(w.clone().split(60928))
    h = _handle("fp8", d, B)
    h.bind(chunks)
    g0 = torch.zeros(B, d, dtype=torch.float32, device=dev)
    for stochastic in (False, True):
        h.step(x, lab, 0.0, seed=7, step=1, stochastic=stochastic, grad_f32=g0)
        h.check()
        now = torch.cat(chunks)
        # the only bits that may move are signs of zeros (w - 0*acc is +0 or -0 depending on the sign of acc)
        diff = now.view(torch.uint8) != w.view(torch.uint8)
        assert bool(((w.view(torch.uint8)[diff] & 0x7F) == 0).all()) and bool(((now.view(torch.uint8)[diff] & 0x7F) == 0).all())
        assert float(diff.float().mean()) < 0.05
        w = now.clone()
    assert torch.isfinite(g0).all() and float(g0.abs().max()) > 0

    # (2) one handle over all rows == two handles over the two halves (same Philox stream)
    h.step(x, lab, wl.lr, seed=7, step=2, stochastic=True, grad_f32=g0)
    h.check()
    full = torch.cat(chunks)
    half = 335104                                            # multiple of 16
    parts, gsum = [], torch.zeros_like(g0)
    for lo, hi in ((0, half), (half, L)):
        wp = [w[lo:hi].clone()]
        hp = _handle("fp8", d, B, offset=lo)
        hp.bind(wp)
        gp = torch.zeros_like(g0)
        hp.step(x, lab, wl.lr, seed=7, step=2, stochastic=True, grad_f32=gp)
        hp.check()
        parts.append(wp[0]); gsum += gp
        hp.close()
    assert torch.equal(torch.cat(parts).view(torch.uint8), full.view(torch.uint8))
    assert float((gsum - g0).abs().max()) <= 1e-4 * float(g0.abs().max())
    changed = float((full.view(torch.uint8) != w.view(torch.uint8)).float().mean())
    assert changed > 0.5                                     # at initialisation (sigmoid ~ 0.5) most weights move
    h.close()


@pytest.mark.parametrize("mode,dtype", [("fp8", E4M3), ("bf16", torch.bfloat16)])
def test_stochastic_rounding_is_unbiased_over_1e7_draws(mode, dtype):
    """With X = 0 the contraction vanishes and the update is w <- SR(w * (1 - lr*wd)): every element
    is an independent draw with a known target that is off the grid."""
    dev = torch.device("cuda", 0)
    L, d, B = 16384, 768, 16                                 # 12.6 M draws
    values = torch.tensor([0.3125, -1.75, 0.0234375, -0.0078125, 0.001953125, 104.0, -0.01171875, 0.5],
                          dtype=torch.float32)               # normal and subnormal e4m3 magnitudes
    w0 = values.repeat((L * d) // len(values)).reshape(L, d).to(dtype).to(dev)
    assert torch.equal(w0.float().cpu().reshape(-1)[:8], values)       # all exactly representable
    w = [w0.clone()]
    h = _handle(mode, d, B)
    h.bind(w)
    x = torch.zeros(B, d, dtype=torch.bfloat16, device=dev)
    lr, wd = 1.0, 0.37
    h.step(x, None, lr, wd=wd, seed=123, step=5, stochastic=True)
    h.check()
    got = w[0].float().cpu().reshape(-1, len(values))
    factor = float(torch.tensor(1.0, dtype=torch.float32) - torch.tensor(lr * wd, dtype=torch.float32))
    for j, v in enumerate(values.tolist()):
        # target as the kernel computes it: fma(-lr, wd*w, w) in fp32
        t32 = torch.tensor(v, dtype=torch.float32)
        target = float(torch.addcmul(t32, torch.tensor(-lr, dtype=torch.float32), torch.tensor(wd, dtype=torch.float32) * t32))
        col = got[:, j].double()
        lo, hi = float(col.min()), float(col.max())
        assert lo <= target <= hi and len(torch.unique(col)) == 2, (v, lo, hi)     # the two grid neighbours
        p_up = (target - lo) / (hi - lo)
        n = col.numel()
        sigma_mean = (hi - lo) * math.sqrt(p_up * (1 - p_up) / n)
        err = float(col.mean()) - target
        assert abs(err) <= 3 * sigma_mean + (hi - lo) * 2.0 ** -16, (v, err, sigma_mean)
        assert abs(factor * v - target) <= abs(v) * 1e-6
    h.close()
