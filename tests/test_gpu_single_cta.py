"""The single-CTA kernels (what a device that cannot hold CTA pairs gets, XMC_NO_PAIRS=1) against the CPU
oracle, and against the CTA-pair kernels of the same build.

The switch is read once per process, so the single-CTA step runs in a child process that writes its
results to a file; this process runs the same step on CTA pairs.  Forward and update use the same
arithmetic on both paths (updated weights bit for bit); grad_X and the loss group their sums differently."""
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu

CHILD = r"""
import sys, torch
sys.path.insert(0, sys.argv[1])
from tests.test_gpu_step import _inputs, _run_gpu
L, d, B = 2304 + 128, 512, 512            # an odd number of 128-row label tiles, two batch tiles
w, x, lab = _inputs(L, d, B, 6 * B, seed=77)
got_w, g32, g16, loss = _run_gpu("fp8", [w[:1280], w[1280:]], x, lab, 0.5, stochastic=True, step=4, loss=True)
torch.save({"w": got_w, "g32": g32, "loss": loss}, sys.argv[2])
"""


def test_single_cta_kernels_match_the_oracle_and_the_pair_kernels(tmp_path):
    from oracle import xmc_oracle as O
    from tests._util import rel_inf
    from tests.test_gpu_step import _check_weights, _inputs, _run_gpu
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    out = str(tmp_path / "single.pt")
    env = dict(os.environ, XMC_NO_PAIRS="1")
    res = subprocess.run([sys.executable, "-c", CHILD, root, out], env=env, capture_output=True, text=True, timeout=600)
    assert res.returncode == 0, res.stderr[-2000:]
    single = torch.load(out)
    L, d, B = 2304 + 128, 512, 512
    w, x, lab = _inputs(L, d, B, 6 * B, seed=77)
    chunks = [w[:1280], w[1280:]]
    want_w, want_gx, want_loss = O.fp8_chunked_step(chunks, x, lab, 0.5, rounding="sr", seed=5, step=4, compute_loss=True)
    _check_weights(single["w"], want_w)
    assert rel_inf(single["g32"], want_gx) < 1e-2
    assert abs(single["loss"] - want_loss) < 1e-3 * abs(want_loss)
    pair_w, pair_g32, _, pair_loss = _run_gpu("fp8", chunks, x, lab, 0.5, stochastic=True, step=4, loss=True)
    for a, b in zip(pair_w, single["w"]):
        assert torch.equal(a.view(torch.uint8), b.view(torch.uint8))
    assert rel_inf(pair_g32, single["g32"]) < 1e-5
    assert abs(pair_loss - single["loss"]) <= 1e-6 * abs(pair_loss)      # partial sums are grouped differently
