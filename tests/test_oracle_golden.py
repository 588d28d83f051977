"""The CPU oracle replayed against fixtures produced by the unmodified reference on CPU
(tests/golden/make_golden.py)."""
import numpy as np
import torch

from oracle import xmc_oracle as O
from tests._util import as_bf16, as_e4m3, load_golden, rel_inf


def test_chunked_fp32_matches_reference():
    g = load_golden("chunked_fp32.npz")
    w = torch.from_numpy(g["w0"])
    for s in range(2):
        x = torch.from_numpy(g[f"x{s}"]); lab = torch.from_numpy(g[f"labels{s}"])
        w, gx, _ = O.chunked_step(w, x, lab, float(g["lr"]), num_chunks=int(g["nc"]))
        ref_w = torch.from_numpy(g[f"w{s + 1}"])
        # same torch ops in the same order -> equal up to matmul blocking (threads differ)
        assert rel_inf(w, ref_w) < 1e-6
        assert rel_inf(gx, torch.from_numpy(g[f"grad_input{s}"])) < 1e-5


def test_chunked_bf16_matches_reference_rn():
    g = load_golden("chunked_bf16.npz")
    w = as_bf16(g["w0"])
    for s in range(2):
        x = as_bf16(g[f"x{s}"]); lab = torch.from_numpy(g[f"labels{s}"])
        w, gx, _ = O.chunked_step(w, x, lab, float(g["lr"]), num_chunks=int(g["nc"]), rounding="rn")
        ref_w = as_bf16(g[f"w{s + 1}"])
        same = (w.view(torch.int16) == ref_w.view(torch.int16)).float().mean()
        assert same >= 0.999, same
        assert (w.float() - ref_w.float()).abs().max() <= 2.0 ** -8 * ref_w.float().abs().max()
        ref_gx = as_bf16(g[f"grad_input{s}"])
        assert rel_inf(gx.to(torch.bfloat16), ref_gx) < 1e-2
    logits = O.forward_logits([w], as_bf16(g["x1"]))
    assert rel_inf(logits, as_bf16(g["logits_last"])) < 1e-2


def test_fp8_forward_matches_reference():
    g = load_golden("fp8_forward.npz")
    nc = int(g["nc"]); L = int(g["L"])
    assert O.fp8_padded_labels(L, nc) == (int(g["L_padded"]), int(g["L_i"]))
    for tag, sim in (("real", False), ("sim", True)):
        ws = [as_e4m3(g[f"{tag}_w{i}"]) for i in range(nc)]
        x = as_bf16(g[f"{tag}_x"])
        z = O.forward_logits(ws, x, simulated=sim, num_labels=L)
        ref = as_bf16(g[f"{tag}_logits"])
        assert z.shape == ref.shape
        same = (z.view(torch.int16) == ref.view(torch.int16)).float().mean()
        assert same >= 0.999, (tag, same)
        assert rel_inf(z, ref) < 1e-2
        z8 = O.forward_logits(ws, x.to(torch.float8_e4m3fn), simulated=sim, num_labels=L)
        assert rel_inf(z8, as_bf16(g[f"{tag}_logits_e4m3_embed"])) < 1e-2


def test_loss_matches_reference():
    g = load_golden("loss.npz")
    z = torch.from_numpy(g["z"])
    y = torch.zeros_like(z, dtype=torch.bool)
    y[torch.from_numpy(g["rows"]), torch.from_numpy(g["cols"])] = True
    assert abs(O.bce_sum_loss(z, y) - float(g["loss"])) < 1e-3 * abs(float(g["loss"]))


def test_padding_formula_adds_full_block_when_aligned():
    # chunked_fp8xmc_clf.py:26: an already aligned label count still grows by 16*nc
    assert O.fp8_padded_labels(500000, 10) == (500160, 50016)
    assert O.fp8_padded_labels(670091, 11) == (670208, 60928)
    assert O.fp8_padded_labels(670091, 2) == (670112, 335056)
