"""The CPU oracle replayed against outputs of the reference's own Triton kernels and FP8 layer classes,
recorded on a B200 by tests/golden/make_golden_gpu.py (fixtures tests/golden/gpu_*.npz).

With rounding mode 'sr_triton' the oracle draws the reference's random stream (tl.randint with the
host-drawn per-launch seed), so stochastically rounded weights are compared bit for bit."""
import json
import os

import numpy as np
import pytest
import torch

from oracle import xmc_oracle as O
from tests._util import GOLDEN, as_bf16, as_e4m3, frac_equal_bits, load_golden, rel_inf
from tests.golden import gpu_cases


def as_e5m2(a):
    return torch.from_numpy(np.ascontiguousarray(a)).view(torch.float8_e5m2)


def test_sr_helpers_bit_exact():
    # stochastic_rounding_kernel.py:10-27,54-62: pins tl.randint's stream and the fp32->e4m3 convert
    # (round-to-nearest-even below 2^-6, saturation at +-448) on normal, subnormal and overflowing inputs
    g = load_golden("gpu_sr_helpers.npz")
    x = g["x"]
    finite = ~np.isnan(x)
    for seed in (123, 999983):
        o8 = O.sr_triton(x, seed, "e4m3").view(torch.uint8).numpy()
        assert np.array_equal(o8, g[f"e4m3_seed{seed}"])               # NaN included
        o16 = O.sr_triton(x, seed, "bf16").view(torch.uint16).numpy()
        assert np.array_equal(o16[finite], g[f"bf16_seed{seed}"][finite])


def test_large_k_matmul_matches_reference():
    # matmul_kernel.py:204-239: fp32 atomics in unspecified order -> tolerance, not bits
    g = load_golden("gpu_large_k.npz")
    for i, (tag, k, m, n) in enumerate(gpu_cases.LARGE_K_CASES):
        G, w8, w16 = gpu_cases.large_k_inputs(i)
        if gpu_cases.digest(G, w8, w16) != str(g[f"{tag}_inputs_sha256"]):
            pytest.skip("this torch build's CPU generator does not reproduce the fixture inputs")
        assert tuple(g[f"{tag}_shape"]) == (k, m, n)
        for wname, W in (("w8", w8), ("w16", w16)):
            ref = torch.from_numpy(g[f"{tag}_c_{wname}"])
            assert rel_inf(O.large_k_matmul(G, W), ref) < 1e-5, (tag, wname)


@pytest.mark.parametrize("tag", ["small", "wide", "top", "odd"])
def test_matmul_update_bit_exact(tag):
    # fuse_kernel.py:63-131 on e4m3 weights: acc, the lr*acc contraction, the SR bit trick and the
    # saturating convert ('top' pushes weights past +-448)
    g = load_golden("gpu_matmul_update.npz")
    G, X = as_bf16(g[f"{tag}_g"]), as_bf16(g[f"{tag}_x"])
    W, ref = as_e4m3(g[f"{tag}_w8_before"]), as_e4m3(g[f"{tag}_w8_after"])
    w_upd = O.fused_update(W.float(), O.matmul_acc(G, X), float(g[f"{tag}_lr"]))
    out = O.round_update(w_upd, O.E4M3, "sr_triton", int(g[f"{tag}_seed"]), 0, 0)
    assert frac_equal_bits(out, ref) >= 0.999
    assert not torch.isnan(ref.float()).any()                          # the convert saturates, no NaN
    # every reference value is one of the two e4m3 neighbours of the fp32 update
    # (grid step <= |w| / 8 in the normal range, 2^-9 below 2^-6)
    assert ((ref.float() - w_upd.clamp(-448, 448)).abs() <= w_upd.abs().clamp_min(2.0 ** -6) * 0.125).all()


@pytest.mark.parametrize("tag,conv", [("dbf16", as_bf16), ("de5m2", as_e5m2)])
def test_kahan_update_matches_reference(tag, conv):
    # fuse_kernel.py:202-287.  W' is bit exact.  On the stack the fixture was recorded with (triton 3.6.0,
    # sm_100) the kernel's re-conversion of the freshly rounded e4m3 weights to fp32 (:266) comes back
    # wrong in columns 0 and 1 of every group of four (W' read as 0, or the buffer set to 384.0), so the
    # compensation buffer is compared on columns 2 and 3 of every four, where the reference is sane.
    g = load_golden("gpu_kahan_update.npz")
    G, X = as_bf16(g[f"{tag}_g"]), as_bf16(g[f"{tag}_x"])
    W, D = as_e4m3(g[f"{tag}_w_before"]), conv(g[f"{tag}_d_before"])
    lr, seed = float(g[f"{tag}_lr"]), int(g[f"{tag}_seed"])
    for s in range(2):
        acc = O.matmul_acc(G, X)
        w32, k32 = W.float(), D.float()
        head = O.round_update(O.fused_update(w32 + k32, acc, lr), O.E4M3, "sr_triton", seed + s, 0, 0)
        knew = (k32 + w32 - head.float() - float(np.float32(lr)) * acc).to(D.dtype)
        ref_w, ref_d = as_e4m3(g[f"{tag}_w_after{s}"]), conv(g[f"{tag}_d_after{s}"])
        assert frac_equal_bits(head, ref_w) >= 0.999
        sane = torch.zeros_like(acc, dtype=torch.bool)
        sane[:, 2::4] = True
        sane[:, 3::4] = True
        assert frac_equal_bits(knew[sane], ref_d[sane]) >= 0.999
        W, D = ref_w, ref_d                                            # carry the reference's state forward


def test_sgd_update_bit_exact():
    # stochastic_rounding_kernel.py:65-99 on bf16 weights
    g = load_golden("gpu_sgd_update.npz")
    W, dW = as_bf16(g["w_before"]), as_bf16(g["dw"])
    upd = (W.double() - dW.double() * float(np.float32(float(g["lr"])))).float()
    out = O.round_update(upd, torch.bfloat16, "sr_triton", int(g["seed"]), 0, 0)
    assert frac_equal_bits(out, as_bf16(g["w_after"])) >= 0.999


@pytest.mark.parametrize("fname", ["gpu_fp8_layer.npz", "gpu_kahan_layer.npz"])
def test_fp8_layer_steps_match_reference(fname):
    # Fp8XMCBCEChunkedLayer / Fp8XMCBCEChunkedHeadKahanLayer.xfc_forward_backward, two steps, real FP8
    g = load_golden(fname)
    nc, lr, L = int(g["nc"]), float(g["lr"]), int(g["L"])
    assert O.fp8_padded_labels(L, nc) == (int(g["L_padded"]), int(g["L_i"]))
    ws = [as_e4m3(g[f"w0_{i}"]) for i in range(nc)]
    for s in range(2):
        x, lab = as_bf16(g[f"x{s}"]), torch.from_numpy(g[f"labels{s}"])
        kah = as_bf16(g[f"kahan{s}"]).clone() if "kahan0" in g else None
        new, gx, _ = O.fp8_chunked_step(ws, x, lab, lr, rounding="sr_triton",
                                        chunk_seeds=g["seeds"][s].tolist(), kahan=kah)
        for i in range(nc):
            assert frac_equal_bits(new[i], as_e4m3(g[f"w{s + 1}_{i}"])) >= 0.999, (s, i)
        ref_gx = as_bf16(g[f"grad_input{s}"])
        assert rel_inf(gx.to(torch.bfloat16), ref_gx) < 1e-2
        assert frac_equal_bits(gx.to(torch.bfloat16), ref_gx) >= 0.99
        if kah is not None:                                            # see test_kahan_update_matches_reference
            ref_k = as_bf16(g[f"kahan{s + 1}"])
            sane = torch.zeros_like(kah, dtype=torch.bool)
            sane[:, 2::4] = True
            sane[:, 3::4] = True
            assert frac_equal_bits(kah[sane], ref_k[sane]) >= 0.999
        ws = [as_e4m3(g[f"w{s + 1}_{i}"]) for i in range(nc)]
    z = O.forward_logits(ws, x, num_labels=L)
    assert frac_equal_bits(z, as_bf16(g["logits_last"])) >= 0.999


def test_chunked_bf16_steps_match_reference():
    # XMCBCECHUNKEDLayer in bfloat16 on the GPU, its own stochastic rounding included
    g = load_golden("gpu_chunked_bf16.npz")
    nc, lr = int(g["nc"]), float(g["lr"])
    w = as_bf16(g["w0"])
    for s in range(2):
        x, lab = as_bf16(g[f"x{s}"]), torch.from_numpy(g[f"labels{s}"])
        wn, gx, _ = O.chunked_step(w, x, lab, lr, num_chunks=nc, rounding="sr_triton",
                                   chunk_seeds=g["seeds"][s].tolist())
        ref = as_bf16(g[f"w{s + 1}"])
        assert frac_equal_bits(wn, ref) >= 0.999
        assert rel_inf(gx.to(torch.bfloat16), as_bf16(g[f"grad_input{s}"])) < 1e-2
        w = ref


def test_report_records_what_ran():
    rep = json.load(open(os.path.join(GOLDEN, "gpu_report.json")))
    ok = {k for k, v in rep["parts"].items() if v["ok"]}
    assert {"sr_helpers", "large_k", "matmul_update", "kahan_update", "sgd_update", "fp8_layer", "kahan_layer",
            "chunked_bf16"} <= ok
    # the simulated-FP8 update does not compile on this Triton (fuse_kernel.py:42 masks an unsigned
    # tensor with a negative constant): recorded, not pinned
    assert not rep["parts"]["fakefp8_update"]["ok"]
