"""Generate tests/golden/gpu_*.npz by running the UNMODIFIED reference Triton kernels and FP8 layer
classes on one B200.

    python oracle/make_ref.py /path/to/reference          # where the reference is checked out
    python tests/golden/make_golden_gpu.py --out <dir>    # on the GPU box; then copy <dir>/gpu_*.npz here

The reference's packages are imported from ``oracle/_ref/src`` (the byte-for-byte staging copy that
``oracle/make_ref.py`` makes; git-ignored).  Inputs are drawn on the CPU from seeded generators
(tests/golden/gpu_cases.py) and stored next to the outputs -- the large_k_matmul inputs, which are
megabytes, are regenerated from their seed instead -- so the CPU tests need neither a GPU nor the
reference.

Fixtures (bf16 stored as uint16 bit patterns, e4m3/e5m2 as uint8):
  gpu_sr_helpers.npz     stochastic_rounding(x, out, seed)      stochastic_rounding_kernel.py:54-62 (e4m3, bf16)
  gpu_large_k.npz        large_k_matmul(G, W, bs=16)            matmul_kernel.py:204-239,342-353 (outputs; inputs by seed)
  gpu_matmul_update.npz  matmul_update(G, X, W, lr, seed)       fuse_kernel.py:63-131 (e4m3 and bf16 W)
  gpu_kahan_update.npz   kahan_matmul_update(...)               fuse_kernel.py:202-287 (bf16 and e5m2 buffer)
  gpu_fakefp8_update.npz fakefp8_matmul_update(...)             fuse_kernel.py:134-199
  gpu_sgd_update.npz     sgd_update(W, dW, ...)                 stochastic_rounding_kernel.py:65-99
  gpu_fp8_layer.npz      Fp8XMCBCEChunkedLayer.xfc_forward_backward x2 steps (real FP8)
  gpu_fp8_layer_sim.npz  same, simulated_fp8=True
  gpu_kahan_layer.npz    Fp8XMCBCEChunkedHeadKahanLayer x2 steps
  gpu_chunked_bf16.npz   XMCBCECHUNKEDLayer in bfloat16 x2 steps (stochastic rounding, as the reference does)
  gpu_report.json        versions, what compiled, what failed (with the error text), and -- with
                         --time-cfg2 -- the reference FP8 layer's step time and peak memory at 670 091 x 768
Every part runs once inside try/except: a part that does not compile is reported, not retried.
"""
import argparse
import json
import os
import sys
import time
import traceback
from types import SimpleNamespace as NS

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
REF_SRC = os.path.join(ROOT, "oracle", "_ref", "src")

sys.path.insert(0, HERE)
from gpu_cases import LARGE_K_CASES, digest, large_k_inputs, make_labels, update_inputs  # noqa: E402

E4M3 = torch.float8_e4m3fn
DEV = "cuda"


def bits(t):
    t = t.detach().cpu().contiguous()
    if t.dtype == torch.bfloat16:
        return t.view(torch.uint16).numpy()
    if t.dtype in (torch.float8_e4m3fn, torch.float8_e5m2):
        return t.view(torch.uint8).numpy()
    return t.numpy()


def cfg(L, d, B, nc, dtype="float8", sim=False, kahan=False, fp8_kahan=False, head_ratio=0.0):
    return NS(environment=NS(device=DEV),
              model=NS(xmc=NS(dtype=dtype, num_chunks=nc, input_features=d)),
              training=NS(precision=NS(mode="mixed", purelp_dtype="bfloat16"),
                          xmc=NS(momentum=0, wd=0.0, simulated_fp8=sim),
                          FP8=NS(using_head_kahan=kahan, fp8_head_kahan=fp8_kahan, head_ratio=head_ratio)),
              data=NS(num_labels=L, batch_size=B))


def seeds_after(manual_seed, count):
    """The per-chunk seeds the reference draws with torch.randint(0, 1000000, (1,)) from the global CPU
    generator after torch.manual_seed(manual_seed) (chunked_fp8xmc_clf.py:113)."""
    st = torch.random.get_rng_state()
    torch.manual_seed(manual_seed)
    out = [int(torch.randint(0, 1000000, (1,)).item()) for _ in range(count)]
    torch.random.set_rng_state(st)
    return out


# ----------------------------------------------------------------------------------------------
def part_sr_helpers(out_dir, rep):
    from triton_kernels.stochastic_rounding_kernel import stochastic_rounding
    g = torch.Generator().manual_seed(11)
    # a log-uniform sweep across e4m3's subnormal and normal range, signs mixed, plus edge values
    mag = torch.exp2(torch.rand(30000, generator=g) * 22.0 - 13.0)
    x = mag * torch.where(torch.rand(30000, generator=g) < 0.5, -1.0, 1.0)
    edge = torch.tensor([0.0, -0.0, 2.0 ** -9, 2.0 ** -10, 2.0 ** -11, 3 * 2.0 ** -10, 2.0 ** -6, 0.015624, 0.0157,
                         447.9, 448.0, 449.0, 463.9, 464.0, 465.0, 479.0, 480.0, 500.0, 1000.0, 1e6, -448.0, -470.0, -1e4,
                         float("inf"), float("-inf"), float("nan"), 1e-30, -1e-30, 3.3895e38])
    x = torch.cat([edge, x]).to(torch.float32).contiguous()
    res = {"x": x.numpy()}
    for seed in (123, 999983):
        for name, dt in (("e4m3", E4M3), ("bf16", torch.bfloat16)):
            o = torch.empty(x.shape, dtype=dt, device=DEV)
            stochastic_rounding(x.to(DEV), o, seed)
            torch.cuda.synchronize()
            res[f"{name}_seed{seed}"] = bits(o)
    np.savez_compressed(os.path.join(out_dir, "gpu_sr_helpers.npz"), **res)


def part_large_k(out_dir, rep):
    from triton_kernels.matmul_kernel import large_k_matmul
    res = {}
    for i, (tag, k, m, n) in enumerate(LARGE_K_CASES):
        G, w8, w16 = large_k_inputs(i)                      # regenerated from their seed by the test
        for wname, W in (("w8", w8), ("w16", w16)):
            c = large_k_matmul(G.to(DEV).contiguous(), W.to(DEV).contiguous(), 16)
            torch.cuda.synchronize()
            res[f"{tag}_c_{wname}"] = bits(c)
        res[f"{tag}_shape"] = np.array([k, m, n])
        res[f"{tag}_inputs_sha256"] = np.array(digest(G, w8, w16))
    np.savez_compressed(os.path.join(out_dir, "gpu_large_k.npz"), **res)


def part_matmul_update(out_dir, rep):
    from triton_kernels.fuse_kernel import matmul_update
    g = torch.Generator().manual_seed(31)
    res = {}
    cases = [("small", 384, 192, 64, 0.05, 4242), ("wide", 300, 200, 48, 0.5, 17), ("top", 128, 64, 32, 50.0, 5),
             ("odd", 130, 72, 17, 0.05, 999999)]
    for tag, m, n, k, lr, seed in cases:
        G, X, w = update_inputs(g, m, n, k, tag if tag in ("small", "wide", "top") else "small")
        for wname, dt in (("w8", E4M3), ("w16", torch.bfloat16)):
            W = w.to(dt).to(DEV).contiguous()
            before = bits(W)
            try:
                matmul_update(G.to(DEV).contiguous(), X.to(DEV).contiguous(), W, lr, seed)
                torch.cuda.synchronize()
                res[f"{tag}_{wname}_before"] = before
                res[f"{tag}_{wname}_after"] = bits(W)
            except Exception as e:                        # the bf16 helper may not compile on newer Triton
                rep.setdefault("matmul_update_errors", {})[f"{tag}_{wname}"] = type(e).__name__ + ": " + str(e)[-300:]
        res[f"{tag}_g"] = bits(G); res[f"{tag}_x"] = bits(X)
        res[f"{tag}_lr"] = np.float64(lr); res[f"{tag}_seed"] = np.int64(seed)
    np.savez_compressed(os.path.join(out_dir, "gpu_matmul_update.npz"), **res)


def part_kahan_update(out_dir, rep):
    from triton_kernels.fuse_kernel import kahan_matmul_update
    g = torch.Generator().manual_seed(41)
    res = {}
    for tag, ddt in (("dbf16", torch.bfloat16), ("de5m2", torch.float8_e5m2)):
        m, n, k, lr, seed = 256, 128, 32, 0.05, 777
        G, X, w = update_inputs(g, m, n, k, "small")
        W = w.to(E4M3).to(DEV).contiguous()
        D = (torch.randn(m, n, generator=g) * 2.0 ** -9).to(ddt).to(DEV).contiguous()
        res[f"{tag}_w_before"] = bits(W); res[f"{tag}_d_before"] = bits(D)
        for s in range(2):                                  # two updates in a row: the buffer carries over
            kahan_matmul_update(G.to(DEV).contiguous(), X.to(DEV).contiguous(), W, D, lr, seed + s)
            torch.cuda.synchronize()
            res[f"{tag}_w_after{s}"] = bits(W); res[f"{tag}_d_after{s}"] = bits(D)
        res[f"{tag}_g"] = bits(G); res[f"{tag}_x"] = bits(X)
        res[f"{tag}_lr"] = np.float64(lr); res[f"{tag}_seed"] = np.int64(seed)
    np.savez_compressed(os.path.join(out_dir, "gpu_kahan_update.npz"), **res)


def part_fakefp8_update(out_dir, rep):
    from triton_kernels.fuse_kernel import fakefp8_matmul_update
    g = torch.Generator().manual_seed(51)
    m, n, k, lr, seed = 256, 128, 32, 0.05, 31337
    G, X, w = update_inputs(g, m, n, k, "small")
    W16 = w.to(E4M3).to(torch.bfloat16).to(DEV).contiguous()
    res = {"w_before": bits(W16), "g": bits(G), "x": bits(X), "lr": np.float64(lr), "seed": np.int64(seed)}
    fakefp8_matmul_update(G.to(DEV).contiguous(), X.to(DEV).contiguous(), W16, lr, seed)
    torch.cuda.synchronize()
    res["w_after_bf16"] = bits(W16)
    res["w_after_e4m3"] = bits(W16.to(E4M3))                # chunked_fp8xmc_clf.py:116
    np.savez_compressed(os.path.join(out_dir, "gpu_fakefp8_update.npz"), **res)


def part_sgd_update(out_dir, rep):
    from triton_kernels.stochastic_rounding_kernel import sgd_update
    g = torch.Generator().manual_seed(61)
    m, n, lr, seed = 300, 96, 0.05, 4711
    W = (torch.randn(m, n, generator=g) * 0.02).to(torch.bfloat16).to(DEV).contiguous()
    dW = (torch.randn(m, n, generator=g) * 0.1).to(torch.bfloat16).to(DEV).contiguous()
    res = {"w_before": bits(W), "dw": bits(dW), "lr": np.float64(lr), "seed": np.int64(seed)}
    sgd_update(W, dW, None, lr, 0.0, True, seed)
    torch.cuda.synchronize()
    res["w_after"] = bits(W)
    np.savez_compressed(os.path.join(out_dir, "gpu_sgd_update.npz"), **res)


def run_fp8_layer(out_dir, fname, cls, c, steps=2, lr=0.05, manual_seed=2024, spread=True):
    g = torch.Generator().manual_seed(71)
    torch.manual_seed(5)
    layer = cls(c)
    nc, d, B = layer.num_chunks, c.model.xmc.input_features, c.data.batch_size
    if spread:
        # Xavier at scale 1 lands on three e4m3 values; spread the weights like the bench does
        for i in range(nc):
            w = (torch.rand(layer.num_labels_i, d, generator=g) * 2 - 1) / 768 ** 0.5
            layer.xfc_weight[i].data.copy_(w.to(E4M3))
    res = {"L": c.data.num_labels, "d": d, "B": B, "nc": nc, "lr": lr, "L_padded": layer.num_labels,
           "L_i": layer.num_labels_i}
    for i in range(nc):
        res[f"w0_{i}"] = bits(layer.xfc_weight[i].data)
    if hasattr(layer, "head_kahan"):
        res["num_head"] = layer.num_head
        res["kahan0"] = bits(layer.head_kahan)
    res["seeds"] = np.array(seeds_after(manual_seed, steps * nc), dtype=np.int64).reshape(steps, nc)
    torch.manual_seed(manual_seed)
    for s in range(steps):
        x = (torch.randn(B, d, generator=g) / d ** 0.5).to(torch.bfloat16)
        lab = make_labels(g, B, c.data.num_labels, 6)
        layer.xfc_forward_backward(x.to(DEV), lab.to(DEV), [lr], skip_loss=True)
        torch.cuda.synchronize()
        res[f"x{s}"] = bits(x); res[f"labels{s}"] = lab.numpy()
        for i in range(nc):
            res[f"w{s + 1}_{i}"] = bits(layer.xfc_weight[i].data)
        res[f"grad_input{s}"] = bits(layer.grad_input)
        if hasattr(layer, "head_kahan"):
            res[f"kahan{s + 1}"] = bits(layer.head_kahan)
    res["logits_last"] = bits(layer.xfc_forward(x.to(DEV)))
    np.savez_compressed(os.path.join(out_dir, fname), **res)


def part_fp8_layer(out_dir, rep):
    from xmc_classifiers.chunked_fp8xmc_clf import Fp8XMCBCEChunkedLayer
    run_fp8_layer(out_dir, "gpu_fp8_layer.npz", Fp8XMCBCEChunkedLayer, cfg(1000, 128, 32, 3))


def part_fp8_layer_sim(out_dir, rep):
    from xmc_classifiers.chunked_fp8xmc_clf import Fp8XMCBCEChunkedLayer
    run_fp8_layer(out_dir, "gpu_fp8_layer_sim.npz", Fp8XMCBCEChunkedLayer, cfg(1000, 128, 32, 3, sim=True))


def part_kahan_layer(out_dir, rep):
    from xmc_classifiers.chunked_head_kahan_fp8xmc_clf import Fp8XMCBCEChunkedHeadKahanLayer
    run_fp8_layer(out_dir, "gpu_kahan_layer.npz", Fp8XMCBCEChunkedHeadKahanLayer,
                  cfg(1000, 128, 32, 3, kahan=True, fp8_kahan=False, head_ratio=0.2))


def part_chunked_bf16(out_dir, rep):
    import xmc_classifiers.chunked as ref_chunked
    L, d, B, nc, lr, steps, manual_seed = 520, 64, 24, 3, 0.05, 2, 77
    g = torch.Generator().manual_seed(81)
    layer = ref_chunked.XMCBCECHUNKEDLayer(cfg(L, d, B, nc, dtype="bfloat16"))
    w0 = ((torch.rand(L, d, generator=g) * 2 - 1) / d ** 0.5).to(torch.bfloat16)
    layer.xfc_weight.copy_(w0)
    res = {"L": L, "d": d, "B": B, "nc": nc, "lr": lr, "w0": bits(w0),
           "seeds": np.array(seeds_after(manual_seed, steps * nc), dtype=np.int64).reshape(steps, nc)}
    torch.manual_seed(manual_seed)
    for s in range(steps):
        x = (torch.randn(B, d, generator=g) / d ** 0.5).to(torch.bfloat16)
        lab = make_labels(g, B, L, 6)
        layer.xfc_forward_backward(x.to(DEV), lab.to(DEV), [lr], skip_loss=True)
        torch.cuda.synchronize()
        res[f"x{s}"] = bits(x); res[f"labels{s}"] = lab.numpy()
        res[f"w{s + 1}"] = bits(layer.xfc_weight); res[f"grad_input{s}"] = bits(layer.grad_input)
    np.savez_compressed(os.path.join(out_dir, "gpu_chunked_bf16.npz"), **res)


def part_time_cfg2(out_dir, rep):
    """Step time and peak memory of the reference's own FP8 layer at 670 091 x 768, batch 512, 11 chunks."""
    from xmc_classifiers.chunked_fp8xmc_clf import Fp8XMCBCEChunkedLayer
    sys.path.insert(0, ROOT)
    from elmo_b200 import synth
    wl = synth.WORKLOADS["cfg2"]
    torch.cuda.empty_cache()
    torch.cuda.reset_peak_memory_stats()
    base = torch.cuda.memory_allocated()
    layer = Fp8XMCBCEChunkedLayer(cfg(wl.num_labels, wl.dim, wl.batch, wl.num_chunks))
    gen = torch.Generator().manual_seed(0)
    for p in layer.xfc_weight:
        p.data.copy_(synth.make_weights_f32(p.shape[0], wl.dim, gen).to(E4M3))
    weights_bytes = torch.cuda.memory_allocated() - base
    pool = [synth.make_step_inputs(wl, seed=1000 + i) for i in range(4)]
    pool = [(x.to(DEV), l.to(DEV)) for x, l in pool]
    for i in range(3):
        layer.xfc_forward_backward(*pool[i % 4], [wl.lr], skip_loss=True)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    n = 10
    e0.record()
    for i in range(n):
        layer.xfc_forward_backward(*pool[i % 4], [wl.lr], skip_loss=True)
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / n
    rep["reference_fp8_layer_cfg2"] = {
        "ms_per_step": ms, "samples_per_s": wl.batch / (ms * 1e-3), "steps_timed": n, "warmup": 3,
        "num_chunks": wl.num_chunks, "rows_padded": layer.num_labels,
        "weights_bytes": int(weights_bytes),
        "max_memory_allocated_bytes": int(torch.cuda.max_memory_allocated() - base),
        "note": "unmodified Fp8XMCBCEChunkedLayer.xfc_forward_backward, CUDA events, inputs resident"}


PARTS = [("sr_helpers", part_sr_helpers), ("large_k", part_large_k), ("matmul_update", part_matmul_update),
         ("kahan_update", part_kahan_update), ("fakefp8_update", part_fakefp8_update), ("sgd_update", part_sgd_update),
         ("fp8_layer", part_fp8_layer), ("fp8_layer_sim", part_fp8_layer_sim), ("kahan_layer", part_kahan_layer),
         ("chunked_bf16", part_chunked_bf16)]


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--out", default=HERE)
    ap.add_argument("--time-cfg2", action="store_true")
    ap.add_argument("--only", default="")
    args = ap.parse_args()
    if not os.path.isdir(REF_SRC):
        sys.exit("oracle/_ref/src is missing: run oracle/make_ref.py where the reference is checked out")
    assert torch.cuda.is_available(), "this generator runs the reference's Triton kernels: it needs a GPU"
    sys.path.insert(0, REF_SRC)
    os.environ.setdefault("TORCHDYNAMO_DISABLE", "1")
    os.makedirs(args.out, exist_ok=True)
    import triton
    rep = {"torch": torch.__version__, "triton": triton.__version__, "gpu": torch.cuda.get_device_name(0),
           "capability": list(torch.cuda.get_device_capability(0)), "parts": {}}
    parts = list(PARTS) + ([("time_cfg2", part_time_cfg2)] if args.time_cfg2 else [])
    for name, fn in parts:
        if args.only and name not in args.only.split(","):
            continue
        t0 = time.time()
        try:
            fn(args.out, rep)
            rep["parts"][name] = {"ok": True, "seconds": round(time.time() - t0, 2)}
        except Exception as e:
            rep["parts"][name] = {"ok": False, "error": type(e).__name__, "trace_tail": traceback.format_exc()[-700:]}
        print(name, rep["parts"][name].get("ok"), flush=True)
        with open(os.path.join(args.out, "gpu_report.json"), "w") as fh:
            json.dump(rep, fh, indent=1)
    print(json.dumps({k: v.get("ok") for k, v in rep["parts"].items()}))


if __name__ == "__main__":
    main()
