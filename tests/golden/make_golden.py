"""Generate tests/golden/*.npz by running the UNMODIFIED reference on CPU.

Run in a container that has the reference checked out:

    TORCHDYNAMO_DISABLE=1 python tests/golden/make_golden.py /path/to/reference

The fixtures hold inputs and the reference's outputs for the parts of the hot path that
execute without a GPU:
  chunked_fp32.npz   XMCBCECHUNKEDLayer, float32, end to end (chunked.py:75-133)
  chunked_bf16.npz   same in bfloat16; the Triton launcher ``sgd_update`` (GPU only) is replaced
                     by ``W <- bf16_rn(float(W) - float(dW)*lr)``, everything else is reference code
  fp8_forward.npz    Fp8XMCBCEChunkedLayer.xfc_forward, real (torch._scaled_mm) and simulated
  loss.npz           XMCBCECHUNKEDLayer._compute_loss on given logits
bf16 tensors are stored as their uint16 bit patterns, e4m3 tensors as uint8.
"""
import os
import sys
from types import SimpleNamespace as NS

import numpy as np
import torch

os.environ.setdefault("TORCHDYNAMO_DISABLE", "1")
if len(sys.argv) < 2:
    sys.exit("usage: make_golden.py /path/to/reference")
ref_root = sys.argv[1]
sys.path.insert(0, os.path.join(ref_root, "src"))
here = os.path.dirname(os.path.abspath(__file__))

import xmc_classifiers.chunked as ref_chunked                      # noqa: E402
from xmc_classifiers.chunked_fp8xmc_clf import Fp8XMCBCEChunkedLayer  # noqa: E402


def bits(t):
    if t.dtype == torch.bfloat16:
        return t.view(torch.uint16).numpy()
    if t.dtype == torch.float8_e4m3fn:
        return t.view(torch.uint8).numpy()
    return t.numpy()


def cfg(L, d, B, nc, dtype, sim=False):
    return NS(environment=NS(device="cpu"),
              model=NS(xmc=NS(dtype=dtype, num_chunks=nc, input_features=d)),
              training=NS(precision=NS(mode="mixed", purelp_dtype="bfloat16"),
                          xmc=NS(momentum=0, wd=0.0, simulated_fp8=sim)),
              data=NS(num_labels=L, batch_size=B))


def make_labels(g, B, L, per_row):
    rows, cols = [], []
    for r in range(B):
        n = int(torch.randint(1, per_row + 1, (1,), generator=g))
        c = torch.randint(0, L, (n,), generator=g)
        # head-heavy ids + a duplicated pair now and then (index_put set semantics)
        c = torch.where(torch.rand(n, generator=g) < 0.3, c % 7, c)
        rows += [r] * n
        cols += c.tolist()
        if r % 5 == 0:
            rows.append(r); cols.append(cols[-1])
    return torch.tensor(list(zip(rows, cols)), dtype=torch.int32)


def run_chunked(dtype_name, fname, L=520, d=64, B=24, nc=3, lr=0.05, steps=2):
    g = torch.Generator().manual_seed(1234)
    layer = ref_chunked.XMCBCECHUNKEDLayer(cfg(L, d, B, nc, dtype_name))
    w0 = (torch.rand(L, d, generator=g) * 2 - 1) / d ** 0.5
    layer.xfc_weight = w0.to(layer._dtype)
    out = {"L": L, "d": d, "B": B, "nc": nc, "lr": lr, "w0": bits(layer.xfc_weight.clone())}
    if dtype_name == "bfloat16":
        def sgd_rn(weights, gradient, compensation, learning_rate, weight_decay, sr, seed):
            weights.copy_((weights.float() - gradient.float() * learning_rate).to(weights.dtype))
        ref_chunked.sgd_update = sgd_rn
    for s in range(steps):
        x = (torch.randn(B, d, generator=g) / d ** 0.5).to(layer._dtype)
        lab = make_labels(g, B, L, 6)
        layer.xfc_forward_backward(x, lab, [lr], skip_loss=True)
        out[f"x{s}"] = bits(x); out[f"labels{s}"] = lab.numpy()
        out[f"w{s + 1}"] = bits(layer.xfc_weight.clone())
        out[f"grad_input{s}"] = bits(layer.grad_input.clone())
    out["logits_last"] = bits(layer.xfc_forward(x))
    np.savez_compressed(os.path.join(here, fname), **out)


def run_fp8_forward(fname, L=500, d=64, B=32, nc=3):
    g = torch.Generator().manual_seed(99)
    res = {"L": L, "d": d, "B": B, "nc": nc}
    for sim in (False, True):
        torch.manual_seed(7)
        layer = Fp8XMCBCEChunkedLayer(cfg(L, d, B, nc, "float8", sim))
        # spread the weights over the e4m3 range (Xavier at scale 1 lands on 3 values only)
        for i in range(nc):
            w = torch.randn(layer.num_labels_i, d, generator=g) * 0.25
            layer.xfc_weight[i].data = w.to(torch.float8_e4m3fn)
        x = (torch.randn(B, d, generator=g) / d ** 0.5).to(torch.bfloat16)
        tag = "sim" if sim else "real"
        res[f"{tag}_x"] = bits(x)
        for i in range(nc):
            res[f"{tag}_w{i}"] = bits(layer.xfc_weight[i].data)
        res[f"{tag}_logits"] = bits(layer.xfc_forward(x))
        # the evaluator hands in e4m3-cast embeds (evaluate.py:155-156)
        res[f"{tag}_logits_e4m3_embed"] = bits(layer.xfc_forward(x.to(torch.float8_e4m3fn)))
        res["L_padded"] = layer.num_labels
        res["L_i"] = layer.num_labels_i
    np.savez_compressed(os.path.join(here, fname), **res)


def run_loss(fname):
    g = torch.Generator().manual_seed(5)
    layer = ref_chunked.XMCBCECHUNKEDLayer(cfg(64, 16, 8, 1, "float32"))
    z = torch.randn(8, 64, generator=g) * 3
    rows = torch.tensor([0, 1, 1, 5, 7]); cols = torch.tensor([3, 0, 63, 17, 9])
    loss = layer._compute_loss(z, rows, cols)
    np.savez_compressed(os.path.join(here, fname), z=z.numpy(), rows=rows.numpy(),
                        cols=cols.numpy(), loss=np.float64(loss))


if __name__ == "__main__":
    torch.set_num_threads(1)
    run_chunked("float32", "chunked_fp32.npz")
    run_chunked("bfloat16", "chunked_bf16.npz")
    run_fp8_forward("fp8_forward.npz")
    run_loss("loss.npz")
    print("golden fixtures written to", here)
