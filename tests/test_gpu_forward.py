"""xfc_forward (inference logits) of the CUDA classes against the reference's own outputs
(golden fixtures produced by the unmodified reference on CPU) and against the oracle."""
from types import SimpleNamespace as NS

import pytest
import torch

from tests._util import as_bf16, as_e4m3, load_golden, rel_inf

pytestmark = pytest.mark.gpu


def _cfg(L, d, B, nc, sim=False, dtype="bfloat16"):
    return NS(environment=NS(device="cuda:0"),
              model=NS(xmc=NS(dtype=dtype, num_chunks=nc, input_features=d)),
              training=NS(precision=NS(mode="mixed", purelp_dtype="bfloat16"),
                          xmc=NS(momentum=0, wd=0.0, simulated_fp8=sim)),
              data=NS(num_labels=L, batch_size=B))


@pytest.mark.parametrize("tag,sim", [("real", False), ("sim", True)])
def test_fp8_forward_matches_reference_fixture(tag, sim):
    from elmo_b200.xmc_classifiers import Fp8XMCBCEChunkedLayer
    g = load_golden("fp8_forward.npz")
    L, d, B, nc = int(g["L"]), int(g["d"]), int(g["B"]), int(g["nc"])
    layer = Fp8XMCBCEChunkedLayer(_cfg(L, d, B, nc, sim))
    assert layer.num_labels == int(g["L_padded"]) and layer.num_labels_i == int(g["L_i"])
    for i in range(nc):
        layer.xfc_weight[i].data.copy_(as_e4m3(g[f"{tag}_w{i}"]))
    x = as_bf16(g[f"{tag}_x"]).cuda()
    z = layer.xfc_forward(x).cpu()
    ref = as_bf16(g[f"{tag}_logits"])
    assert z.shape == ref.shape == (B, L)
    same = (z.view(torch.int16) == ref.view(torch.int16)).float().mean()
    assert same >= 0.99, same                       # tensor-core vs CPU accumulation order
    assert rel_inf(z, ref) < 1e-2
    # the evaluator hands in e4m3-cast embeds (evaluate.py:155-156)
    z8 = layer.xfc_forward(x.to(torch.float8_e4m3fn)).cpu()
    assert rel_inf(z8, as_bf16(g[f"{tag}_logits_e4m3_embed"])) < 1e-2
    layer._handle.check()


def test_bf16_forward_matches_reference_fixture():
    from elmo_b200.xmc_classifiers import XMCBCECHUNKEDLayer
    g = load_golden("chunked_bf16.npz")
    L, d, B, nc = int(g["L"]), int(g["d"]), int(g["B"]), int(g["nc"])
    layer = XMCBCECHUNKEDLayer(_cfg(L, d, B, nc))
    layer.xfc_weight.copy_(as_bf16(g["w2"]))
    z = layer.xfc_forward(as_bf16(g["x1"]).cuda()).cpu()
    ref = as_bf16(g["logits_last"])
    assert z.shape == ref.shape
    assert rel_inf(z, ref) < 1e-2
    layer._handle.check()


def test_forward_large_odd_shapes_match_oracle():
    from elmo_b200.xmc_classifiers import Fp8XMCBCEChunkedLayer
    from oracle import xmc_oracle as O
    L, d, B, nc = 70001, 256, 200, 3
    layer = Fp8XMCBCEChunkedLayer(_cfg(L, d, B, nc))
    gen = torch.Generator().manual_seed(0)
    ws = []
    for p in layer.xfc_weight:
        w = (torch.randn(p.shape, generator=gen) * 0.25).to(torch.float8_e4m3fn)
        p.data.copy_(w); ws.append(w)
    x = (torch.randn(B - 3, d, generator=gen) / d ** 0.5).to(torch.bfloat16)     # short last batch
    z = layer.xfc_forward(x.cuda()).cpu()
    ref = O.forward_logits(ws, x, num_labels=L)
    assert z.shape == ref.shape == (B - 3, L)
    assert rel_inf(z, ref) < 1e-2
    layer._handle.check()


def test_layer_step_through_class_api_matches_oracle():
    """The runner's call sequence (runner.py:146-157) on the drop-in class."""
    from elmo_b200.xmc_classifiers import Fp8XMCBCEChunkedLayer
    from oracle import xmc_oracle as O
    L, d, B, nc = 3000, 128, 64, 2
    cfg = _cfg(L, d, B, nc)
    cfg.training.xmc.rounding = "rn"
    layer = Fp8XMCBCEChunkedLayer(cfg)
    gen = torch.Generator().manual_seed(3)
    ws = []
    for p in layer.xfc_weight:
        w = (torch.randn(p.shape, generator=gen) * 0.25).to(torch.float8_e4m3fn)
        p.data.copy_(w); ws.append(w)
    for it in range(2):
        x = (torch.randn(B, d, generator=gen) / d ** 0.5).to(torch.bfloat16)
        lab = torch.stack([torch.randint(0, B, (200,), generator=gen),
                           torch.randint(0, L, (200,), generator=gen)], 1).to(torch.int32)
        loss = layer.xfc_forward_backward(x.cuda(), lab.cuda(), [0.5], skip_loss=(it == 0))
        ws, gx, want_loss = O.fp8_chunked_step(ws, x, lab, 0.5, rounding="rn", compute_loss=True)
        assert rel_inf(layer.grad_input.float().cpu(), gx) < 1e-2
        if it == 1:
            assert abs(loss - want_loss) < 1e-3 * abs(want_loss)
        else:
            assert loss == 0
        layer.grad_input[0:B].div_(2)                       # the runner mutates it in place
    for p, w in zip(layer.xfc_weight, ws):
        assert (p.data.cpu().view(torch.uint8) == w.view(torch.uint8)).float().mean() >= 0.999
    assert layer.iteration == 2
    sd = layer.state_dict()
    assert sorted(k for k in sd if k != "_extra_state") == [f"xfc_weight.{i}" for i in range(nc)]
    layer._handle.check()


def test_checkpoint_round_trip_continues_the_same_stochastic_stream():
    """runner.py:242-268: state_dict save / load; a restored layer must take the same next step."""
    import io
    from elmo_b200.xmc_classifiers import Fp8XMCBCEChunkedHeadKahanLayer
    L, d, B, nc = 2000, 128, 32, 2
    cfg = _cfg(L, d, B, nc)
    cfg.training.FP8 = NS(using_head_kahan=True, fp8_head_kahan=False, head_ratio=0.1)
    torch.manual_seed(1)
    a = Fp8XMCBCEChunkedHeadKahanLayer(cfg)
    gen = torch.Generator().manual_seed(5)
    for p in a.xfc_weight:
        p.data.copy_((torch.randn(p.shape, generator=gen) * 0.25).to(torch.float8_e4m3fn))
    x = (torch.randn(B, d, generator=gen) / d ** 0.5).to(torch.bfloat16).cuda()
    lab = torch.stack([torch.randint(0, B, (100,), generator=gen),
                       torch.randint(0, L, (100,), generator=gen)], 1).to(torch.int32).cuda()
    a.xfc_forward_backward(x, lab, [0.5])
    buf = io.BytesIO()
    torch.save(a.state_dict(), buf)
    buf.seek(0)
    torch.manual_seed(999)                                   # a different construction-time seed
    b = Fp8XMCBCEChunkedHeadKahanLayer(cfg)
    b.load_state_dict(torch.load(buf))
    assert b.iteration == 1 and b.base_seed == a.base_seed
    assert torch.equal(b.head_kahan.view(torch.int16), a.head_kahan.view(torch.int16))
    a.xfc_forward_backward(x, lab, [0.5])
    b.xfc_forward_backward(x, lab, [0.5])
    for pa, pb in zip(a.xfc_weight, b.xfc_weight):
        assert torch.equal(pa.data.view(torch.uint8), pb.data.view(torch.uint8))
    assert torch.equal(a.grad_input, b.grad_input)
    a._handle.check(); b._handle.check()


def test_sigmoid_of_every_bf16_input():
    """The epilogue's sigmoid (approximate ex2 + rcp, rounded to bf16) against torch.sigmoid on bf16
    (chunked_fp8xmc_clf.py:107) for all 65 536 bf16 bit patterns."""
    import ctypes as C
    from elmo_b200 import _lib
    lib = _lib.load()
    bits = torch.arange(65536, dtype=torch.int32).to(torch.uint16)
    x = bits.view(torch.bfloat16)
    want = torch.sigmoid(x.float()).to(torch.bfloat16)
    xd = x.cuda()
    out = torch.empty_like(xd)
    _lib.check(lib.xmc_test_sigmoid(0, C.c_void_p(xd.data_ptr()), C.c_void_p(out.data_ptr()), 65536,
                                    C.c_void_p(torch.cuda.current_stream().cuda_stream)))
    got = out.cpu()
    ok = ~torch.isnan(x.float())
    same = (got.view(torch.int16) == want.view(torch.int16))[ok]
    # flush-to-zero of the approximate ops may turn a result below 2^-126 into 0: allow those
    tiny = want.float().abs()[ok] < 2.0 ** -120
    assert bool((same | tiny).all()), int((~(same | tiny)).sum())


@pytest.mark.parametrize("dtype_name", ["float32", "float16"])
def test_chunked_layer_float_weights_match_reference_fixture(dtype_name):
    """float32 / float16 weights of XMCBCECHUNKEDLayer (plain torch statements, as in the reference)
    against the fixture the unmodified reference produced in float32 (tests/golden/chunked_fp32.npz)."""
    from types import SimpleNamespace as NS
    from elmo_b200.xmc_classifiers import XMCBCECHUNKEDLayer
    from tests._util import load_golden, rel_inf
    g = load_golden("chunked_fp32.npz")
    L, d, B, nc, lr = int(g["L"]), int(g["d"]), int(g["B"]), int(g["nc"]), float(g["lr"])
    cfg = NS(environment=NS(device="cuda:0"),
             model=NS(xmc=NS(dtype=dtype_name, num_chunks=nc, input_features=d)),
             training=NS(precision=NS(mode="mixed", purelp_dtype="bfloat16"), xmc=NS(momentum=0, wd=0.0, simulated_fp8=False)),
             data=NS(num_labels=L, batch_size=B))
    layer = XMCBCECHUNKEDLayer(cfg)
    layer.xfc_weight.copy_(torch.from_numpy(g["w0"]).to(layer._dtype))
    tol = 1e-5 if dtype_name == "float32" else 2e-2
    for s in range(2):
        x = torch.from_numpy(g[f"x{s}"]).cuda()
        lab = torch.from_numpy(g[f"labels{s}"]).cuda()
        loss = layer.xfc_forward_backward(x, lab, [lr], skip_loss=(s == 0))
        assert rel_inf(layer.xfc_weight.float().cpu(), torch.from_numpy(g[f"w{s + 1}"])) < tol
        assert rel_inf(layer.grad_input.float().cpu(), torch.from_numpy(g[f"grad_input{s}"])) < max(tol, 1e-4)
    assert loss > 0 and layer.iteration == 2
    z = layer.xfc_forward(torch.from_numpy(g["x1"]).cuda())
    assert rel_inf(z.float().cpu(), torch.from_numpy(g["logits_last"])) < max(tol, 1e-4)
