"""CPU-side checks of the boundary: the library builds and loads without a GPU, exports every
symbol include/elmo_xmc.h declares, validates arguments, and the product path refuses to run
without a CUDA device instead of falling back to anything."""
import ctypes as C
from types import SimpleNamespace as NS

import pytest
import torch

from elmo_b200 import _lib


def test_library_exports_every_declared_symbol():
    lib = _lib.load()
    declared = _lib.declared_symbols()
    assert {"xmc_create", "xmc_destroy", "xmc_bind_weights", "xmc_bind_kahan", "xmc_step", "xmc_forward_logits",
            "xmc_forward_topk", "xmc_check", "xmc_large_k_matmul_noalloc", "xmc_test_gemm"} <= set(declared)
    for name in declared:
        assert hasattr(lib, name), name
        assert name in _lib._SIGNATURES, f"{name} is declared but has no ctypes signature"
    assert lib.xmc_version().startswith(b"elmo_xmc sm_100a")


def test_argument_validation_needs_no_gpu():
    lib = _lib.load()
    h = C.c_void_p()
    for cfg, msg in [(_lib.XmcConfig(0, 100, 64, 1, 0, 0, 1.0, 0), b"multiple of 64"),
                     (_lib.XmcConfig(0, 768, 0, 1, 0, 0, 1.0, 0), b"max_batch"),
                     (_lib.XmcConfig(0, 768, 64, 9, 0, 0, 1.0, 0), b"mode"),
                     (_lib.XmcConfig(0, 768, 64, 1, 0, 100, 1.0, 0), b"sched_labels"),
                     (_lib.XmcConfig(0, 768, 64, 1, 0, 0, 0.0, 0), b"w_scale")]:
        assert lib.xmc_create(C.byref(cfg), C.byref(h)) == 1
        assert msg in lib.xmc_last_error()
    assert lib.xmc_large_k_matmul_noalloc(0, None, None, 0, 1, 64, 64, None, None) == 1
    assert lib.xmc_step(None, None, 0, 1, None, 0, 0.1, 0.0, 0, 0, 0, None, None, None, None) == 1


@pytest.mark.skipif(torch.cuda.is_available(), reason="checks the no-GPU behaviour")
def test_no_cpu_fallback():
    lib = _lib.load()
    h = C.c_void_p()
    cfg = _lib.XmcConfig(0, 768, 64, 1, 0, 0, 1.0, 0)
    assert lib.xmc_create(C.byref(cfg), C.byref(h)) == 2            # XMC_ERR_CUDA, loudly
    assert lib.xmc_last_error() != b""
    from elmo_b200.xmc_classifiers import Fp8XMCBCEChunkedLayer, XMCBCECHUNKEDLayer
    cfg = NS(environment=NS(device="cpu"),
             model=NS(xmc=NS(dtype="bfloat16", num_chunks=2, input_features=64)),
             training=NS(precision=NS(mode="mixed", purelp_dtype="bfloat16"),
                         xmc=NS(momentum=0, wd=0.0, simulated_fp8=False)),
             data=NS(num_labels=256, batch_size=16))
    for cls in (Fp8XMCBCEChunkedLayer, XMCBCECHUNKEDLayer):
        with pytest.raises(RuntimeError, match="CUDA"):
            cls(cfg)
    cfg.model.xmc.dtype = "float32"                                # the torch-statement path refuses a CPU device too
    with pytest.raises(RuntimeError, match="CUDA"):
        XMCBCECHUNKEDLayer(cfg)
    cfg.model.xmc.dtype = "float8"
    with pytest.raises(NotImplementedError):
        XMCBCECHUNKEDLayer(cfg)


def test_padding_and_shard_geometry_match_reference_formula():
    from elmo_b200.sharded import shard_bounds
    L, nc = 670091, 11
    padded = L + 16 * nc - L % (16 * nc)                          # chunked_fp8xmc_clf.py:26
    assert (padded, padded // nc) == (670208, 60928)
    b = shard_bounds(padded, 8)
    assert sum(hi - lo for lo, hi in b) == padded
