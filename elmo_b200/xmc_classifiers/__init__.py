"""Drop-in counterparts of the reference's ``src/xmc_classifiers`` modules.

Selection mirrors src/model.py:144-156:
    chunked             -> chunked.XMCBCECHUNKEDLayer
    fp8chunked          -> chunked_fp8xmc_clf.Fp8XMCBCEChunkedLayer
    fp8chunkedheadkahan -> chunked_head_kahan_fp8xmc_clf.Fp8XMCBCEChunkedHeadKahanLayer
"""
from .chunked import XMCBCECHUNKEDLayer
from .chunked_fp8xmc_clf import Fp8XMCBCEChunkedLayer
from .chunked_head_kahan_fp8xmc_clf import Fp8XMCBCEChunkedHeadKahanLayer

IMPLEMENTATIONS = {"chunked": XMCBCECHUNKEDLayer, "fp8chunked": Fp8XMCBCEChunkedLayer,
                   "fp8chunkedheadkahan": Fp8XMCBCEChunkedHeadKahanLayer}

__all__ = ["XMCBCECHUNKEDLayer", "Fp8XMCBCEChunkedLayer", "Fp8XMCBCEChunkedHeadKahanLayer", "IMPLEMENTATIONS"]
