"""Drop-in counterparts of the reference's ``src/xmc_classifiers`` modules.

Selection mirrors src/model.py:144-156:
    chunked             -> chunked.XMCBCECHUNKEDLayer
    fp8chunked          -> chunked_fp8xmc_clf.Fp8XMCBCEChunkedLayer
"""
from .chunked import XMCBCECHUNKEDLayer
from .chunked_fp8xmc_clf import Fp8XMCBCEChunkedLayer

IMPLEMENTATIONS = {"chunked": XMCBCECHUNKEDLayer, "fp8chunked": Fp8XMCBCEChunkedLayer}

__all__ = ["XMCBCECHUNKEDLayer", "Fp8XMCBCEChunkedLayer", "IMPLEMENTATIONS"]
