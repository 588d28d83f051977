"""ctypes binding of the C ABI declared in include/elmo_xmc.h.

The shared library is built in-tree by ``elmo_b200.build``.  There is no fallback: if the
library cannot be built or loaded, importing a layer class fails with the reason.
"""
import ctypes as C
import os
import re

from . import build as _build

XMC_OK = 0
DT_BF16, DT_E4M3, DT_F32, DT_E5M2 = 0, 1, 2, 3
MODE_BF16, MODE_FP8, MODE_SIMFP8 = 0, 1, 2
STEP_COMPUTE_LOSS, STEP_STOCHASTIC, STEP_ROUND_DW_BF16, STEP_FP8_DW = 1, 2, 4, 8


class XmcConfig(C.Structure):
    _fields_ = [("device", C.c_int32), ("dim", C.c_int32), ("max_batch", C.c_int32),
                ("mode", C.c_int32), ("label_offset", C.c_int64), ("sched_labels", C.c_int64),
                ("w_scale", C.c_float), ("reserved", C.c_int32)]


class XmcError(RuntimeError):
    def __init__(self, code, msg):
        super().__init__(f"elmo_xmc error {code}: {msg}")
        self.code = code


_SIGNATURES = {
    "xmc_create": (C.c_int, [C.POINTER(XmcConfig), C.POINTER(C.c_void_p)]),
    "xmc_destroy": (C.c_int, [C.c_void_p]),
    "xmc_bind_weights": (C.c_int, [C.c_void_p, C.c_int32, C.POINTER(C.c_void_p), C.POINTER(C.c_int64)]),
    "xmc_bind_kahan": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int64, C.c_int32]),
    "xmc_step": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int32, C.c_int32, C.c_void_p, C.c_int64,
                           C.c_float, C.c_float, C.c_uint64, C.c_uint64, C.c_uint32,
                           C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p]),
    "xmc_forward_logits": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int32, C.c_int32, C.c_void_p,
                                     C.c_int64, C.c_int64, C.c_void_p]),
    "xmc_forward_topk": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int32, C.c_int32, C.c_int32, C.c_int64,
                                   C.c_void_p, C.c_void_p, C.c_void_p]),
    "xmc_check": (C.c_int, [C.c_void_p, C.c_void_p]),
    "xmc_weight_stats": (C.c_int, [C.c_void_p, C.POINTER(C.c_int64), C.POINTER(C.c_float), C.c_void_p]),
    "xmc_rescale": (C.c_int, [C.c_void_p, C.c_int32, C.c_int32, C.c_uint64, C.c_uint64, C.c_void_p]),
    "xmc_get_scale": (C.c_float, [C.c_void_p]),
    "xmc_set_scale": (C.c_int, [C.c_void_p, C.c_float]),
    "xmc_workspace_bytes": (C.c_int64, [C.c_void_p]),
    "xmc_launch_count": (C.c_int64, [C.c_void_p]),
    "xmc_profile": (C.c_int, [C.c_void_p, C.c_int32, C.POINTER(C.c_double), C.POINTER(C.c_int64)]),
    "xmc_last_error": (C.c_char_p, []),
    "xmc_version": (C.c_char_p, []),
    "xmc_large_k_matmul_noalloc": (C.c_int, [C.c_int32, C.c_void_p, C.c_void_p, C.c_int32, C.c_int32, C.c_int32,
                                             C.c_int32, C.c_void_p, C.c_void_p]),
    "xmc_noalloc_check": (C.c_int, [C.c_int32, C.c_void_p]),
    "xmc_test_sigmoid": (C.c_int, [C.c_int32, C.c_void_p, C.c_void_p, C.c_int32, C.c_void_p]),
    "xmc_test_gemm": (C.c_int, [C.c_int32, C.c_int32, C.c_int32, C.c_int32, C.c_int32, C.c_int32,
                                C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p]),
}

_lib = None


def header_path():
    return os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "include", "elmo_xmc.h")


def declared_symbols():
    """Names of all functions declared in include/elmo_xmc.h."""
    text = open(header_path()).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(xmc_[a-z_0-9]+)\s*\(", text)))


def load():
    """Build (if stale) and load the library; bind argument types. Raises on any failure."""
    global _lib
    if _lib is not None:
        return _lib
    path = _build.build()
    lib = C.CDLL(path)
    for name, (res, args) in _SIGNATURES.items():
        fn = getattr(lib, name)
        fn.restype = res
        fn.argtypes = args
    _lib = lib
    return lib


def check(code):
    if code != XMC_OK:
        raise XmcError(code, load().xmc_last_error().decode())
