"""Python face of one library handle: owns the C handle, passes raw device pointers and the
current CUDA stream.  torch is used for memory and streams only."""
import ctypes as C
from typing import List, Optional, Sequence

import torch

from . import _lib

_MODE_NAMES = {"bf16": _lib.MODE_BF16, "fp8": _lib.MODE_FP8, "simfp8": _lib.MODE_SIMFP8}


def _ptr(t: Optional[torch.Tensor]):
    return C.c_void_p(0 if t is None else t.data_ptr())


class XmcHandle:
    """One contiguous range of label rows on one GPU (the whole layer, or one label shard)."""

    def __init__(self, device: torch.device, dim: int, max_batch: int, mode: str, *,
                 label_offset: int = 0, sched_labels: int = 0, w_scale: float = 1.0):
        device = torch.device(device)
        if device.type != "cuda":
            raise RuntimeError("elmo_b200 runs on CUDA devices (sm_100a) only; got device %s" % device)
        self.lib = _lib.load()
        self.device = device
        self.index = device.index if device.index is not None else torch.cuda.current_device()
        self.dim, self.max_batch, self.mode = dim, max_batch, mode
        self.label_offset = int(label_offset)
        self.w_scale = float(w_scale)
        torch.cuda.init()
        with torch.cuda.device(self.index):
            torch.zeros(1, device=device)            # make sure the primary context exists
        cfg = _lib.XmcConfig(self.index, dim, max_batch, _MODE_NAMES[mode], self.label_offset,
                             int(sched_labels), self.w_scale, 0)
        h = C.c_void_p()
        _lib.check(self.lib.xmc_create(C.byref(cfg), C.byref(h)))
        self._h = h
        self._bound: List[int] = []
        self._keep: List[torch.Tensor] = []
        self.total_rows = 0

    def close(self):
        if getattr(self, "_h", None) is not None and self._h.value:
            self.lib.xmc_destroy(self._h)
            self._h = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def _stream(self):
        return C.c_void_p(torch.cuda.current_stream(self.index).cuda_stream)

    @property
    def workspace_bytes(self) -> int:
        return int(self.lib.xmc_workspace_bytes(self._h))

    def bind(self, weights: Sequence[torch.Tensor]):
        """Borrow the weight chunks (row-major [rows_i, dim]); re-binds only when storage moved."""
        ptrs = [int(w.data_ptr()) for w in weights]
        if ptrs == self._bound:
            return
        want = torch.bfloat16 if self.mode == "bf16" else torch.float8_e4m3fn
        for w in weights:
            if w.dtype != want or w.dim() != 2 or w.shape[1] != self.dim or not w.is_contiguous() \
                    or w.device.type != "cuda":
                raise ValueError(f"weight chunk must be a contiguous CUDA {want} [rows, {self.dim}] tensor, "
                                 f"got {w.dtype} {tuple(w.shape)} on {w.device}")
        n = len(weights)
        arr_p = (C.c_void_p * n)(*ptrs)
        arr_r = (C.c_int64 * n)(*[int(w.shape[0]) for w in weights])
        _lib.check(self.lib.xmc_bind_weights(self._h, n, arr_p, arr_r))
        self._bound = ptrs
        self._keep = list(weights)
        self.total_rows = sum(int(w.shape[0]) for w in weights)

    def bind_kahan(self, buf: Optional[torch.Tensor]):
        """Attach (or with None detach) the compensation buffer of the Kahan head rows."""
        if buf is None:
            _lib.check(self.lib.xmc_bind_kahan(self._h, C.c_void_p(0), 0, _lib.DT_BF16))
            self._kahan = None
            return
        assert buf.is_cuda and buf.is_contiguous() and buf.dim() == 2 and buf.shape[1] == self.dim
        dt = {torch.bfloat16: _lib.DT_BF16, torch.float8_e5m2: _lib.DT_E5M2}[buf.dtype]
        _lib.check(self.lib.xmc_bind_kahan(self._h, _ptr(buf), int(buf.shape[0]), dt))
        self._kahan = buf

    def step(self, x: torch.Tensor, labels: Optional[torch.Tensor], lr: float, *, wd: float = 0.0,
             seed: int = 0, step: int = 0, stochastic: bool = True, compute_loss: bool = False,
             round_dw_bf16: bool = False, fp8_dw: bool = False, grad_f32: Optional[torch.Tensor] = None,
             grad_bf16: Optional[torch.Tensor] = None, loss_out: Optional[torch.Tensor] = None):
        assert x.dtype == torch.bfloat16 and x.is_contiguous() and x.is_cuda and x.shape[1] == self.dim
        nnz = 0
        if labels is not None and labels.numel() > 0:
            assert labels.dtype == torch.int32 and labels.is_contiguous() and labels.shape[1] == 2
            nnz = labels.shape[0]
        flags = (_lib.STEP_COMPUTE_LOSS if compute_loss else 0) | (_lib.STEP_STOCHASTIC if stochastic else 0) \
            | (_lib.STEP_ROUND_DW_BF16 if round_dw_bf16 else 0) | (_lib.STEP_FP8_DW if fp8_dw else 0)
        batch = x.shape[0]
        for g, dt in ((grad_f32, torch.float32), (grad_bf16, torch.bfloat16)):
            if g is not None:
                assert g.dtype == dt and g.is_contiguous() and g.shape[0] >= batch and g.shape[1] == self.dim
        if compute_loss:
            assert loss_out is not None and loss_out.dtype == torch.float64
        _lib.check(self.lib.xmc_step(self._h, _ptr(x), _lib.DT_BF16, batch,
                                     _ptr(labels if nnz else None), nnz, float(lr), float(wd),
                                     int(seed) & (2 ** 64 - 1), int(step) & (2 ** 64 - 1), flags,
                                     _ptr(grad_f32), _ptr(grad_bf16), _ptr(loss_out), self._stream()))

    def forward_logits(self, x: torch.Tensor, out: torch.Tensor, n_out: int):
        dt = _lib.DT_E4M3 if x.dtype == torch.float8_e4m3fn else _lib.DT_BF16
        assert x.is_contiguous() and out.dtype == torch.bfloat16 and out.stride(1) == 1
        _lib.check(self.lib.xmc_forward_logits(self._h, _ptr(x), dt, x.shape[0], _ptr(out),
                                               out.stride(0), int(n_out), self._stream()))

    def forward_topk(self, x: torch.Tensor, k: int, n_out: int):
        dt = _lib.DT_E4M3 if x.dtype == torch.float8_e4m3fn else _lib.DT_BF16
        vals = torch.empty(x.shape[0], k, dtype=torch.float32, device=x.device)
        idx = torch.empty(x.shape[0], k, dtype=torch.int32, device=x.device)
        _lib.check(self.lib.xmc_forward_topk(self._h, _ptr(x), dt, x.shape[0], k, int(n_out),
                                             _ptr(vals), _ptr(idx), self._stream()))
        return vals, idx

    @property
    def launch_count(self) -> int:
        return int(self.lib.xmc_launch_count(self._h))

    KINDS = ("prep", "unused1", "forward", "grad_x", "update", "reduce", "logits", "unused7")

    def profile(self, enable: bool, read: bool = False):
        """Switch per-kernel-class event timing on/off; with ``read`` return
        {class: (ms, launches)} accumulated since the last call."""
        if read:
            ms = (C.c_double * 8)()
            cnt = (C.c_int64 * 8)()
            _lib.check(self.lib.xmc_profile(self._h, int(enable), ms, cnt))
            return {k: (ms[i], cnt[i]) for i, k in enumerate(self.KINDS) if cnt[i]}
        _lib.check(self.lib.xmc_profile(self._h, int(enable), None, None))
        return None

    def weight_stats(self):
        """One pass over the stored e4m3 weights (synchronises): dict of counts and fractions."""
        counts = (C.c_int64 * 5)()
        amax = C.c_float()
        _lib.check(self.lib.xmc_weight_stats(self._h, counts, C.byref(amax), self._stream()))
        n = max(int(counts[4]), 1)
        return {"zeros": int(counts[0]), "subnormal": int(counts[1]), "saturated": int(counts[2]),
                "nan": int(counts[3]), "elements": int(counts[4]), "amax_stored": float(amax.value),
                "frac_zero": counts[0] / n, "frac_subnormal": counts[1] / n, "frac_saturated": counts[2] / n,
                "scale": self.w_scale}

    def rescale(self, shift: int, *, stochastic: bool = True, seed: int = 0, step: int = 0):
        """scale <- scale * 2^shift, stored <- round(stored * 2^-shift) (real values unchanged)."""
        _lib.check(self.lib.xmc_rescale(self._h, int(shift), int(stochastic), int(seed) & (2 ** 64 - 1),
                                        int(step) & (2 ** 64 - 1), self._stream()))
        self.w_scale = float(self.lib.xmc_get_scale(self._h))

    def set_scale(self, scale: float):
        """Declare the scale the stored weights are expressed in (checkpoint restore); rewrites nothing."""
        _lib.check(self.lib.xmc_set_scale(self._h, float(scale)))
        self.w_scale = float(scale)

    def check(self):
        """Synchronise the current stream and raise if a kernel flagged an error."""
        _lib.check(self.lib.xmc_check(self._h, self._stream()))


def test_gemm(a: torch.Tensor, b: torch.Tensor, layout: int) -> torch.Tensor:
    """D = A B^T on the library's tensor-core engine (self-test hook of the C ABI)."""
    lib = _lib.load()
    if (layout & 1) == 0:
        (m, k), (n, _) = a.shape, b.shape
    else:
        (k, m), (_, n) = a.shape, b.shape
    d = torch.empty(m, n, dtype=torch.float32, device=a.device)
    dt = _lib.DT_E4M3 if a.dtype == torch.float8_e4m3fn else _lib.DT_BF16
    idx = a.device.index if a.device.index is not None else torch.cuda.current_device()
    _lib.check(lib.xmc_test_gemm(idx, layout, dt, m, n, k, _ptr(a), _ptr(b), _ptr(d),
                                 C.c_void_p(torch.cuda.current_stream(idx).cuda_stream)))
    return d
