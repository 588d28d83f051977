"""Counterpart of the reference's src/xmc_classifiers/chunked_fp8xmc_clf.py
(Fp8XMCBCEChunkedLayer): e4m3 weight chunks in a ``ParameterList``, forward in FP8
(``simulated_fp8``: bf16), backward contractions in bf16, SGD fused into the dW contraction.

Same constructor ``(cfg)``, padding rule, attributes and methods as the reference.  New optional
config keys (defaults reproduce the reference): ``training.xmc.rounding`` ('sr' | 'rn'),
``training.xmc.w_scale`` (per-tensor scale, stored = real / w_scale; a number, or 'auto' to derive it
from the initialisation bound), ``training.xmc.scale_interval`` (steps between checks of the scale
keeper, 0 = the scale never changes), ``training.xmc.fp8_dw`` (FP8 operands in the dW contraction; faster,
not the reference's arithmetic), ``model.xmc.sched_labels``.
"""
import math

import torch
from torch import nn

from ..handle import XmcHandle
from ..scale import ScaleKeeper, initial_scale
from ._common import as_labels, cfg_get, draw_base_seed


class Fp8XMCBCEChunkedLayer(nn.Module):
    def __init__(self, cfg):
        super().__init__()
        self.cfg = cfg
        self.device = torch.device(cfg.environment.device)
        self._dtype = torch.float8_e4m3fn
        self.fake_fp8_matmul = cfg.training.xmc.simulated_fp8
        self.num_chunks = cfg.model.xmc.num_chunks
        # chunked_fp8xmc_clf.py:26-28: pad so that every chunk has a multiple of 16 rows
        self.num_labels = cfg.data.num_labels + 16 * self.num_chunks - cfg.data.num_labels % (16 * self.num_chunks)
        self.num_labels_i = self.num_labels // self.num_chunks
        assert self.num_labels_i % 16 == 0
        d = cfg.model.xmc.input_features
        self.input_features = d
        w_scale = cfg_get(cfg, 'training.xmc.w_scale', 1.0)
        if w_scale == 'auto':                 # Xavier-uniform bound sqrt(6 / (fan_in + fan_out))
            w_scale = initial_scale((6.0 / (d + self.num_labels)) ** 0.5)
        self.w_scale = float(w_scale)
        self.scale_keeper = ScaleKeeper(int(cfg_get(cfg, 'training.xmc.scale_interval', 0)))
        xfc_weight = torch.empty(self.num_labels, d, dtype=torch.float32)
        nn.init.xavier_uniform_(xfc_weight)                                            # :29-30
        if self.w_scale != 1.0:
            xfc_weight /= self.w_scale
        self.xfc_weight = nn.ParameterList([
            nn.Parameter(xfc_weight[i * self.num_labels_i:(i + 1) * self.num_labels_i]
                         .to(torch.float8_e4m3fn).to(self.device), requires_grad=False)
            for i in range(self.num_chunks)])
        self.block_size = 16
        self.loss = torch.tensor(0.0, device=self.device)
        self._loss_dev = torch.zeros(1, dtype=torch.float64, device=self.device)
        # inference batches may be larger than training batches (src/config.py keeps the two apart)
        self.max_batch = max(int(cfg.data.batch_size), int(cfg_get(cfg, 'data.test_batch_size', 0) or 0))
        self._grad_buf = torch.zeros(cfg.data.batch_size, d, dtype=torch.bfloat16, device=self.device)
        self.grad_input = self._grad_buf
        self.iteration = 0
        self.rounding = cfg_get(cfg, 'training.xmc.rounding', 'sr')
        # optional, off by default, not the reference's arithmetic: FP8 operands in the dW contraction
        self.fp8_dw = bool(cfg_get(cfg, 'training.xmc.fp8_dw', False))
        self.base_seed = draw_base_seed()
        self._handle = XmcHandle(self.device, d, self.max_batch,
                                 'simfp8' if self.fake_fp8_matmul else 'fp8',
                                 label_offset=cfg_get(cfg, 'model.xmc.label_offset', 0),
                                 sched_labels=cfg_get(cfg, 'model.xmc.sched_labels', 0),
                                 w_scale=self.w_scale)

    def _weights(self):
        return [p.data for p in self.xfc_weight]

    @torch.no_grad()
    def xfc_forward(self, embed):
        """Logits [B, cfg.data.num_labels] bf16, padding rows hidden (:45-60).  ``embed`` may be
        bf16 or already cast to e4m3 (the evaluator does that: src/evaluate.py:155-156)."""
        self._handle.bind(self._weights())
        n = self.cfg.data.num_labels
        x = embed if embed.dtype in (torch.bfloat16, torch.float8_e4m3fn) else embed.to(torch.bfloat16)
        out = torch.empty(x.shape[0], (n + 7) // 8 * 8, dtype=torch.bfloat16, device=x.device)
        self._handle.forward_logits(x.contiguous(), out, n)
        return out[:, :n]

    @torch.no_grad()
    def xfc_topk(self, embed, k):
        """Fused ``xfc_forward`` + ``torch.topk`` (src/evaluate.py:158-159) without the logits."""
        self._handle.bind(self._weights())
        x = embed if embed.dtype in (torch.bfloat16, torch.float8_e4m3fn) else embed.to(torch.bfloat16)
        return self._handle.forward_topk(x.contiguous(), k, self.cfg.data.num_labels)

    @torch.no_grad()
    def xfc_forward_backward(self, embed, labels, xmc_lr, skip_loss=True):
        """One train step (:81-123).  The reference never computes the loss here (``skip_loss`` is
        ignored and 0 returned); this class returns the summed BCE loss when ``skip_loss=False``."""
        bsz = embed.shape[0]
        if embed.dtype != torch.bfloat16:
            embed = embed.to(torch.bfloat16)
        self._handle.bind(self._weights())
        self._handle.step(embed.contiguous(), as_labels(labels, embed.device), xmc_lr[0],
                          seed=self.base_seed, step=self.iteration,
                          stochastic=(self.rounding == 'sr'), compute_loss=not skip_loss, fp8_dw=self.fp8_dw,
                          grad_bf16=self._grad_buf, loss_out=self._loss_dev)
        self.iteration += 1
        self.grad_input = self._grad_buf[:bsz]
        if self.scale_keeper.interval > 0 and self.scale_keeper.maybe_update(self._handle, self.iteration, self.base_seed):
            self.w_scale = self._handle.w_scale
        return 0 if skip_loss else float(self._loss_dev.item())

    # --- checkpoint: the weights travel in state_dict as in the reference (runner.py:242-251); what the
    # reference has no slot for (scale, stochastic-rounding stream position) rides along as extra state
    def get_extra_state(self):
        return {"w_scale": self.w_scale, "base_seed": self.base_seed, "iteration": self.iteration,
                "rounding": self.rounding}

    def set_extra_state(self, state):
        if not state:
            return
        saved = float(state.get("w_scale", self.w_scale))
        if saved != self.w_scale:
            # the stored weights of the checkpoint belong to ITS scale (the keeper may have moved it):
            # adopt it, which is exact because scales are powers of two apart
            ratio = saved / self.w_scale
            shift = round(math.log2(ratio)) if ratio > 0 else None
            if shift is None or 2.0 ** shift != ratio:
                raise ValueError(f"checkpoint was written with w_scale={saved}, layer has {self.w_scale}")
            self._handle.bind(self._weights())
            self._handle.set_scale(saved)
            self.w_scale = saved
        self.base_seed = int(state.get("base_seed", self.base_seed))
        self.iteration = int(state.get("iteration", self.iteration))
        self.rounding = state.get("rounding", self.rounding)
