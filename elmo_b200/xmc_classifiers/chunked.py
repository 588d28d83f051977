"""Counterpart of the reference's src/xmc_classifiers/chunked.py (XMCBCECHUNKEDLayer).

Same constructor ``(cfg)``, attributes (``xfc_weight``, ``grad_input``, ``_dtype``, ``iteration``,
``num_chunks``, ``chunk_size``) and methods (``xfc_forward``, ``xfc_forward_backward``).  The dense
weight tensor lives in torch memory and is borrowed by the CUDA library; forward, loss gradient,
grad_X and the SGD update run there for bfloat16 weights, the precision the chunked layer is trained
in.  float32 / float16 weights -- in the reference a handful of plain torch (cuBLAS) calls with an
un-fused SGD step, chunked.py:96-124 -- take the same torch statements here, on the layer's device:
they are a library path kept for interface completeness, not one of this package's kernels.
"""
import torch
from torch import nn

from ..handle import XmcHandle
from ._common import as_labels, cfg_get, draw_base_seed, dtype_map


class XMCBCECHUNKEDLayer(nn.Module):
    def __init__(self, cfg):
        super().__init__()
        self.cfg = cfg
        self.device = torch.device(cfg.environment.device)
        self._dtype = dtype_map[cfg.model.xmc.dtype]                                   # chunked.py:20-23
        self._dtype = torch.float32 if cfg.training.precision.mode in ['purefp'] else self._dtype
        self._dtype = dtype_map[cfg.training.precision.purelp_dtype] \
            if cfg.training.precision.mode in ['purelp'] else self._dtype
        if self._dtype not in (torch.bfloat16, torch.float32, torch.float16):
            raise NotImplementedError(f"XMCBCECHUNKEDLayer: unsupported weight dtype {self._dtype}")
        self._native = self._dtype == torch.bfloat16       # the CUDA library's path
        if not self._native and self.device.type != "cuda":
            raise RuntimeError("elmo_b200 runs on CUDA devices only; got device %s" % self.device)
        self.num_labels = cfg.data.num_labels
        self.num_chunks = cfg.model.xmc.num_chunks
        self.chunk_size = (self.num_labels + self.num_chunks - 1) // self.num_chunks   # chunked.py:30
        d = cfg.model.xmc.input_features
        self.input_features = d
        self.xfc_weight = torch.empty(self.num_labels, d, dtype=self._dtype).to(self.device)
        nn.init.normal_(self.xfc_weight, mean=0.0, std=0.02)                           # chunked.py:34
        self._grad_buf = torch.zeros(cfg.data.batch_size, d, dtype=self._dtype, device=self.device)
        self.grad_input = self._grad_buf
        self.loss = torch.tensor(0.0, device=self.device)
        self._loss_dev = torch.zeros(1, dtype=torch.float64, device=self.device)
        self.iteration = 0
        # the reference's bf16 path always rounds stochastically (stochastic_rounding_kernel.py:82-89)
        self.rounding = cfg_get(cfg, 'training.xmc.rounding', 'sr')
        self.base_seed = draw_base_seed()
        self.max_batch = max(int(cfg.data.batch_size), int(cfg_get(cfg, 'data.test_batch_size', 0) or 0))
        self._handle = XmcHandle(self.device, d, self.max_batch, 'bf16',
                                 label_offset=cfg_get(cfg, 'model.xmc.label_offset', 0),
                                 sched_labels=cfg_get(cfg, 'model.xmc.sched_labels', 0)) if self._native else None

    # ``xfc_weight`` is a plain attribute as in the reference (saved separately by runner.py:246); the
    # stochastic-rounding stream position rides along in state_dict as extra state
    def get_extra_state(self):
        return {"base_seed": self.base_seed, "iteration": self.iteration, "rounding": self.rounding}

    def set_extra_state(self, state):
        if state:
            self.base_seed = int(state.get("base_seed", self.base_seed))
            self.iteration = int(state.get("iteration", self.iteration))
            self.rounding = state.get("rounding", self.rounding)

    @torch.no_grad()
    def xfc_forward(self, embed):
        """Logits [B, num_labels] (chunked.py:48-53)."""
        if not self._native:
            return torch.matmul(embed.to(self._dtype), self.xfc_weight.t())
        self._handle.bind([self.xfc_weight])
        x = embed if embed.dtype in (torch.bfloat16, torch.float8_e4m3fn) else embed.to(torch.bfloat16)
        out = torch.empty(x.shape[0], (self.num_labels + 7) // 8 * 8, dtype=torch.bfloat16, device=x.device)
        self._handle.forward_logits(x.contiguous(), out, self.num_labels)
        return out[:, :self.num_labels]

    @torch.no_grad()
    def xfc_forward_backward(self, embed, labels, xmc_lr, skip_loss=True):
        """One train step of the layer (chunked.py:75-133): updates ``xfc_weight`` in place, leaves
        the activation gradient in ``grad_input`` and returns the summed BCE loss (0 when skipped).

        The bf16 reference materialises dW in bf16 (chunked.py:119) and applies no weight decay
        (stochastic_rounding_kernel.py:91-99 ignores it); both are reproduced.
        """
        bsz = embed.shape[0]
        if embed.dtype != self._dtype:
            embed = embed.to(self._dtype)
        if not self._native:
            return self._step_torch(embed, as_labels(labels, embed.device), xmc_lr[0], skip_loss)
        self._handle.bind([self.xfc_weight])
        self._handle.step(embed.contiguous(), as_labels(labels, embed.device), xmc_lr[0],
                          wd=0.0, seed=self.base_seed, step=self.iteration,
                          stochastic=(self.rounding == 'sr'), compute_loss=not skip_loss,
                          round_dw_bf16=True, grad_bf16=self._grad_buf, loss_out=self._loss_dev)
        self.grad_input = self._grad_buf[:bsz]
        self.iteration += 1
        return 0 if skip_loss else float(self._loss_dev.item())

    def _step_torch(self, embed, labels, lr, skip_loss):
        """float32 / float16 weights: the reference's own statements (chunked.py:96-124) -- per chunk
        ``Z = X W_c^T``; ``G = sigmoid(Z) - Y``; ``grad_X += G W_c``; ``dW = G^T X + wd W_c``;
        ``W_c -= lr dW`` -- with the loss taken from the logits (the reference passes the weights to
        ``_compute_loss`` by mistake, chunked.py:109)."""
        rows, cols = labels[:, 0].long(), labels[:, 1].long()
        grad = torch.zeros(embed.shape[0], self.input_features, dtype=torch.float32, device=embed.device)
        loss = 0.0
        wd = float(cfg_get(self.cfg, 'training.xmc.wd', 0.0))
        for c in range(self.num_chunks):
            s0, e0 = c * self.chunk_size, min((c + 1) * self.chunk_size, self.num_labels)
            if s0 >= e0:
                continue
            w = self.xfc_weight[s0:e0]
            z = torch.matmul(embed, w.t())                                              # :101
            m = (cols >= s0) & (cols < e0)
            r, cc = rows[m], cols[m] - s0
            if not skip_loss:
                zf = z.float()
                loss += float(zf.clamp(min=0).sum() + torch.log1p(torch.exp(-zf.abs())).sum())     # :57-72
                y = torch.zeros_like(zf, dtype=torch.bool)
                y[r, cc] = True
                loss -= float(zf[y].sum())
            torch.sigmoid(z, out=z)                                                     # :112
            z[r, cc] -= 1.0                                                             # :113 (set semantics)
            grad += torch.matmul(z, w)                                                  # :116
            dw = z.t().mm(embed)                                                        # :119
            dw.add_(w, alpha=wd)                                                        # :123
            w.add_(dw, alpha=-lr)                                                       # :124
        self.grad_input = grad.to(self._dtype)
        self.iteration += 1
        return 0 if skip_loss else loss
