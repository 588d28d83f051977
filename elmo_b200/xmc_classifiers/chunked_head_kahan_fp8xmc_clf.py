"""Counterpart of the reference's src/xmc_classifiers/chunked_head_kahan_fp8xmc_clf.py
(Fp8XMCBCEChunkedHeadKahanLayer): the FP8 chunked layer whose first ``head_ratio * num_labels`` rows
(the head labels, when the data pipeline sorts labels by frequency) carry a Kahan compensation
buffer in e5m2 or bf16, so that small updates to frequently hit rows are not lost to e4m3 rounding.
"""
import torch

from .chunked_fp8xmc_clf import Fp8XMCBCEChunkedLayer


class Fp8XMCBCEChunkedHeadKahanLayer(Fp8XMCBCEChunkedLayer):
    def __init__(self, cfg):
        super().__init__(cfg)
        self.using_head_kahan = cfg.training.FP8.using_head_kahan
        if not self.using_head_kahan:
            self.head_kahan = None
        if self.using_head_kahan:
            self.fp8_head_kahan = cfg.training.FP8.fp8_head_kahan
            self.num_head = int(cfg.training.FP8.head_ratio * self.num_labels)        # :42
            dt = torch.float8_e5m2 if self.fp8_head_kahan else torch.bfloat16         # :43-46
            # a registered buffer, so that it is checkpointed with the weights (the reference keeps it
            # as a plain attribute and loses it on save/load)
            self.register_buffer("head_kahan", torch.zeros(self.num_head, self.input_features, dtype=dt,
                                                           device=self.device))
            assert self.num_head <= self.num_labels_i                                 # :47
        self._kahan_ptr = None

    @torch.no_grad()
    def xfc_forward_backward(self, embed, labels, xmc_lr, skip_loss=True):
        """As the base class; rows [0, num_head) of chunk 0 take the compensated update
        (chunked_head_kahan_fp8xmc_clf.py:127-131).  The simulated-FP8 path has no Kahan head in the
        reference either (:123-125)."""
        self._handle.bind(self._weights())
        want = None
        if self.using_head_kahan and not self.fake_fp8_matmul and self.head_kahan is not None \
                and self.head_kahan.shape[0] > 0:
            want = self.head_kahan
        ptr = None if want is None else want.data_ptr()
        if ptr != self._kahan_ptr:
            self._handle.bind_kahan(want)
            self._kahan_ptr = ptr
        return super().xfc_forward_backward(embed, labels, xmc_lr, skip_loss)
