"""Caller-side glue for the XMC layer step: label collation, host->device staging, the runner's step.

Mirrors the three places of the reference that sit directly around ``xfc_forward_backward``:

* ``collate`` (data.py:16-33): per-sample label lists -> int32 COO ``[nnz, 2]`` of (batch row, label id).
  The reference builds a Python list of tuples and goes through a float32 tensor; here the pairs are
  written straight into an int32 buffer (pinned when CUDA is present), which also keeps ids above
  2^24 exact.
* the ``.to(device)`` of the runner (runner.py:139-140): ``StepStager`` double-buffers pinned host
  memory and copies on a side stream, so the copy of step t+1 overlaps the layer step of step t.
* the call sequence of the runner (runner.py:146-157): ``xmc_train_step``.

Nothing in here computes; the layer itself is ``elmo_b200.xmc_classifiers``.
"""
from typing import Iterable, List, Optional, Sequence, Tuple

import numpy as np
import torch


def collate_labels(label_lists: Sequence[Iterable[int]], pin: Optional[bool] = None) -> torch.Tensor:
    """int32 ``[nnz, 2]`` COO of (batch row, label id), rows ascending, ids in the order given
    (data.py:24-28).  An empty batch of labels gives shape ``[0, 2]``."""
    counts = np.fromiter((len(l) for l in label_lists), dtype=np.int64, count=len(label_lists))
    nnz = int(counts.sum())
    pin = torch.cuda.is_available() if pin is None else pin
    out = torch.empty((nnz, 2), dtype=torch.int32, pin_memory=bool(pin and nnz > 0))
    if nnz:
        arr = out.numpy()
        arr[:, 0] = np.repeat(np.arange(len(label_lists), dtype=np.int32), counts)
        arr[:, 1] = np.fromiter((x for l in label_lists for x in l), dtype=np.int64, count=nnz).astype(np.int32)
    return out


def collate(batch):
    """Drop-in for data.py:16-33: ``(tokens, attention_mask, labels)`` with default collation of the
    first two and ``collate_labels`` for the third."""
    tokens = [b[0] for b in batch]
    masks = [b[1] for b in batch]
    return (torch.utils.data.default_collate(tokens), torch.utils.data.default_collate(masks),
            collate_labels([b[2] for b in batch]))


class StepStager:
    """Double-buffered host->device staging of the per-step label COO (and, optionally, of host
    embeddings): ``put`` enqueues the copies on a side stream, ``get`` makes the current stream wait
    for them and returns device tensors that stay valid until the second-next ``put``."""

    def __init__(self, device, label_capacity: int, embed_shape: Optional[Tuple[int, int]] = None,
                 embed_dtype=torch.bfloat16, depth: int = 2):
        self.device = torch.device(device)
        self.cuda = self.device.type == "cuda"
        self.depth = depth
        self.capacity = int(label_capacity)
        mk = dict(pin_memory=self.cuda)
        self._h_lab = [torch.empty((self.capacity, 2), dtype=torch.int32, **mk) for _ in range(depth)]
        self._d_lab = [torch.empty((self.capacity, 2), dtype=torch.int32, device=self.device) for _ in range(depth)]
        self._h_x = self._d_x = None
        if embed_shape is not None:
            self._h_x = [torch.empty(embed_shape, dtype=embed_dtype, **mk) for _ in range(depth)]
            self._d_x = [torch.empty(embed_shape, dtype=embed_dtype, device=self.device) for _ in range(depth)]
        self._stream = torch.cuda.Stream(self.device) if self.cuda else None
        self._ready = [torch.cuda.Event() for _ in range(depth)] if self.cuda else None
        self._consumed = [None] * depth
        self._used = [False] * depth
        self._nnz = [0] * depth
        self._rows = [0] * depth
        self._put = 0
        self._got = 0

    def put(self, labels: torch.Tensor, embed: Optional[torch.Tensor] = None):
        if self._put - self._got >= self.depth:
            raise RuntimeError("StepStager.put called %d times without get" % self.depth)
        s = self._put % self.depth
        n = int(labels.shape[0])
        if n > self.capacity:
            raise ValueError(f"{n} label pairs exceed the staging capacity {self.capacity}")
        if labels.dtype != torch.int32 or (n and tuple(labels.shape[1:]) != (2,)):
            raise ValueError("labels must be int32 [nnz, 2]")
        if self.cuda and self._used[s]:
            # the pinned slot is about to be rewritten by the host: the copy that last read it (queued on
            # the side stream behind the step two puts ago) must have run, or that step would see these data
            self._ready[s].synchronize()
        self._used[s] = True
        self._nnz[s] = n
        self._h_lab[s][:n].copy_(labels.reshape(n, 2))
        if embed is not None:
            if self._h_x is None:
                raise ValueError("the stager was built without an embedding buffer")
            self._rows[s] = int(embed.shape[0])
            self._h_x[s][:embed.shape[0]].copy_(embed)
        if self.cuda:
            if self._consumed[s] is not None:
                self._stream.wait_event(self._consumed[s])      # the step that read slot s has finished with it
            with torch.cuda.stream(self._stream):
                self._d_lab[s][:n].copy_(self._h_lab[s][:n], non_blocking=True)
                if embed is not None:
                    self._d_x[s][:self._rows[s]].copy_(self._h_x[s][:self._rows[s]], non_blocking=True)
                self._ready[s].record(self._stream)
        else:
            self._d_lab[s][:n].copy_(self._h_lab[s][:n])
            if embed is not None:
                self._d_x[s][:self._rows[s]].copy_(self._h_x[s][:self._rows[s]])
        self._put += 1

    def get(self):
        """(labels on the device, embeddings on the device or None) of the oldest staged step."""
        if self._got >= self._put:
            raise RuntimeError("StepStager.get called with nothing staged")
        s = self._got % self.depth
        if self.cuda:
            torch.cuda.current_stream(self.device).wait_event(self._ready[s])
        self._got += 1
        lab = self._d_lab[s][:self._nnz[s]]
        x = self._d_x[s][:self._rows[s]] if self._d_x is not None and self._rows[s] else None
        return lab, x

    def release(self):
        """Call after enqueuing the step that consumed the last ``get``: marks its slot reusable once
        the work enqueued so far on the current stream has run."""
        s = (self._got - 1) % self.depth
        if self.cuda:
            ev = torch.cuda.Event()
            ev.record(torch.cuda.current_stream(self.device))
            self._consumed[s] = ev


def xmc_train_step(layer, out: torch.Tensor, labels: torch.Tensor, xmc_lr: List[float], *,
                   grad_accum_step: int = 1, skip_loss: bool = True):
    """runner.py:146-157 in one call: layer step, scale of the embedding gradient by the encoder's
    gradient-accumulation factor, back-propagation into the encoder graph.  Returns the loss value
    the layer reports (0 when skipped)."""
    bsz = out.shape[0]
    with torch.no_grad():
        loss = layer.xfc_forward_backward(out.detach(), labels, xmc_lr, skip_loss=skip_loss)
        g = layer.grad_input[0:bsz, :]
        if grad_accum_step != 1:
            g.div_(grad_accum_step)
    if out.requires_grad:
        out.backward(g)
    return loss
