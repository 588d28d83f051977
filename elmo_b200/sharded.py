"""Label-range sharding of the FP8 chunked XMC layer across the GPUs of one node.

The reference is single-GPU; its sequential chunk loop (chunked_fp8xmc_clf.py:96-118) shows that
label rows interact only through the sum ``grad_X += G^T W``.  Here each rank owns a contiguous
range of label rows (weights and their stochastic-rounding stream), the encoder stays data
parallel:

    X_local [B_loc, d]  --all-gather-->  X [B, d]           (bf16, B = world * B_loc)
    labels_local        --all-gather-->  labels [nnz, 2]    (rows shifted by rank * B_loc)
    local shard step on the CUDA library (forward, grad_X partial, weight update)
    grad_X [B, d] fp32  --reduce-scatter(sum)-->  grad_input [B_loc, d]

Collectives go through ``torch.distributed`` (NCCL on GPUs); all buffers are local device memory.
Results do not depend on the number of ranks: the Philox counter is the global element index.
"""
from typing import List, Optional, Tuple

import torch
import torch.distributed as dist

INT32_MAX = 2 ** 31 - 1


def shard_bounds(num_rows: int, world: int, align: int = 16) -> List[Tuple[int, int]]:
    """Contiguous ranges: rank r owns [r*per, min((r+1)*per, L)), per = ceil(L/world) rounded up
    to ``align`` rows."""
    per = (num_rows + world - 1) // world
    per = (per + align - 1) // align * align
    return [(min(r * per, num_rows), min((r + 1) * per, num_rows)) for r in range(world)]


def pad_labels(labels: Optional[torch.Tensor], capacity: int, row_offset: int, device) -> torch.Tensor:
    """Fixed-size [capacity, 2] int32 block for the all-gather: real pairs first (rows shifted to
    global batch rows), the rest filled with (0, INT32_MAX), an id no shard owns."""
    buf = torch.empty(capacity, 2, dtype=torch.int32, device=device)
    buf[:, 0] = 0
    buf[:, 1] = INT32_MAX
    n = 0 if labels is None else labels.shape[0]
    if n > capacity:
        raise ValueError(f"{n} label pairs exceed the per-rank capacity {capacity}")
    if n:
        buf[:n] = labels.to(device=device, dtype=torch.int32)
        buf[:n, 0] += row_offset
    return buf


class CudaShardEngine:
    """The local shard on the CUDA library (the only engine the product uses)."""

    def __init__(self, device, dim, max_batch, mode, label_offset, weights, w_scale=1.0, sched_labels=0):
        from .handle import XmcHandle
        self.handle = XmcHandle(device, dim, max_batch, mode, label_offset=label_offset,
                                w_scale=w_scale, sched_labels=sched_labels)
        self.weights = weights
        self.handle.bind(weights)

    def step(self, x, labels, lr, seed, step, stochastic, grad_f32, compute_loss=False, loss_out=None):
        self.handle.bind(self.weights)
        self.handle.step(x, labels, lr, seed=seed, step=step, stochastic=stochastic,
                         compute_loss=compute_loss, grad_f32=grad_f32, loss_out=loss_out)

    def topk(self, x, k, n_out):
        """(values fp32 [B, k], GLOBAL label ids int32 [B, k]) over this shard's first n_out rows."""
        self.handle.bind(self.weights)
        return self.handle.forward_topk(x, k, n_out)


class LabelShardedXMC:
    """One rank's view of a label-sharded FP8 XMC layer.

    ``weights``: this rank's e4m3 chunks (rows of ``bounds[rank]``).  ``engine`` runs the local
    step; tests substitute a CPU engine to exercise the collective plumbing with gloo.
    """

    def __init__(self, engine, *, dim: int, local_batch: int, num_rows: int, group=None,
                 label_capacity: Optional[int] = None, device=None, base_seed: int = 0,
                 rounding: str = "sr"):
        self.engine = engine
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.dim, self.local_batch = dim, local_batch
        self.bounds = shard_bounds(num_rows, self.world)
        self.device = torch.device(device) if device is not None else torch.device("cpu")
        self.capacity = label_capacity or local_batch * 64
        self.base_seed, self.rounding = base_seed, rounding
        self.iteration = 0
        B = self.world * local_batch
        self._xg = torch.empty(B, dim, dtype=torch.bfloat16, device=self.device)
        self._lg = torch.empty(self.world * self.capacity, 2, dtype=torch.int32, device=self.device)
        self._g32 = torch.zeros(B, dim, dtype=torch.float32, device=self.device)
        self._gl = torch.zeros(local_batch, dim, dtype=torch.float32, device=self.device)
        self.grad_input = torch.zeros(local_batch, dim, dtype=torch.bfloat16, device=self.device)

    def gather_inputs(self, embed_local: torch.Tensor, labels_local: Optional[torch.Tensor]):
        assert embed_local.shape == (self.local_batch, self.dim)
        x = embed_local.to(torch.bfloat16).contiguous()
        lab = pad_labels(labels_local, self.capacity, self.rank * self.local_batch, self.device)
        if self.world == 1:
            return x, lab
        dist.all_gather_into_tensor(self._xg, x, group=self.group)
        dist.all_gather_into_tensor(self._lg, lab, group=self.group)
        return self._xg, self._lg

    @torch.no_grad()
    def xfc_topk(self, embed_local, k: int, num_labels: int):
        """Top-k labels of the rank's own batch rows over ALL shards: every rank scores the gathered
        batch against its label range (fused logits + top-k, nothing materialised), the per-shard
        candidates [B, k] are all-gathered and merged locally.  ``num_labels`` is the true label count
        (padding rows beyond it never appear).  Returns (values [B_loc, k], ids [B_loc, k])."""
        x, _ = self.gather_inputs(embed_local, None)
        lo, hi = self.bounds[self.rank]
        n_out = max(0, min(hi, num_labels) - lo)
        B = x.shape[0]
        if n_out > 0:
            vals, idx = self.engine.topk(x, min(k, n_out), n_out)
            if vals.shape[1] < k:
                pad = k - vals.shape[1]
                vals = torch.cat([vals, vals.new_full((B, pad), float("-inf"))], 1)
                idx = torch.cat([idx, idx.new_full((B, pad), -1)], 1)
        else:
            vals = torch.full((B, k), float("-inf"), dtype=torch.float32, device=self.device)
            idx = torch.full((B, k), -1, dtype=torch.int32, device=self.device)
        if self.world > 1:
            all_v = torch.empty(self.world * B, k, dtype=vals.dtype, device=self.device)
            all_i = torch.empty(self.world * B, k, dtype=idx.dtype, device=self.device)
            dist.all_gather_into_tensor(all_v, vals.contiguous(), group=self.group)
            dist.all_gather_into_tensor(all_i, idx.contiguous(), group=self.group)
            cand_v = all_v.view(self.world, B, k).permute(1, 0, 2).reshape(B, self.world * k)
            cand_i = all_i.view(self.world, B, k).permute(1, 0, 2).reshape(B, self.world * k)
            # shards are in ascending label order, so a stable descending sort keeps the lower id on ties
            order = torch.argsort(cand_v, dim=1, descending=True, stable=True)[:, :k]
            vals, idx = torch.gather(cand_v, 1, order), torch.gather(cand_i, 1, order)
        r0 = self.rank * self.local_batch
        return vals[r0:r0 + self.local_batch], idx[r0:r0 + self.local_batch]

    def xfc_forward_backward(self, embed_local, labels_local, xmc_lr, skip_loss=True):
        x, lab = self.gather_inputs(embed_local, labels_local)
        self.engine.step(x, lab, xmc_lr[0], self.base_seed, self.iteration,
                         self.rounding == "sr", self._g32)
        if self.world == 1:
            self._gl = self._g32
        else:
            dist.reduce_scatter_tensor(self._gl, self._g32, op=dist.ReduceOp.SUM, group=self.group)
        self.grad_input = self._gl.to(torch.bfloat16)
        self.iteration += 1
        return 0
