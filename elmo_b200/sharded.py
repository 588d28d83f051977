"""Label-range sharding of the FP8 chunked XMC layer across the GPUs of one node.

The reference is single-GPU; its sequential chunk loop (chunked_fp8xmc_clf.py:96-118) shows that
label rows interact only through the sum ``grad_X += G^T W``.  Here each rank owns a contiguous
range of label rows (weights and their stochastic-rounding stream), the encoder stays data
parallel:

    X_local [B_loc, d]  --all-gather-->  X [B, d]           (bf16, B = world * B_loc)
    labels_local        --all-gather-->  labels [nnz, 2]    (rows shifted by rank * B_loc; can be started
                                                             before the encoder runs: ``prefetch_labels``)
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
                 rounding: str = "sr", time_comm: bool = False):
        self.engine = engine
        self.group = group
        self.num_rows = num_rows
        self.time_comm = time_comm          # record CUDA events around the collectives (bench bookkeeping)
        self._comm_events = []
        self._side = None                   # stream of the prefetched label all-gather
        self._lab_ready = None
        self._lab_local = None
        self._lab_prefetched = False
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

    def prefetch_labels(self, labels_local: Optional[torch.Tensor]):
        """Start the all-gather of this step's labels now -- they are known before the encoder runs
        (runner.py:139-146 moves them to the device, then calls the encoder) -- on a side stream, so that
        it overlaps the encoder forward and only the embeddings are gathered once the encoder is done.
        The next ``xfc_forward_backward`` / ``gather_inputs`` call must then pass ``labels_local=None``.
        All ranks must call it (it is a collective)."""
        lab = pad_labels(labels_local, self.capacity, self.rank * self.local_batch, self.device)
        self._lab_prefetched = True
        if self.world == 1:
            self._lab_local = lab
            return
        if self.device.type == "cuda":
            if self._side is None:
                self._side = torch.cuda.Stream(self.device)
            cur = torch.cuda.current_stream(self.device)
            self._side.wait_stream(cur)                 # `lab` was produced on the current stream
            with torch.cuda.stream(self._side):
                dist.all_gather_into_tensor(self._lg, lab, group=self.group)
                self._lab_ready = torch.cuda.Event()
                self._lab_ready.record(self._side)
            lab.record_stream(self._side)
        else:
            dist.all_gather_into_tensor(self._lg, lab, group=self.group)

    def gather_inputs(self, embed_local: torch.Tensor, labels_local: Optional[torch.Tensor]):
        assert embed_local.shape == (self.local_batch, self.dim)
        x = embed_local.to(torch.bfloat16).contiguous()
        pre = self._lab_prefetched and labels_local is None
        self._lab_prefetched = False
        lab = self._lab_local if (pre and self.world == 1) else \
            (None if pre else pad_labels(labels_local, self.capacity, self.rank * self.local_batch, self.device))
        if self.world == 1:
            return x, lab
        with self._comm():
            dist.all_gather_into_tensor(self._xg, x, group=self.group)
            if not pre:
                dist.all_gather_into_tensor(self._lg, lab, group=self.group)
        if pre and self._lab_ready is not None:
            torch.cuda.current_stream(self.device).wait_event(self._lab_ready)
        return self._xg, self._lg

    # --- collective timing -------------------------------------------------------------------
    class _Span:
        def __init__(self, owner):
            self.o = owner

        def __enter__(self):
            o = self.o
            if o.time_comm and o.device.type == "cuda":
                self.e0 = torch.cuda.Event(enable_timing=True)
                self.e1 = torch.cuda.Event(enable_timing=True)
                self.e0.record(torch.cuda.current_stream(o.device))

        def __exit__(self, *a):
            o = self.o
            if o.time_comm and o.device.type == "cuda":
                self.e1.record(torch.cuda.current_stream(o.device))
                o._comm_events.append((self.e0, self.e1))

    def _comm(self):
        return LabelShardedXMC._Span(self)

    def comm_ms(self) -> float:
        """Device milliseconds spent inside the collectives since the last call (``time_comm`` only)."""
        if not self._comm_events:
            return 0.0
        self._comm_events[-1][1].synchronize()
        ms = sum(a.elapsed_time(b) for a, b in self._comm_events)
        self._comm_events = []
        return ms

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
            with self._comm():
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
            with self._comm():
                dist.reduce_scatter_tensor(self._gl, self._g32, op=dist.ReduceOp.SUM, group=self.group)
        self.grad_input = self._gl.to(torch.bfloat16)
        self.iteration += 1
        return 0

    # --- checkpoint (runner.py:242-251 saves ``xmc_weight: model.xfc.xfc_weight``) ---------------
    def state_dict(self):
        """This rank's part of the layer: its weight chunks (CPU copies), the shard map that says which
        label rows they are, and the position of the stochastic-rounding stream.  Every rank saves its
        own; ``load_state_dict`` checks that the map matches the layer it is loaded into."""
        lo, hi = self.bounds[self.rank]
        return {"shard_map": {"world": self.world, "rank": self.rank, "num_rows": self.num_rows,
                              "bounds": [list(b) for b in self.bounds], "rows": [lo, hi]},
                "weights": [w.detach().cpu().clone() for w in self.engine.weights],
                "base_seed": self.base_seed, "iteration": self.iteration, "rounding": self.rounding,
                "w_scale": getattr(self.engine, "w_scale", 1.0)}

    def load_state_dict(self, sd):
        m = sd["shard_map"]
        if (m["world"], m["rank"], m["num_rows"]) != (self.world, self.rank, self.num_rows) or \
                [list(b) for b in self.bounds] != [list(b) for b in m["bounds"]]:
            raise ValueError(f"checkpoint shard map {m} does not match this layer "
                             f"(world {self.world}, rank {self.rank}, rows {self.num_rows})")
        if len(sd["weights"]) != len(self.engine.weights):
            raise ValueError("checkpoint has a different number of weight chunks")
        for dst, src in zip(self.engine.weights, sd["weights"]):
            if dst.shape != src.shape or dst.dtype != src.dtype:
                raise ValueError(f"weight chunk mismatch: {tuple(src.shape)} {src.dtype} vs {tuple(dst.shape)} {dst.dtype}")
            dst.copy_(src)
        self.base_seed, self.iteration = int(sd["base_seed"]), int(sd["iteration"])
        self.rounding = sd.get("rounding", self.rounding)

    def _local_rows(self) -> torch.Tensor:
        return torch.cat([w.detach() for w in self.engine.weights], 0)

    @torch.no_grad()
    def export_reference_layout(self, num_labels: int, num_chunks: int):
        """The whole layer in the reference's layout, on every rank: the list of ``num_chunks`` e4m3
        tensors ``[L_i, d]`` that ``Fp8XMCBCEChunkedLayer.xfc_weight`` holds (padding rule of
        chunked_fp8xmc_clf.py:26-28; rows this layer does not have are zero).  For bf16 weights pass
        ``num_chunks=0`` to get the dense ``[num_labels, d]`` tensor of ``XMCBCECHUNKEDLayer``."""
        mine = self._local_rows()
        per = max(hi - lo for lo, hi in self.bounds)
        raw = mine.view(torch.uint8) if mine.element_size() == 1 else mine.view(torch.int16)
        pad = torch.zeros(per, raw.shape[1], dtype=raw.dtype, device=raw.device)
        pad[:raw.shape[0]] = raw
        if self.world > 1:
            allr = torch.empty(self.world * per, raw.shape[1], dtype=raw.dtype, device=raw.device)
            dist.all_gather_into_tensor(allr, pad, group=self.group)
            parts = [allr[r * per:r * per + (hi - lo)] for r, (lo, hi) in enumerate(self.bounds)]
            rows = torch.cat(parts, 0)
        else:
            rows = pad[:raw.shape[0]]
        rows = rows.view(mine.dtype)
        if num_chunks <= 0:
            return rows[:num_labels].contiguous()
        lp = num_labels + 16 * num_chunks - num_labels % (16 * num_chunks)
        li = lp // num_chunks
        full = torch.zeros(lp, rows.shape[1], dtype=torch.uint8, device=rows.device).view(mine.dtype) \
            if mine.element_size() == 1 else torch.zeros(lp, rows.shape[1], dtype=mine.dtype, device=rows.device)
        n = min(lp, rows.shape[0])
        full[:n] = rows[:n]
        return [full[i * li:(i + 1) * li].contiguous() for i in range(num_chunks)]

    @torch.no_grad()
    def import_reference_layout(self, chunks):
        """Inverse of ``export_reference_layout``: every rank takes its label rows out of the reference's
        chunk list (or dense tensor)."""
        rows = torch.cat(list(chunks), 0) if isinstance(chunks, (list, tuple, torch.nn.ParameterList)) else chunks
        lo, hi = self.bounds[self.rank]
        src = rows[lo:min(hi, rows.shape[0])]
        off = 0
        for w in self.engine.weights:
            n = max(0, min(w.shape[0], src.shape[0] - off))
            if n:
                w[:n].copy_(src[off:off + n])
            if n < w.shape[0]:
                w[n:].zero_() if w.element_size() != 1 else w.view(torch.uint8)[n:].zero_()
            off += w.shape[0]
