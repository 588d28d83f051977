#!/usr/bin/env python
"""Benchmark of the chunked XMC classifier layer train step (samples/s).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload cfg2]
    python bench.py --pass topk [--topk 5]        # the fused top-k inference pass, one GPU

N = 1: the FP8 chunked step the headline metric is quoted on (670 091 labels x 768, batch 512,
e4m3 weights, stochastic rounding, skip-loss), through ``Fp8XMCBCEChunkedLayer``.
N > 1 (launched by torch.distributed.run, one rank per GPU): the same label space sharded by
contiguous label ranges, data-parallel batch of 512 per rank (global batch 512 N) all-gathered,
grad_X reduce-scattered: per-GPU work is constant, so scaling is "weak".

One "step" is one ``xfc_forward_backward``.  ``value`` is measured with the inputs resident on the
device over exactly ``--steps`` steps; ``sustained`` repeats such blocks until the GPU has been busy
for at least two seconds and reports the later blocks (the 1 kW power cap lowers the clocks within
about a second).  ``e2e`` feeds pinned host buffers and reads the activation gradient back every step
(the host waits for the previous step's read-back, so one step is in flight while the next is queued).
``--impl reference`` times the CPU restatement of the reference's step (oracle/) with all host threads:
the whole workload at one GPU's configuration, one shard's label rows (time scaled by the number of
shards) at larger ones.  With more than one rank the sharded layer is first checked against the CPU
oracle on a small case (``parity_check``), outside the timed region.
"""
import argparse
import json
import os
import subprocess
import sys
import threading
import time
from types import SimpleNamespace as NS

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

from elmo_b200 import synth  # noqa: E402

METRIC = "xmc_layer_train_samples_per_sec"
UNIT = "samples/s"
# dram__bytes_read.sum + dram__bytes_write.sum of one launch over 65 536 label rows (batch 512, d 768, e4m3
# weights), per label row, from an ncu capture of each kernel of the step
DRAM_BYTES_PER_ROW = {"update": 137.1e6 / 65536, "grad_x": 121.6e6 / 65536, "forward": 68.2e6 / 65536}


# --------------------------------------------------------------------------------------------
def env_int(name, default):
    return int(os.environ.get(name, default))


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        p = json.load(open(path))
        return {"hbm_gbs": p["hbm_gbs"], "bf16": p["bf16_tflops"], "bf16_sustained": p["bf16_tflops_sustained"],
                "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16": 1590.0, "bf16_sustained": 1400.0, "source": "fallback"}


class ClockSampler:
    """nvidia-smi clocks/throttle reasons sampled every 200 ms while the timed region runs."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
         "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.rows, self.proc = index, [], None

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.index), f"--query-gpu={self.Q}",
                                          "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.t = threading.Thread(target=self._read, daemon=True)
            self.t.start()
        except Exception:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def __exit__(self, *a):
        if self.proc is not None:
            time.sleep(0.25)
            self.proc.terminate()
            try:
                self.proc.wait(timeout=2)
            except Exception:
                self.proc.kill()

    def summary(self):
        sm, mx, reasons = [], [], set()
        for r in self.rows:
            try:
                sm.append(float(r[1])); mx.append(float(r[2]))
            except Exception:
                continue
            for name, col in (("hw_slowdown", 5), ("hw_thermal_slowdown", 6), ("sw_thermal_slowdown", 7),
                              ("sw_power_cap", 8)):
                if len(r) > col and r[col].lower().startswith("active"):
                    reasons.add(name)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2], "sm_max_mhz": max(mx), "reasons": sorted(reasons),
                "samples": len(sm)}


def layer_cfg(wl, device, batch, num_labels=None, num_chunks=None, sched=0, fp8_dw=False):
    return NS(environment=NS(device=str(device)),
              model=NS(xmc=NS(dtype="bfloat16", num_chunks=num_chunks or wl.num_chunks, input_features=wl.dim,
                              sched_labels=sched)),
              training=NS(precision=NS(mode="mixed", purelp_dtype="bfloat16"),
                          xmc=NS(momentum=0, wd=0.0, simulated_fp8=(wl.mode == "simfp8"), rounding=wl.rounding,
                                 fp8_dw=fp8_dw),
                          FP8=NS(using_head_kahan=False, fp8_head_kahan=False, head_ratio=0.0)),
              data=NS(num_labels=num_labels or wl.num_labels, batch_size=batch))


def L_true(wl):
    return wl.num_labels


def fill_weights(chunks, dim, seed):
    """U(+-1/sqrt(d)) e4m3 weights, generated chunk by chunk on the CPU."""
    gen = torch.Generator().manual_seed(seed)
    for c in chunks:
        c.copy_(synth.make_weights_f32(c.shape[0], dim, gen).to(torch.float8_e4m3fn))


def padded_rows(wl, world):
    """Label rows the layer holds: the FP8 class's padding rule at one GPU, a multiple of 16 rows per
    rank when sharded."""
    if world == 1:
        if wl.mode == "bf16":
            return wl.num_labels
        nc = wl.num_chunks
        return wl.num_labels + 16 * nc - wl.num_labels % (16 * nc)
    return (wl.num_labels + 16 * world - 1) // (16 * world) * (16 * world)


def workload_config(wl, world):
    """The ``config`` object both arms print."""
    B, L = wl.batch * world, wl.num_labels
    wbytes = 2 if wl.mode == "bf16" else 1
    per_gpu_mb = padded_rows(wl, world) * wl.dim * wbytes / world / 1e6
    return {"workload": f"{wl.name}: W[{L}x{wl.dim}] {'bf16' if wl.mode == 'bf16' else 'e4m3'} (padded to "
                        f"{padded_rows(wl, world)} rows), X[{B}x{wl.dim}] bf16, Poisson({wl.poisson:g}) positives/row, "
                        f"Zipf({wl.zipf_s}) ids, {'stochastic-rounding' if wl.rounding == 'sr' else 'round-to-nearest'} "
                        f"SGD lr={wl.lr}, skip-loss on",
            "labels": L, "dim": wl.dim, "global_batch": B, "parallelism": f"label-shard x{world}",
            "l2": ("inputs larger than L2: %.0f MB of weights per GPU stream through every step (L2 126 MB)" % per_gpu_mb)
            if per_gpu_mb > 126 else
            ("weights %.0f MB per GPU fit the 126 MB L2 and stay there from step to step, as they do in training; "
             "no flush between steps" % per_gpu_mb),
            "input_pool": 4}


# --------------------------------------------------------------------------------------------
def cpu_step_fn(wl, rows, batch_scale=1):
    """(closure running one CPU-oracle step over ``rows`` label rows chunked like the workload, batch)."""
    from oracle import xmc_oracle as O
    torch.set_num_threads(os.cpu_count() or 1)        # torch.distributed.run exports OMP_NUM_THREADS=1
    gen = torch.Generator().manual_seed(0)
    # label rows are independent, so the CPU walks them in blocks of 8192 (cache-sized temporaries)
    # instead of the workload's chunk size; the arithmetic per row is the same
    chunk = min(wl.chunk_labels, rows, 8192)
    chunks = []
    for s0 in range(0, rows, chunk):
        w = synth.make_weights_f32(min(chunk, rows - s0), wl.dim, gen)
        chunks.append(w.to(torch.bfloat16) if wl.mode == "bf16" else w.to(torch.float8_e4m3fn))
    B = wl.batch * batch_scale
    x, labels = synth.make_step_inputs(wl, seed=1, batch=B)
    w_all = torch.cat(chunks) if wl.mode == "bf16" else None

    def step(i):
        if wl.mode == "bf16":
            O.chunked_step(w_all, x, labels, wl.lr, num_chunks=len(chunks), rounding=wl.rounding,
                           seed=1, step=i)
        else:
            O.fp8_chunked_step(chunks, x, labels, wl.lr, simulated=(wl.mode == "simfp8"),
                               rounding=wl.rounding, seed=1, step=i)
    return step, B


def cpu_baseline_leg(wl, budget_s=20.0):
    """``cpu_baseline`` of the default run: the whole workload, all host threads, a few passes."""
    rows = padded_rows(wl, 1)
    step, B = cpu_step_fn(wl, rows)
    step(0)                                           # warm-up: thread pool, build of the C accelerator
    times = []
    t_end = time.perf_counter() + budget_s
    while len(times) < 2 or (time.perf_counter() < t_end and len(times) < 8):
        t0 = time.perf_counter()
        step(len(times) + 1)
        times.append(time.perf_counter() - t0)
    times.sort()
    t = times[len(times) // 2]
    return {"value": B / t, "unit": UNIT, "cores": torch.get_num_threads(), "kind": "port",
            "sample": f"the whole workload ({rows} label rows, batch {B}), median of {len(times)} passes "
                      f"({t:.2f} s each)"}


def run_reference(args, wl, rank, world):
    """CPU arm: the oracle port of the reference's step with all host threads.  One GPU's configuration is
    timed whole; at N > 1 each step covers one shard's label rows at the global batch and the time is
    multiplied by N (label rows are independent: chunked_fp8xmc_clf.py:96-118)."""
    if rank != 0:
        return
    rows_all = padded_rows(wl, world)
    rows = rows_all if world == 1 else rows_all // world
    step, B = cpu_step_fn(wl, rows, batch_scale=world)
    times = []
    for i in range(args.warmup + args.steps):
        t0 = time.perf_counter()
        step(i)
        if i >= args.warmup:
            times.append(time.perf_counter() - t0)
    ms = sum(times) / len(times) * 1e3 * (rows_all / rows)
    value = B / (ms / 1e3)
    sample = (f"the whole workload: {rows} label rows, batch {B}" if world == 1 else
              f"each step = one shard's {rows} of {rows_all} label rows at the global batch {B}; time x{world}")
    cpu = {"value": value, "unit": UNIT, "cores": torch.get_num_threads(), "kind": "port", "sample": sample}
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True,
        "scaling": args.scaling, "vs_baseline": None, "dtype": "e4m3/bf16 storage, fp32 arithmetic on CPU",
        "data": "synthetic", "config": workload_config(wl, world), "cpu_baseline": cpu,
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}))


# --------------------------------------------------------------------------------------------
def timed_block(fn, first, steps, world, device):
    """``steps`` calls fn(first + i) bracketed by barrier + synchronize on both sides, CUDA events on the
    current stream, max over ranks.  Returns milliseconds."""
    import torch.distributed as dist
    torch.cuda.synchronize(device)
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize(device)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(steps):
        fn(first + i)
    e1.record()
    torch.cuda.synchronize(device)
    ms = torch.tensor([e0.elapsed_time(e1)], device=device, dtype=torch.float64)
    if world > 1:
        dist.barrier()
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    return float(ms.item())


def run_ours(args, wl, rank, local_rank, world):
    import torch.distributed as dist
    assert torch.cuda.is_available(), "bench.py needs a CUDA device (sm_100a); there is no CPU fallback"
    device = torch.device("cuda", local_rank)
    torch.cuda.set_device(device)
    parity = None
    if world > 1:
        dist.init_process_group("nccl", device_id=device)
        # sharded layer vs the CPU oracle on a small case, before anything is timed
        from tests.dist_sharded_check import run_check
        parity = run_check(device, rank, world)
    from elmo_b200.sharded import CudaShardEngine, LabelShardedXMC, shard_bounds
    from elmo_b200.xmc_classifiers import Fp8XMCBCEChunkedLayer

    b_loc = wl.batch
    B = b_loc * world
    n_pool = 4
    sampler = synth.ZipfSampler(wl.num_labels, wl.zipf_s)
    pool = []
    for i in range(n_pool):
        gen = torch.Generator().manual_seed(1000 + 17 * rank + i)
        x = synth.make_embeddings(b_loc, wl.dim, gen)
        lab = synth.make_labels(b_loc, sampler, wl.poisson, wl.clip, gen)
        pool.append((x, lab))

    n_rows = padded_rows(wl, world)
    layer_sharded = None
    if world == 1:
        if wl.mode == "bf16":
            from elmo_b200.xmc_classifiers import XMCBCECHUNKEDLayer
            layer = XMCBCECHUNKEDLayer(layer_cfg(wl, device, b_loc, sched=args.sched))
            gen = torch.Generator().manual_seed(0)
            for s0 in range(0, wl.num_labels, 65536):
                blk = layer.xfc_weight[s0:s0 + 65536]
                blk.copy_(synth.make_weights_f32(blk.shape[0], wl.dim, gen).to(torch.bfloat16))
        else:
            layer = Fp8XMCBCEChunkedLayer(layer_cfg(wl, device, b_loc, sched=args.sched, fp8_dw=(args.backward == "fp8dw")))
            fill_weights([p.data for p in layer.xfc_weight], wl.dim, seed=0)
            assert layer.num_labels == n_rows
        handle = layer._handle
    else:
        lo, hi = shard_bounds(n_rows, world)[rank]
        w = torch.empty(hi - lo, wl.dim, dtype=torch.float8_e4m3fn, device=device)
        fill_weights([w], wl.dim, seed=rank)
        engine = CudaShardEngine(device, wl.dim, B, wl.mode, lo, [w], sched_labels=args.sched)
        layer = LabelShardedXMC(engine, dim=wl.dim, local_batch=b_loc, num_rows=n_rows, label_capacity=b_loc * 64,
                                device=device, base_seed=1234, rounding=wl.rounding)
        layer_sharded = layer
        handle = engine.handle
    step_fn = lambda x, lab: layer.xfc_forward_backward(x, lab, [wl.lr], skip_loss=True)
    grad_of = lambda: layer.grad_input
    dev_pool = [(x.to(device), l.to(device)) for x, l in pool]
    pin_pool = [(x.pin_memory(), l.pin_memory()) for x, l in pool]
    host_grad = [torch.empty(b_loc, wl.dim, dtype=torch.bfloat16).pin_memory() for _ in range(2)]
    read_done = [torch.cuda.Event(), torch.cuda.Event()]
    e2e_state = {"prev": -1}

    def step_resident(i):
        x, lab = dev_pool[i % n_pool]
        step_fn(x, lab)

    def step_e2e(i):
        # every step: inputs come from pinned host memory, the activation gradient goes back to pinned
        # host memory.  The host waits for the PREVIOUS step's read-back while this step is already
        # queued (two host buffers), as a training loop that consumes the result one step later would.
        x, lab = pin_pool[i % n_pool]
        step_fn(x.to(device, non_blocking=True), lab.to(device, non_blocking=True))
        s = i & 1
        host_grad[s].copy_(grad_of(), non_blocking=True)
        read_done[s].record(torch.cuda.current_stream(device))
        if e2e_state["prev"] >= 0:
            read_done[e2e_state["prev"]].synchronize()
        e2e_state["prev"] = s

    torch.cuda.reset_peak_memory_stats(device)
    for i in range(args.warmup):
        step_resident(i)
    l0 = handle.launch_count
    with ClockSampler(local_rank) as clk:
        ms = timed_block(step_resident, args.warmup, args.steps, world, device)
    launches = (handle.launch_count - l0) // args.steps

    # sustained figure: keep going in blocks of --steps until 2 s of GPU time have passed since the timed
    # block began; the blocks that start after the first second are averaged
    busy, blocks = ms, []
    with ClockSampler(local_rank) as clk_s:
        n_blk = 0
        while busy < 2000.0 and n_blk < 400:
            t = timed_block(step_resident, args.warmup + args.steps * (n_blk + 1), args.steps, world, device)
            if busy >= 1000.0:
                blocks.append(t)
            busy += t
            n_blk += 1
    sus_ms = (sum(blocks) / len(blocks) / args.steps) if blocks else ms / args.steps

    for i in range(3):
        step_e2e(i)
    ms_e2e = timed_block(step_e2e, 3, args.steps, world, device)
    handle.check()

    # collectives: CUDA events around every NCCL call of a few steps (they serialise with the kernels on
    # the step's stream, so their share is read directly)
    comm_ms = None
    if layer_sharded is not None:
        layer_sharded.time_comm = True
        layer_sharded.comm_ms()
        for i in range(10):
            step_resident(i)
        comm_ms = layer_sharded.comm_ms() / 10
        layer_sharded.time_comm = False

    # per-kernel-class timing (CUDA events inside the library, on the launching stream)
    handle.profile(True)
    n_prof = 5
    for i in range(n_prof):
        step_resident(i)
    prof = handle.profile(False, read=True)
    peak_hbm = (torch.cuda.max_memory_allocated(device) + handle.workspace_bytes) / 1e9

    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    if rank != 0:
        return
    pk = peaks()
    L = wl.num_labels
    gemm_flops = 2.0 * B * (L / world) * wl.dim        # per rank, per contraction, padding not credited
    per_step = {k: v[0] / n_prof for k, v in prof.items()}
    dominant = max(("forward", "grad_x", "update"), key=lambda k: per_step.get(k, 0.0))
    dom_ms = per_step[dominant]
    dom_launches = prof[dominant][1] / n_prof
    achieved = gemm_flops / (dom_ms * 1e-3) / 1e12
    # DRAM bytes (read + write) one launch over a 65 536-row chunk moves at batch 512, d 768, from an ncu
    # capture of each kernel; traffic grows with the label rows a launch covers, so it is scaled by them
    dram_per_row = {"update": DRAM_BYTES_PER_ROW["update"], "grad_x": DRAM_BYTES_PER_ROW["grad_x"],
                    "forward": DRAM_BYTES_PER_ROW["forward"]}
    rows_per_launch = (L / world) / max(dom_launches, 1.0)
    traffic = dram_per_row[dominant] * rows_per_launch if (wl.dim == 768 and B == 512 and wl.mode == "fp8") else None
    clocks = clk.summary()
    at_max = bool(clocks["sm_mhz"]) and clocks["sm_mhz"] >= 0.97 * (clocks["sm_max_mhz"] or 1e9)
    fp8_dom = dominant == "forward" and wl.mode == "fp8"
    base_peak = pk["bf16"] if at_max else pk["bf16_sustained"]
    peak = base_peak * (2.0 if fp8_dom else 1.0)
    peak_name = pk["source"] + (" bf16 burst" if at_max else " bf16 sustained") + \
        (" (SM clock stayed at its maximum during the timed block)" if at_max else " (SM clock dropped during the timed block)") + \
        (" x2: no measured fp8 figure" if fp8_dom else "")
    step_ms = ms / args.steps
    total_flops = 6.0 * B * L * wl.dim
    cfg = workload_config(wl, world)
    cfg["input_pool"] = n_pool
    out = {
        "metric": METRIC, "value": B * args.steps / (ms * 1e-3), "unit": UNIT, "n_gpus": world,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": step_ms, "higher_is_better": True,
        "scaling": args.scaling, "vs_baseline": None,
        "dtype": ("bf16 weights; all contractions bf16 x bf16, fp32 accumulate" if wl.mode == "bf16" else
                  ("e4m3 weights; forward and dW e4m3 x e4m3, grad_X bf16 x bf16, fp32 accumulate (variant, not the reference's arithmetic)"
                   if args.backward == "fp8dw" else
                   "e4m3 weights; forward e4m3 x e4m3, backward bf16 x bf16, fp32 accumulate") if wl.mode == "fp8" else
                  "e4m3 weights up-converted to bf16; all contractions bf16 x bf16, fp32 accumulate"),
        "data": "synthetic", "config": cfg, "clocks": clocks,
        "sustained": {"ms_per_step": sus_ms, "value": B / (sus_ms * 1e-3), "unit": UNIT,
                      "gpu_seconds": busy / 1e3, "blocks_averaged": len(blocks),
                      "sm_mhz_median": clk_s.summary()["sm_mhz"], "reasons": clk_s.summary()["reasons"]},
        "e2e": {"value": B * args.steps / (ms_e2e * 1e-3), "unit": UNIT,
                "h2d_bytes_per_step": int(sum(x.numel() * 2 + l.numel() * 4 for x, l in pool) / n_pool),
                "d2h_bytes_per_step": int(host_grad[0].numel() * 2)},
        "gpu_launches": int(launches),
        "roofline": {"bound": "tensor", "kernel": dominant, "achieved": achieved, "peak": peak, "unit": "TFLOP/s",
                     "frac": achieved / peak, "traffic": traffic,
                     "traffic_note": "DRAM bytes per launch, ncu capture of a 65536-row chunk scaled by rows per launch",
                     "peak_source": peak_name, "launches_per_step": dom_launches, "ms_per_step": dom_ms},
        "kernel_ms_per_step": per_step,
        "step_tflops": total_flops / (step_ms * 1e-3) / 1e12,
        "peak_hbm_gb_per_gpu": peak_hbm,
    }
    if comm_ms is not None:
        out["comm_ms_per_step"] = comm_ms
    if parity is not None:
        out["parity_check"] = parity
    if world == 1 and not args.no_cpu:
        out["cpu_baseline"] = cpu_baseline_leg(wl)
    print(json.dumps(out))


def run_topk(args, wl, rank, local_rank, world):
    """``--pass topk``: the fused logits + top-k inference pass (a line of its own; the default run never
    comes here).  One GPU: through ``Fp8XMCBCEChunkedLayer.xfc_topk``.  N GPUs: label shards, the batch
    of wl.batch rows per rank all-gathered, per-shard top-k candidates all-gathered and merged."""
    import torch.distributed as dist
    assert torch.cuda.is_available(), "bench.py needs a CUDA device (sm_100a); there is no CPU fallback"
    device = torch.device("cuda", local_rank)
    torch.cuda.set_device(device)
    k = args.topk
    B = wl.batch * world
    gen = torch.Generator().manual_seed(5 + rank)
    xs = [synth.make_embeddings(wl.batch, wl.dim, gen).to(device) for _ in range(4)]
    sharded = None
    if world == 1:
        from elmo_b200.xmc_classifiers import Fp8XMCBCEChunkedLayer
        layer = Fp8XMCBCEChunkedLayer(layer_cfg(wl, device, wl.batch, sched=args.sched))
        fill_weights([p.data for p in layer.xfc_weight], wl.dim, seed=0)
        handle = layer._handle
        call = lambda x: layer.xfc_topk(x, k)
    else:
        dist.init_process_group("nccl", device_id=device)
        from elmo_b200.sharded import CudaShardEngine, LabelShardedXMC, shard_bounds
        n_rows = padded_rows(wl, world)
        lo, hi = shard_bounds(n_rows, world)[rank]
        w = torch.empty(hi - lo, wl.dim, dtype=torch.float8_e4m3fn, device=device)
        fill_weights([w], wl.dim, seed=rank)
        engine = CudaShardEngine(device, wl.dim, B, wl.mode, lo, [w], sched_labels=args.sched)
        sharded = LabelShardedXMC(engine, dim=wl.dim, local_batch=wl.batch, num_rows=n_rows, device=device,
                                  time_comm=True)
        handle = engine.handle
        call = lambda x: sharded.xfc_topk(x, k, wl.num_labels)
    for i in range(max(3, args.warmup)):
        call(xs[i % 4])
    if sharded is not None:
        sharded.comm_ms()
    ms = timed_block(lambda i: call(xs[i % 4]), 0, args.steps, world, device) / args.steps
    comm = sharded.comm_ms() / args.steps if sharded is not None else None
    handle.check()
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    if rank != 0:
        return
    flops = 2.0 * B * wl.num_labels * wl.dim
    pk = peaks()
    out = {
        "metric": "xmc_layer_topk_samples_per_sec", "value": B / (ms * 1e-3), "unit": UNIT, "n_gpus": world,
        "steps": args.steps, "warmup": max(3, args.warmup), "ms_per_step": ms, "higher_is_better": True,
        "dtype": "e4m3 x e4m3, fp32 accumulate, bf16 logits", "data": "synthetic",
        "config": {"workload": f"{wl.name}: top-{k} of W[{wl.num_labels}x{wl.dim}] e4m3 for X[{B}x{wl.dim}] bf16",
                   "parallelism": f"label-shard x{world}", "l2": "weights larger than L2"},
        "roofline": {"bound": "tensor", "kernel": "top-k", "achieved": flops / world / (ms * 1e-3) / 1e12,
                     "peak": pk["bf16_sustained"] * 2.0, "unit": "TFLOP/s",
                     "frac": flops / world / (ms * 1e-3) / 1e12 / (pk["bf16_sustained"] * 2.0), "traffic": None,
                     "peak_source": pk["source"] + " bf16 sustained x2 (no measured fp8 figure)"}}
    if comm is not None:
        out["comm_ms_per_step"] = comm
    print(json.dumps(out))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=100)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="cfg2", choices=sorted(synth.WORKLOADS))
    ap.add_argument("--sched", type=int, default=0, help="labels per scheduling chunk (0 = library default)")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg (tuning runs)")
    ap.add_argument("--rounding", default="", choices=["", "rn", "sr"], help="override the rounding mode")
    ap.add_argument("--labels", type=int, default=0, help="override the label count (small profiling captures)")
    ap.add_argument("--batch", type=int, default=0, help="override the per-rank batch")
    ap.add_argument("--pass", dest="which", default="train", choices=["train", "topk"],
                    help="train = the layer's train step (default); topk = the fused top-k inference pass")
    ap.add_argument("--topk", type=int, default=5)
    ap.add_argument("--backward", default="bf16", choices=["bf16", "fp8dw"],
                    help="bf16 = the reference's backward arithmetic (default); fp8dw = e4m3 operands in the dW "
                         "contraction (one GPU; a variant line, not the headline)")
    ap.add_argument("--global-batch", type=int, default=0,
                    help="fix the GLOBAL batch (per-rank batch = this / N): strong scaling instead of the default weak scaling")
    args = ap.parse_args()
    rank, local_rank, world = env_int("RANK", 0), env_int("LOCAL_RANK", 0), env_int("WORLD_SIZE", 1)
    wl = synth.WORKLOADS[args.workload]
    if args.labels or args.batch:
        import dataclasses
        wl = dataclasses.replace(wl, name=wl.name + "-resized", num_labels=args.labels or wl.num_labels,
                                 batch=args.batch or wl.batch)
    if args.rounding:
        import dataclasses
        wl = dataclasses.replace(wl, rounding=args.rounding)
    args.scaling = "weak"
    if args.global_batch:
        import dataclasses
        assert args.global_batch % (16 * world) == 0, "global batch must split into multiples of 16 rows per rank"
        wl = dataclasses.replace(wl, batch=args.global_batch // world)
        args.scaling = "strong"
    if args.impl == "reference":
        run_reference(args, wl, rank, world)
    elif args.which == "topk":
        run_topk(args, wl, rank, local_rank, world)
    else:
        run_ours(args, wl, rank, local_rank, world)


if __name__ == "__main__":
    main()
