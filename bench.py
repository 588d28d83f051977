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
device; ``e2e`` feeds pinned host buffers and reads the activation gradient back every step (the host
waits for the previous step's read-back, so one step is in flight while the next is queued).
``--impl reference`` times the CPU restatement of the reference's step (oracle/) on a bounded
sample of the same workload with all host threads.
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


def layer_cfg(wl, device, batch, num_labels=None, num_chunks=None, sched=0):
    return NS(environment=NS(device=str(device)),
              model=NS(xmc=NS(dtype="bfloat16", num_chunks=num_chunks or wl.num_chunks, input_features=wl.dim,
                              sched_labels=sched)),
              training=NS(precision=NS(mode="mixed", purelp_dtype="bfloat16"),
                          xmc=NS(momentum=0, wd=0.0, simulated_fp8=(wl.mode == "simfp8"), rounding=wl.rounding),
                          FP8=NS(using_head_kahan=False, fp8_head_kahan=False, head_ratio=0.0)),
              data=NS(num_labels=num_labels or wl.num_labels, batch_size=batch))


def L_true(wl):
    return wl.num_labels


def fill_weights(chunks, dim, seed):
    """U(+-1/sqrt(d)) e4m3 weights, generated chunk by chunk on the CPU."""
    gen = torch.Generator().manual_seed(seed)
    for c in chunks:
        c.copy_(synth.make_weights_f32(c.shape[0], dim, gen).to(torch.float8_e4m3fn))


# --------------------------------------------------------------------------------------------
def cpu_step_sample(wl, sample_labels, reps_budget_s, threads=None):
    """Time the CPU restatement of the reference step on the first ``sample_labels`` label rows of
    the workload (same batch, same arithmetic) and scale to the full label count."""
    from oracle import xmc_oracle as O
    if threads:
        torch.set_num_threads(threads)
    gen = torch.Generator().manual_seed(0)
    w = synth.make_weights_f32(sample_labels, wl.dim, gen).to(torch.float8_e4m3fn)
    x, labels = synth.make_step_inputs(wl, seed=1)
    times = []
    t_end = time.perf_counter() + reps_budget_s
    step = 0
    while True:
        t0 = time.perf_counter()
        if wl.mode == "bf16":
            O.chunked_step(w.to(torch.bfloat16), x, labels, wl.lr, num_chunks=1, rounding=wl.rounding,
                           seed=1, step=step)
        else:
            O.fp8_chunked_step([w], x, labels, wl.lr, simulated=(wl.mode == "simfp8"),
                               rounding=wl.rounding, seed=1, step=step)
        times.append(time.perf_counter() - t0)
        step += 1
        if time.perf_counter() > t_end and len(times) >= 2:
            break
    times.sort()
    t = times[len(times) // 2]
    full = t * wl.num_labels / sample_labels
    return {"value": wl.batch / full, "unit": UNIT, "cores": torch.get_num_threads(), "kind": "port",
            "sample": f"first {sample_labels} of {wl.num_labels} label rows, batch {wl.batch}, "
                      f"median of {len(times)} passes ({t * 1e3:.0f} ms each), scaled by label count"}, t


def run_reference(args, wl, rank, world):
    """CPU arm: the oracle port of the reference's step, all host threads, bounded sample/step."""
    if rank != 0:
        return
    sample = 8192
    base, t = cpu_step_sample(wl, sample, reps_budget_s=0.0)       # warm-up + first estimate
    times = []
    from oracle import xmc_oracle as O
    gen = torch.Generator().manual_seed(0)
    w = synth.make_weights_f32(sample, wl.dim, gen).to(torch.float8_e4m3fn)
    x, labels = synth.make_step_inputs(wl, seed=1)
    for i in range(args.warmup + args.steps):
        t0 = time.perf_counter()
        O.fp8_chunked_step([w], x, labels, wl.lr, rounding=wl.rounding, seed=1, step=i)
        if i >= args.warmup:
            times.append(time.perf_counter() - t0)
    ms = sum(times) / len(times) * 1e3
    full_ms = ms * wl.num_labels / sample
    value = wl.batch / (full_ms / 1e3)
    cpu = {"value": value, "unit": UNIT, "cores": torch.get_num_threads(), "kind": "port",
           "sample": f"each step = first {sample} of {wl.num_labels} label rows at batch {wl.batch}; "
                     f"time scaled by label count"}
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": full_ms, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "e4m3/bf16 storage, fp32 arithmetic on CPU",
        "data": "synthetic", "config": {"workload": wl.name + " (CPU restatement of the reference step)"},
        "cpu_baseline": cpu,
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}))


# --------------------------------------------------------------------------------------------
def timed(fn, steps, warmup, world, device):
    """W warm-up + K timed calls of fn(i): barrier + synchronize on both sides, CUDA events on the
    current stream, max over ranks.  Returns total milliseconds."""
    import torch.distributed as dist
    for i in range(warmup):
        fn(i)
    torch.cuda.synchronize(device)
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize(device)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(steps):
        fn(warmup + i)
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
    if world > 1:
        dist.init_process_group("nccl", device_id=device)
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
    cap = max(int(l.shape[0]) for _, l in pool) + 64

    if world == 1:
        if wl.mode == "bf16":
            from elmo_b200.xmc_classifiers import XMCBCECHUNKEDLayer
            layer = XMCBCECHUNKEDLayer(layer_cfg(wl, device, b_loc, sched=args.sched))
            gen = torch.Generator().manual_seed(0)
            for s0 in range(0, wl.num_labels, 65536):
                blk = layer.xfc_weight[s0:s0 + 65536]
                blk.copy_(synth.make_weights_f32(blk.shape[0], wl.dim, gen).to(torch.bfloat16))
        else:
            layer = Fp8XMCBCEChunkedLayer(layer_cfg(wl, device, b_loc, sched=args.sched))
            fill_weights([p.data for p in layer.xfc_weight], wl.dim, seed=0)
        handle = layer._handle
        n_rows = layer.num_labels
        step_fn = lambda x, lab: layer.xfc_forward_backward(x, lab, [wl.lr], skip_loss=True)
        grad_of = lambda: layer.grad_input
    else:
        # label rows padded so that every rank owns a multiple of 16 rows
        n_rows = (L_true(wl) + 16 * world - 1) // (16 * world) * (16 * world)
        lo, hi = shard_bounds(n_rows, world)[rank]
        w = torch.empty(hi - lo, wl.dim, dtype=torch.float8_e4m3fn, device=device)
        fill_weights([w], wl.dim, seed=rank)
        engine = CudaShardEngine(device, wl.dim, B, wl.mode, lo, [w], sched_labels=args.sched)
        cap = b_loc * 64
        layer = LabelShardedXMC(engine, dim=wl.dim, local_batch=b_loc, num_rows=n_rows, label_capacity=cap,
                                device=device, base_seed=1234, rounding=wl.rounding)
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
    l0 = handle.launch_count
    with ClockSampler(local_rank) as clk:
        ms = timed(step_resident, args.steps, args.warmup, world, device)
    launches = (handle.launch_count - l0) * args.steps // (args.steps + args.warmup)
    ms_e2e = timed(step_e2e, args.steps, max(3, args.warmup), world, device)
    handle.check()

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
    # DRAM bytes per label row of one launch (dram__bytes_read.sum + dram__bytes_write.sum of an ncu
    # capture of a 65 536-row chunk at batch 512, d 768: profiles/step_kernels_small_case.md); traffic
    # grows with the rows a launch processes, so it is scaled to this run's rows per launch
    dram_per_row = {"update": 133.8e6 / 65536, "grad_x": 159.1e6 / 65536, "forward": 69.3e6 / 65536}
    rows_per_launch = (L / world) / max(dom_launches, 1.0)
    traffic = dram_per_row[dominant] * rows_per_launch if (wl.dim == 768 and b_loc * world == 512) else None
    fp8_dom = dominant == "forward" and wl.mode == "fp8"
    peak = pk["bf16_sustained"] * (2.0 if fp8_dom else 1.0)
    step_ms = ms / args.steps
    total_flops = 6.0 * B * L * wl.dim
    out = {
        "metric": METRIC, "value": B * args.steps / (ms * 1e-3), "unit": UNIT, "n_gpus": world,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": step_ms, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None,
        "dtype": "e4m3 weights; forward e4m3 x e4m3, backward bf16 x bf16, fp32 accumulate",
        "data": "synthetic",
        "config": {"workload": f"{wl.name}: W[{L}x{wl.dim}] e4m3 (padded to {n_rows} rows per rank-set), "
                               f"X[{B}x{wl.dim}] bf16, Poisson({wl.poisson:g}) positives/row, Zipf({wl.zipf_s}) ids, "
                               f"stochastic-rounding SGD lr={wl.lr}, skip-loss on",
                   "labels": L, "dim": wl.dim, "global_batch": B, "parallelism": f"label-shard x{world}",
                   "l2": "inputs larger than L2 (weights %.0f MB per GPU stream through every step)" % (L * wl.dim / world / 1e6),
                   "input_pool": n_pool},
        "clocks": clk.summary(),
        "e2e": {"value": B * args.steps / (ms_e2e * 1e-3), "unit": UNIT,
                "h2d_bytes_per_step": int(sum(x.numel() * 2 + l.numel() * 4 for x, l in pool) / n_pool),
                "d2h_bytes_per_step": int(host_grad[0].numel() * 2)},
        "gpu_launches": int(launches),
        "roofline": {"bound": "tensor", "kernel": dominant, "achieved": achieved, "peak": peak, "unit": "TFLOP/s",
                     "frac": achieved / peak, "traffic": traffic,
                     "traffic_note": "DRAM bytes per launch, ncu capture of a 65536-row chunk scaled by rows per launch",
                     "peak_source": pk["source"] + (" bf16 sustained x2 (no measured fp8 figure)" if fp8_dom
                                                    else " bf16 sustained"),
                     "launches_per_step": dom_launches, "ms_per_step": dom_ms},
        "kernel_ms_per_step": per_step,
        "step_tflops": total_flops / (step_ms * 1e-3) / 1e12,
        "peak_hbm_gb_per_gpu": peak_hbm,
    }
    if world == 1 and not args.no_cpu:
        cpu, _ = cpu_step_sample(wl, 8192, reps_budget_s=12.0)
        out["cpu_baseline"] = cpu
    print(json.dumps(out))


def run_topk(args, wl):
    """``--pass topk``: the fused logits + top-k inference pass over the same layer (single GPU, one
    line of its own; the default run never comes here)."""
    assert torch.cuda.is_available(), "bench.py needs a CUDA device (sm_100a); there is no CPU fallback"
    device = torch.device("cuda", 0)
    torch.cuda.set_device(device)
    from elmo_b200.xmc_classifiers import Fp8XMCBCEChunkedLayer
    layer = Fp8XMCBCEChunkedLayer(layer_cfg(wl, device, wl.batch, sched=args.sched))
    fill_weights([p.data for p in layer.xfc_weight], wl.dim, seed=0)
    gen = torch.Generator().manual_seed(5)
    xs = [synth.make_embeddings(wl.batch, wl.dim, gen).to(device) for _ in range(4)]
    k = args.topk
    for i in range(max(3, args.warmup)):
        layer.xfc_topk(xs[i % 4], k)
    torch.cuda.synchronize(device)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(args.steps):
        vals, idx = layer.xfc_topk(xs[i % 4], k)
    e1.record()
    torch.cuda.synchronize(device)
    layer._handle.check()
    ms = e0.elapsed_time(e1) / args.steps
    flops = 2.0 * wl.batch * wl.num_labels * wl.dim
    pk = peaks()
    print(json.dumps({
        "metric": "xmc_layer_topk_samples_per_sec", "value": wl.batch / (ms * 1e-3), "unit": UNIT, "n_gpus": 1,
        "steps": args.steps, "warmup": max(3, args.warmup), "ms_per_step": ms, "higher_is_better": True,
        "dtype": "e4m3 x e4m3, fp32 accumulate, bf16 logits", "data": "synthetic",
        "config": {"workload": f"{wl.name}: top-{k} of W[{wl.num_labels}x{wl.dim}] e4m3 for X[{wl.batch}x{wl.dim}] bf16",
                   "l2": "weights larger than L2"},
        "roofline": {"bound": "tensor", "kernel": "top-k", "achieved": flops / (ms * 1e-3) / 1e12,
                     "peak": pk["bf16_sustained"] * 2.0, "unit": "TFLOP/s",
                     "frac": flops / (ms * 1e-3) / 1e12 / (pk["bf16_sustained"] * 2.0), "traffic": None,
                     "peak_source": pk["source"] + " bf16 sustained x2 (no measured fp8 figure)"}}))


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
    if args.impl == "reference":
        run_reference(args, wl, rank, world)
    elif args.which == "topk":
        if world == 1:
            run_topk(args, wl)
        elif rank == 0:
            print(json.dumps({"metric": "xmc_layer_topk_samples_per_sec", "unavailable": "--pass topk is a single-GPU line"}))
    else:
        run_ours(args, wl, rank, local_rank, world)


if __name__ == "__main__":
    main()
