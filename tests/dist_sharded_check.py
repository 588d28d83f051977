"""Multi-GPU parity check of the label-sharded layer (run under torch.distributed.run, one rank per
GPU): the sharded CUDA step and the sharded top-k must equal the CPU oracle on the unsharded layer.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 2 --master-addr 127.0.0.1 \
        --master-port 29533 tests/dist_sharded_check.py
"""
import os
import sys

import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

from elmo_b200.sharded import CudaShardEngine, LabelShardedXMC, shard_bounds  # noqa: E402
from oracle import xmc_oracle as O  # noqa: E402


def run_check(dev, rank, world):
    """Sharded CUDA layer vs the CPU oracle on the unsharded problem, inside an initialised process group.
    Returns {"w_bit_exact", "grad_x_rel", "topk_value_err", "ok"} reduced over all ranks (worst case)."""
    L, d, b_loc, k = 4000 - 16, 128, 48, 7
    g = torch.Generator().manual_seed(0)
    w = (torch.randn(L, d, generator=g) * 0.25).to(torch.float8_e4m3fn)
    xs = [(torch.randn(b_loc, d, generator=g) / d ** 0.5).to(torch.bfloat16) for _ in range(world)]
    labs = []
    for r in range(world):
        n = 150 + 10 * r
        labs.append(torch.stack([torch.randint(0, b_loc, (n,), generator=g),
                                 torch.randint(0, L, (n,), generator=g)], 1).to(torch.int32))
    lo, hi = shard_bounds(L, world)[rank]
    mine = [w[lo:hi].clone().to(dev)]
    eng = CudaShardEngine(dev, d, b_loc * world, "fp8", lo, mine, sched_labels=512)
    layer = LabelShardedXMC(eng, dim=d, local_batch=b_loc, num_rows=L, label_capacity=256, device=dev,
                            base_seed=77, rounding="sr")
    layer.xfc_forward_backward(xs[rank].to(dev), labs[rank].to(dev), [0.4])
    layer.prefetch_labels(labs[rank].to(dev))                   # second step: labels gathered on the side stream
    layer.xfc_forward_backward(xs[rank].to(dev), None, [0.4])
    tv, ti = layer.xfc_topk(xs[rank].to(dev), k, L - 5)
    eng.handle.check()

    # oracle on the unsharded problem
    x = torch.cat(xs)
    lab = torch.cat([torch.stack([l[:, 0] + r * b_loc, l[:, 1]], 1) for r, l in enumerate(labs)]).to(torch.int32)
    chunks = [w]
    for it in range(2):
        chunks, gx, _ = O.fp8_chunked_step(chunks, x, lab, 0.4, rounding="sr", seed=77, step=it)
    same = float((mine[0].cpu().view(torch.uint8) == chunks[0][lo:hi].view(torch.uint8)).float().mean()) if hi > lo else 1.0
    gwant = gx[rank * b_loc:(rank + 1) * b_loc]
    gerr = float((layer.grad_input.float().cpu() - gwant).abs().max() / gwant.abs().max())
    wv, wi = O.topk_logits([chunks[0][:L - 5]], xs[rank], k)
    z = O.forward_logits([chunks[0]], xs[rank], num_labels=L - 5).float()
    ulp = float(z.abs().max()) * 2.0 ** -7
    verr = float((tv.cpu() - wv).abs().max())
    ok = same >= 0.999 and gerr < 1e-2 and verr <= ulp and int(ti.min()) >= 0 and int(ti.max()) < L - 5
    red = torch.tensor([same, -gerr, -verr, 1.0 if ok else 0.0], device=dev, dtype=torch.float64)
    dist.all_reduce(red, op=dist.ReduceOp.MIN)
    eng.handle.close()
    return {"w_bit_exact": float(red[0]), "grad_x_rel": float(-red[1]), "topk_value_err": float(-red[2]),
            "ok": bool(red[3] > 0.5), "ranks": world,
            "case": f"{L} labels x {d}, batch {b_loc} per rank, 2 SR steps + top-{k}, vs the CPU oracle unsharded"}


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", rank)))
    torch.cuda.set_device(dev)
    dist.init_process_group("nccl", device_id=dev)
    res = run_check(dev, rank, world)
    print(f"rank {rank}: W' bit-exact {res['w_bit_exact']:.5f}, grad_X rel err {res['grad_x_rel']:.2e}, "
          f"top-k value err {res['topk_value_err']:.2e} -> {'ok' if res['ok'] else 'FAIL'}", flush=True)
    dist.barrier()
    dist.destroy_process_group()
    sys.exit(0 if res["ok"] else 1)


if __name__ == "__main__":
    main()
