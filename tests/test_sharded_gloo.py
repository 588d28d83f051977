"""World-size-2 CPU (gloo) test of the label-sharding plumbing: gather of embeddings and padded
labels, shard-local step (the CPU oracle stands in for the CUDA engine), reduce-scatter of grad_X.
The sharded result must equal the unsharded oracle step."""
import os
import socket

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from elmo_b200.sharded import LabelShardedXMC, pad_labels, shard_bounds

L, D, B_LOC, WORLD = 416, 32, 8, 2


class OracleEngine:
    def __init__(self, weights, label_offset):
        self.weights, self.label_offset = weights, label_offset

    def step(self, x, labels, lr, seed, step, stochastic, grad_f32, compute_loss=False, loss_out=None):
        from oracle import xmc_oracle as O
        new, gx, _ = O.fp8_chunked_step(self.weights, x, labels, lr, rounding="sr" if stochastic else "rn",
                                        seed=seed, step=step, label_offset=self.label_offset)
        for w, n in zip(self.weights, new):
            w.copy_(n)
        grad_f32.copy_(gx)

    def topk(self, x, k, n_out):
        from oracle import xmc_oracle as O
        v, i = O.topk_logits([w[:n_out] for w in self.weights], x, k)
        return v, (i + self.label_offset).to(torch.int32)


def _data():
    g = torch.Generator().manual_seed(0)
    w = (torch.randn(L, D, generator=g) * 0.25).to(torch.float8_e4m3fn)
    xs, labs = [], []
    for r in range(WORLD):
        xs.append((torch.randn(B_LOC, D, generator=g) / D ** 0.5).to(torch.bfloat16))
        n = 5 + 3 * r
        labs.append(torch.stack([torch.randint(0, B_LOC, (n,), generator=g),
                                 torch.randint(0, L, (n,), generator=g)], 1).to(torch.int32))
    return w, xs, labs


def _worker(rank, port, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=WORLD)
    try:
        w, xs, labs = _data()
        lo, hi = shard_bounds(L, WORLD)[rank]
        mine = [w[lo:hi].clone()]
        layer = LabelShardedXMC(OracleEngine(mine, lo), dim=D, local_batch=B_LOC, num_rows=L,
                                label_capacity=16, base_seed=9, rounding="sr")
        layer.xfc_forward_backward(xs[rank], labs[rank], [0.5])
        layer.prefetch_labels(labs[rank])                       # second step: labels gathered ahead of the "encoder"
        layer.xfc_forward_backward(xs[rank], None, [0.5])
        tv, ti = layer.xfc_topk(xs[rank], 4, L - 7)
        # checkpoint: per-rank state with its shard map, and the gathered reference layout (3 chunks)
        sd = layer.state_dict()
        ref_chunks = layer.export_reference_layout(L - 7, 3)
        twin_w = [torch.zeros_like(mine[0])]
        twin = LabelShardedXMC(OracleEngine(twin_w, lo), dim=D, local_batch=B_LOC, num_rows=L,
                               label_capacity=16, base_seed=0, rounding="rn")
        twin.load_state_dict(sd)
        ok_sd = torch.equal(twin_w[0].view(torch.uint8), mine[0].view(torch.uint8)) and twin.iteration == 2 \
            and twin.base_seed == 9 and twin.rounding == "sr"
        twin_w[0].view(torch.uint8).zero_()
        twin.import_reference_layout(ref_chunks)
        n_keep = max(0, min(hi, sum(c.shape[0] for c in ref_chunks)) - lo)
        ok_imp = torch.equal(twin_w[0].view(torch.uint8)[:n_keep], mine[0].view(torch.uint8)[:n_keep])
        bad_map = dict(sd, shard_map=dict(sd["shard_map"], world=3))
        try:
            twin.load_state_dict(bad_map)
            ok_rej = False
        except ValueError:
            ok_rej = True
        out[rank] = (mine[0].view(torch.uint8).clone(), layer.grad_input.float().clone(), tv.clone(), ti.clone(),
                     [c.view(torch.uint8).clone() for c in ref_chunks], bool(ok_sd and ok_imp and ok_rej))
    finally:
        dist.destroy_process_group()


def test_two_rank_sharded_step_equals_unsharded():
    from oracle import xmc_oracle as O
    s = socket.socket(); s.bind(("127.0.0.1", 0)); port = s.getsockname()[1]; s.close()
    mgr = mp.Manager()
    out = mgr.dict()
    mp.spawn(_worker, args=(port, out), nprocs=WORLD, join=True)
    w, xs, labs = _data()
    x = torch.cat(xs)
    lab = torch.cat([torch.stack([l[:, 0] + r * B_LOC, l[:, 1]], 1) for r, l in enumerate(labs)]).to(torch.int32)
    chunks = [w]
    for it in range(2):
        chunks, gx, _ = O.fp8_chunked_step(chunks, x, lab, 0.5, rounding="sr", seed=9, step=it)
    full = chunks[0].view(torch.uint8)
    for r, (lo, hi) in enumerate(shard_bounds(L, WORLD)):
        w_r, g_r, tv, ti, ref_chunks, ok_ckpt = out[r]
        assert torch.equal(w_r, full[lo:hi])
        assert ok_ckpt
        # the exported list has the reference's padded geometry and holds the unsharded weights
        lp, li = O.fp8_padded_labels(L - 7, 3)
        assert len(ref_chunks) == 3 and all(c.shape == (li, D) for c in ref_chunks)
        cat = torch.cat(ref_chunks)
        n = min(lp, L)
        assert torch.equal(cat[:n], full[:n]) and int(cat[n:].sum()) == 0
        want = gx[r * B_LOC:(r + 1) * B_LOC].to(torch.bfloat16).float()
        assert torch.allclose(g_r, want, rtol=2e-2, atol=1e-6)
        # sharded top-k (after the two steps) == top-k of the unsharded updated weights
        wv, wi = O.topk_logits([chunks[0][:L - 7]], xs[r], 4)
        assert torch.equal(tv, wv) and torch.equal(ti.long(), wi.long())


def test_pad_labels_and_bounds():
    lab = torch.tensor([[1, 7], [2, 9]], dtype=torch.int32)
    p = pad_labels(lab, 4, 10, "cpu")
    assert p.tolist() == [[11, 7], [12, 9], [0, 2 ** 31 - 1], [0, 2 ** 31 - 1]]
    assert pad_labels(None, 2, 0, "cpu")[:, 1].tolist() == [2 ** 31 - 1] * 2
    b = shard_bounds(670208, 8)
    assert b[0][0] == 0 and b[-1][1] == 670208 and all(lo % 16 == 0 for lo, _ in b)
    assert all(b[i][1] == b[i + 1][0] for i in range(7))
    assert shard_bounds(100, 8)[-1] == (100, 100)          # trailing ranks may own nothing
