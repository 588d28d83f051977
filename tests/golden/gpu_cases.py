"""Seeded CPU inputs shared by tests/golden/make_golden_gpu.py (which feeds them to the reference's
Triton kernels on a GPU) and tests/test_oracle_golden_gpu.py (which replays the stored outputs).
Large inputs are regenerated from their seed instead of being stored; the fixture keeps their
sha256 so that a drift of the CPU generator is reported rather than misread as a parity failure."""
import hashlib

import torch

E4M3 = torch.float8_e4m3fn

# (tag, k, m, n): C[m x n] = G[k x m]^T W[k x n]; 'c' is the long-k case
LARGE_K_CASES = [("a", 1000, 48, 80), ("b", 4099, 64, 96), ("c", 70001, 16, 32)]


def digest(*tensors):
    h = hashlib.sha256()
    for t in tensors:
        t = t.detach().cpu().contiguous()
        h.update(t.view(torch.uint8).numpy().tobytes())
    return h.hexdigest()


def logit_gradient(g, rows, cols):
    """bf16 [rows x cols] with the distribution of sigmoid(z) - y: mostly in (0, 1), a few in (-1, 0)."""
    z = torch.randn(rows, cols, generator=g) * 2.0
    s = torch.sigmoid(z).to(torch.bfloat16)
    neg = torch.rand(rows, cols, generator=g) < 0.02
    return torch.where(neg, s - 1.0, s).to(torch.bfloat16)


def large_k_inputs(index):
    """(G bf16 [k x m], W e4m3 [k x n], W bf16 [k x n]) of LARGE_K_CASES[index]."""
    _, k, m, n = LARGE_K_CASES[index]
    g = torch.Generator().manual_seed(2100 + index)
    G = logit_gradient(g, k, m)
    w32 = (torch.rand(k, n, generator=g) * 2 - 1) * 0.25
    return G, w32.to(E4M3), w32.to(torch.bfloat16)


def update_inputs(g, m, n, k, w_kind):
    """(G bf16 [m x k], X bf16 [k x n], W fp32 [m x n]) for the fused update kernels."""
    G = logit_gradient(g, m, k)
    X = (torch.randn(k, n, generator=g) / 768 ** 0.5).to(torch.bfloat16)
    sign = lambda: torch.where(torch.rand(m, n, generator=g) < 0.5, -1.0, 1.0)
    if w_kind == "small":            # U(+-1/sqrt(768)): e4m3 sub-normals and the lowest normal binades
        w = (torch.rand(m, n, generator=g) * 2 - 1) / 768 ** 0.5
    elif w_kind == "wide":           # log-uniform magnitudes over 2^-10 .. 2^7
        w = torch.exp2(torch.rand(m, n, generator=g) * 17.0 - 10.0) * sign()
    else:                            # at the top of the e4m3 range: the update crosses +-448
        w = torch.where(torch.rand(m, n, generator=g) < 0.5, 448.0, 416.0) * sign()
    return G, X, w


def make_labels(g, B, L, per_row):
    rows, cols = [], []
    for r in range(B):
        n = int(torch.randint(1, per_row + 1, (1,), generator=g))
        c = torch.randint(0, L, (n,), generator=g)
        c = torch.where(torch.rand(n, generator=g) < 0.3, c % 7, c)       # head-heavy ids
        rows += [r] * n
        cols += c.tolist()
        if r % 5 == 0:                                                     # a duplicated pair now and then
            rows.append(r); cols.append(cols[-1])
    return torch.tensor(list(zip(rows, cols)), dtype=torch.int32)
