"""Seeded synthetic inputs with the shapes and value distributions of the XMC benchmarks the
reference trains on (the datasets themselves are not redistributable here): embeddings
N(0,1)/sqrt(d), weights U(+-1/sqrt(d)), sparse multi-hot targets with Poisson-many positives per
row and bounded-Zipf label ids (rank = id, so low ids are head labels).  Everything is drawn on the
CPU from one ``torch.Generator`` so that CPU and GPU runs see identical inputs."""
from dataclasses import dataclass
from typing import Optional, Tuple

import numpy as np
import torch


@dataclass
class Workload:
    name: str
    num_labels: int
    dim: int
    batch: int
    chunk_labels: int          # labels per reference chunk
    mode: str                  # 'bf16' | 'fp8' | 'simfp8'
    poisson: float
    clip: Tuple[int, int]
    zipf_s: float
    rounding: str              # 'rn' | 'sr'
    lr: float = 0.05

    @property
    def num_chunks(self) -> int:
        return (self.num_labels + self.chunk_labels - 1) // self.chunk_labels


WORKLOADS = {
    # BF16 chunked step, CPU-runnable reference case
    "cfg1": Workload("cfg1", 131072, 768, 256, 32768, "bf16", 5.0, (1, 20), 1.1, "rn"),
    # FP8 chunked step on one GPU: the configuration the headline metric is quoted on
    "cfg2": Workload("cfg2", 670091, 768, 512, 65536, "fp8", 5.0, (1, 10 ** 9), 1.1, "sr"),
    # simulated FP8
    "cfg3": Workload("cfg3", 500000, 768, 256, 50000, "simfp8", 20.0, (1, 100), 1.0, "rn"),
    # label-sharded steps
    "cfg4": Workload("cfg4", 2812281, 768, 1024, 351536, "fp8", 30.0, (1, 200), 1.05, "sr"),
    "cfg5": Workload("cfg5", 8623847, 768, 2048, 131072, "fp8", 8.0, (1, 10 ** 9), 1.2, "sr"),
}


def make_embeddings(batch: int, dim: int, gen: torch.Generator) -> torch.Tensor:
    return (torch.randn(batch, dim, generator=gen) / dim ** 0.5).to(torch.bfloat16)


def make_weights_f32(rows: int, dim: int, gen: torch.Generator) -> torch.Tensor:
    return (torch.rand(rows, dim, generator=gen) * 2 - 1) / dim ** 0.5


class ZipfSampler:
    """p(id = k-1) proportional to k^-s for k = 1..L, sampled by inverse CDF (float64 table)."""

    def __init__(self, num_labels: int, s: float):
        w = np.arange(1, num_labels + 1, dtype=np.float64) ** (-s)
        self.cdf = np.cumsum(w)
        self.cdf /= self.cdf[-1]
        self.num_labels = num_labels

    def sample(self, n: int, gen: torch.Generator) -> np.ndarray:
        u = torch.rand(n, generator=gen, dtype=torch.float64).numpy()
        return np.minimum(np.searchsorted(self.cdf, u, side="right"), self.num_labels - 1)


def make_labels(batch: int, sampler: ZipfSampler, poisson: float, clip: Tuple[int, int],
                gen: torch.Generator, row_offset: int = 0) -> torch.Tensor:
    """int32 COO [nnz, 2] = (batch row, label id), rows ascending, ids de-duplicated within a row
    (duplicates are dropped, so a row may end up with fewer positives than drawn)."""
    counts = torch.poisson(torch.full((batch,), float(poisson)), generator=gen).clamp_(clip[0], clip[1]).long()
    ids = sampler.sample(int(counts.sum()), gen)
    rows = np.repeat(np.arange(batch, dtype=np.int64), counts.numpy())
    pairs = np.unique(np.stack([rows, ids], 1), axis=0)           # sorts by (row, id), drops duplicates
    pairs[:, 0] += row_offset
    return torch.from_numpy(pairs.astype(np.int32))


def make_step_inputs(wl: Workload, seed: int = 0, batch: Optional[int] = None,
                     sampler: Optional[ZipfSampler] = None):
    """(X bf16 [B, d], labels int32 [nnz, 2]) for one step of workload ``wl``."""
    gen = torch.Generator().manual_seed(seed)
    b = batch or wl.batch
    sampler = sampler or ZipfSampler(wl.num_labels, wl.zipf_s)
    x = make_embeddings(b, wl.dim, gen)
    labels = make_labels(b, sampler, wl.poisson, wl.clip, gen)
    return x, labels
