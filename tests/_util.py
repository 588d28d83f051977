"""Shared helpers for the tests: golden-fixture decoding and comparison metrics."""
import os

import numpy as np
import torch

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def load_golden(name):
    return np.load(os.path.join(GOLDEN, name))


def as_bf16(a):
    return torch.from_numpy(np.ascontiguousarray(a)).view(torch.bfloat16)


def as_e4m3(a):
    return torch.from_numpy(np.ascontiguousarray(a)).view(torch.float8_e4m3fn)


def rel_inf(a, b):
    """||a-b||_inf / ||b||_inf"""
    a = a.to(torch.float64); b = b.to(torch.float64)
    return float((a - b).abs().max() / b.abs().max().clamp_min(1e-30))


def frac_equal_bits(a, b):
    """fraction of elements with identical bit patterns (a, b same narrow dtype)."""
    n = a.numel()
    if a.element_size() == 1:
        return float((a.view(torch.uint8) == b.view(torch.uint8)).sum()) / n
    return float((a.view(torch.int16) == b.view(torch.int16)).sum()) / n


def e4m3_ulp_distance(a, b):
    """max distance in e4m3 grid steps between two e4m3 tensors (sign-magnitude ordering)."""
    def key(t):
        u = t.view(torch.uint8).to(torch.int32)
        mag = u & 0x7F
        return torch.where(u >= 128, -mag, mag)
    return int((key(a) - key(b)).abs().max())
