"""Pieces shared by the layer classes: config access with reference defaults, step plumbing."""
import torch

dtype_map = {'float16': torch.float16, 'bfloat16': torch.bfloat16, 'float32': torch.float32,
             'float8': torch.float8_e4m3fn}


def cfg_get(node, path, default):
    """``cfg.a.b.c`` with a default when any attribute is missing (the reference's config has no
    such key; new knobs default to the reference's behaviour)."""
    cur = node
    for name in path.split('.'):
        if cur is None or not hasattr(cur, name):
            return default
        cur = getattr(cur, name)
    return cur


def draw_base_seed() -> int:
    """One draw from torch's global CPU generator at construction, so ``torch.manual_seed``
    (src/main.py:61) still fixes the stochastic-rounding stream; the per-step counter replaces the
    reference's per-chunk host draw (chunked_fp8xmc_clf.py:113)."""
    return int(torch.randint(0, 2 ** 31 - 1, (1,)).item())


def as_labels(labels: torch.Tensor, device) -> torch.Tensor:
    if labels.dtype != torch.int32:
        labels = labels.to(torch.int32)
    if labels.device != device:
        labels = labels.to(device)
    return labels.contiguous()
