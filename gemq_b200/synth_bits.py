"""Per-expert bit-width draws of the synthetic benchmark layers (no device code: the CPU arm of
the benchmark imports this without loading the CUDA library)."""
from __future__ import annotations

import torch


def draw_expert_bits(n_experts: int, seed: int, lo: float = 1.5, hi: float = 2.5):
    """Per-expert bit-widths from {1,2,3,4} whose mean lies in [lo, hi]."""
    g = torch.Generator().manual_seed(seed)
    while True:
        bits = torch.randint(1, 5, (n_experts,), generator=g).tolist()
        if lo <= sum(bits) / n_experts <= hi:
            return bits
