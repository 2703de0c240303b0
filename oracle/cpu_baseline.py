"""Timed CPU baseline: the reference-convention torch path on the host cores.

TEST / BENCHMARK INFRASTRUCTURE ONLY.  unpack int32 words -> codes
(gemq/triton_kernels/utils.py:116-146), ``W = q * scale + offset``
(gemq/triton_kernels/utils.py:206-210), fp32 ``torch.matmul``, SiLU*mul and the down
projection as in gemq/inference/moe_block.py:146-163 / :200-235.  Multi-threaded through
torch's intra-op pool; ``torch.get_num_threads()`` is the core count to report.
"""
from __future__ import annotations

import time

import torch
import torch.nn.functional as F


def unpack_kernel_form_torch(wq: torch.Tensor, nbits: int, K: int) -> torch.Tensor:
    eps = 32 // nbits
    shifts = (torch.arange(eps, dtype=torch.int32) * nbits).view(1, eps, 1)
    q = (wq.unsqueeze(1) >> shifts) & ((1 << nbits) - 1)
    return q.reshape(-1, wq.shape[1])[:K]


def dequant_matmul(x: torch.Tensor, wq, scales, zeros, nbits: int, group: int) -> torch.Tensor:
    """``x[M,K] (fp32) @ deq(wq)`` with the weights de-quantised on every call."""
    K = x.shape[1]
    q = unpack_kernel_form_torch(wq, nbits, K).to(torch.float32)
    w = q * scales.float().repeat_interleave(group, 0) + zeros.float().repeat_interleave(group, 0)
    return x @ w


def expert_ffn(x: torch.Tensor, w1, w3, w2, nbits: int, group: int) -> torch.Tensor:
    """One expert: ``w?`` = (wq, scales, zeros) CPU tensors."""
    x1 = dequant_matmul(x, *w1, nbits, group).half().float()
    x3 = dequant_matmul(x, *w3, nbits, group).half().float()
    return dequant_matmul(F.silu(x1) * x3, *w2, nbits, group).half()


def time_best(fn, repeats: int = 3, warmup: int = 1) -> float:
    for _ in range(warmup):
        fn()
    best = float("inf")
    for _ in range(repeats):
        t = time.perf_counter()
        fn()
        best = min(best, time.perf_counter() - t)
    return best
