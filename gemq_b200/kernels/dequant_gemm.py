"""Dequant-fused GEMM; same call signature as gemq/triton_kernels/dequant_gemm.py."""
from __future__ import annotations

import torch
from torch import Tensor

from ._runtime import require
from .dequant_gemv import dequant_gemv_rows

_ROW_BLOCK = 64


def dequant_gemm(x: Tensor, w_q: Tensor, scales: Tensor, zeros: Tensor, nbits: int, group_size: int) -> Tensor:
    """``output[M, N] = x[M, K] @ dequantize(w_q, scales, zeros)``, fp16
    (gemq/triton_kernels/dequant_gemm.py:150-193).  Rows are processed eight at a time by the
    decode kernel, in calls of at most 64 rows to bound the split-K workspace."""
    require(x.dim() == 2, "x must be [M, K]")
    M = x.shape[0]
    if M <= _ROW_BLOCK:
        return dequant_gemv_rows(x, w_q, scales, zeros, nbits, group_size)
    return torch.cat([dequant_gemv_rows(x[i:i + _ROW_BLOCK], w_q, scales, zeros, nbits, group_size)
                      for i in range(0, M, _ROW_BLOCK)])


dequant_gemm_triton = dequant_gemm
