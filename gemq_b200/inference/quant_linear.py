"""A quantised ``nn.Linear`` replacement on the MoE kernels.

The reference quantises attention and dense-MLP linears to 4 bits (``--attn_wbits 4
--dense_wbits 4``, gemq/quantize.py:333-343) and runs them with gemlite's kernels
(gemq/inference/patch.py:71-79).  The same packed format goes through this library's GEMV
(a few rows) and tcgen05 GEMM (32 rows or more) entry points, any bit width from 1 to 4.
"""
from __future__ import annotations

import torch
import torch.nn as nn
from torch import Tensor

from ..kernels import dequant_gemm
from .packed_linear import PackedLinear


class QuantLinear(nn.Module):
    def __init__(self, packed: PackedLinear, bias: Tensor = None):
        super().__init__()
        self.in_features, self.out_features = packed.in_features, packed.out_features
        self.W_nbits, self.group_size = packed.W_nbits, packed.group_size
        # plain attributes, like the reference's blocks keep their packed tensors
        self.W_q, self.scales, self.zeros = packed.W_q, packed.scales, packed.zeros
        self.bias = bias

    def forward(self, x: Tensor) -> Tensor:
        """``x [..., in]`` fp16 / bf16 -> ``[..., out]`` in the same dtype."""
        lead = x.shape[:-1]
        rows = x.reshape(-1, self.in_features)
        small = rows.shape[0] < 32 and rows.dtype != torch.float16
        y = dequant_gemm(rows.to(torch.float16) if small else rows, self.W_q, self.scales, self.zeros, self.W_nbits,
                         self.group_size)
        y = y.to(x.dtype)
        if self.bias is not None:
            y = y + self.bias.to(y.dtype)
        return y.reshape(*lead, self.out_features)
