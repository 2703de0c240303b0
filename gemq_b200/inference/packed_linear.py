"""A packed quantised linear layer as the MoE blocks expect to find it.

The reference blocks read ``W_q, scales, zeros, W_nbits, group_size`` from GemLite
linears (gemq/inference/moe_block.py:111-127).  Any object with these attributes works;
this class is the plain container used when no GemLite module is around.
"""
from __future__ import annotations

import torch

from ..kernels.utils import pack_kernel_form


class PackedLinear:
    def __init__(self, W_q: torch.Tensor, scales: torch.Tensor, zeros: torch.Tensor, W_nbits: int, group_size: int,
                 in_features: int, out_features: int):
        eps = 32 // W_nbits
        assert W_q.dtype == torch.int32 and tuple(W_q.shape) == (-(-in_features // eps), out_features)
        assert scales.shape == zeros.shape == (in_features // group_size, out_features)
        self.W_q, self.scales, self.zeros = W_q, scales, zeros
        self.W_nbits, self.group_size = int(W_nbits), int(group_size)
        self.in_features, self.out_features = in_features, out_features

    @classmethod
    def from_codes(cls, codes: torch.Tensor, scale: torch.Tensor, zero_point: torch.Tensor, W_nbits: int,
                   group_size: int) -> "PackedLinear":
        """From uint8 codes ``[out, in]`` and the quantiser's ``W = (Q - zero) * scale`` parameters
        (gemq/quantizers/gptq.py:446-450), both ``[in/group, out]``: the kernels take the additive
        offset ``-zero * scale`` (gemq/triton_kernels/utils.py:196)."""
        out_f, in_f = codes.shape
        offset = (-(zero_point.float() * scale.float())).to(torch.float16)
        return cls(pack_kernel_form(codes, W_nbits), scale.to(torch.float16).contiguous(), offset.contiguous(),
                   W_nbits, group_size, in_f, out_f)


def is_packed_linear(m) -> bool:
    return all(hasattr(m, a) for a in ("W_q", "scales", "zeros", "W_nbits", "group_size"))
