"""Fused gate/up and down projections of the selected experts for one token; same call
signatures as gemq/triton_kernels/fused_dequant_bmm.py."""
from __future__ import annotations

import ctypes
from typing import Tuple

import torch
from torch import Tensor

from .. import _capi
from ._ops import library_op
from ._runtime import gemv_workspace, require, require_cuda, stream_ptr


def _check_stacked(w, s, z, nbits, strides):
    require(w.dtype == torch.int32 and w.is_contiguous(), "stacked weights must be contiguous int32")
    require(s.dtype == torch.float16 and s.is_contiguous() and z.dtype == torch.float16 and z.is_contiguous(),
            "stacked scales / zeros must be contiguous float16")
    require(nbits.dtype == torch.int32 and strides.dtype == torch.int32, "nbits / strides must be int32")


def _fake_up(x, idx, w1, w3, w1_scales, w1_zeros, w3_scales, w3_zeros, nbits, w_strides, group_size):
    n = idx.shape[0] * w1.shape[1]
    return x.new_empty((1, n), dtype=torch.float16), x.new_empty((1, n), dtype=torch.float16)


@library_op("fused_dequant_up_proj", _fake_up)
def fused_dequant_up_proj(x: Tensor, idx: Tensor, w1: Tensor, w3: Tensor,
                          w1_scales: Tensor, w1_zeros: Tensor, w3_scales: Tensor, w3_zeros: Tensor,
                          nbits: Tensor, w_strides: Tensor, group_size: int) -> Tuple[Tensor, Tensor]:
    """``x1, x3 [1, A*N]``: ``x @ deq(w1[e])`` and ``x @ deq(w3[e])`` for ``e`` in ``idx``
    (gemq/triton_kernels/fused_dequant_bmm.py:122-173)."""
    dev = require_cuda(x, idx, w1, w3, w1_scales, w1_zeros, w3_scales, w3_zeros, nbits, w_strides)
    require(x.dim() == 2 and x.shape[0] == 1 and x.dtype == torch.float16, "x must be float16 [1, K]")
    require(idx.dtype == torch.int64 and idx.dim() == 1, "idx must be int64 [A]")
    _check_stacked(w1, w1_scales, w1_zeros, nbits, w_strides)
    _check_stacked(w3, w3_scales, w3_zeros, nbits, w_strides)
    K = x.shape[1]
    N = w1.shape[1]
    A = idx.shape[0]
    x = x.contiguous()
    x1 = torch.empty((1, A * N), dtype=torch.float16, device=dev)
    x3 = torch.empty((1, A * N), dtype=torch.float16, device=dev)
    ws = gemv_workspace(dev, 2 * A * N, K, 1)
    s1 = _capi.stacked(w1, w1_scales, w1_zeros, nbits, w_strides)
    s3 = _capi.stacked(w3, w3_scales, w3_zeros, nbits, w_strides)
    _capi.check("gemq_fused_up_proj", _capi.lib.gemq_fused_up_proj(
        x.data_ptr(), idx.data_ptr(), A, ctypes.byref(s1), ctypes.byref(s3), x1.data_ptr(), x3.data_ptr(),
        N, K, group_size, ws.data_ptr(), ws.numel(), stream_ptr(dev)))
    return x1, x3


@library_op("fused_dequant_down_proj",
            lambda x1, x3, idx, w2, w2_scales, w2_zeros, nbits, w_strides, group_size:
            x1.new_empty((1, idx.shape[0] * w2.shape[1]), dtype=torch.float16))
def fused_dequant_down_proj(x1: Tensor, x3: Tensor, idx: Tensor, w2: Tensor,
                            w2_scales: Tensor, w2_zeros: Tensor, nbits: Tensor, w_strides: Tensor,
                            group_size: int) -> Tensor:
    """``x2 [1, A*N]``: ``(silu(x1[a]) * x3[a]) @ deq(w2[idx[a]])``
    (gemq/triton_kernels/fused_dequant_bmm.py:264-312)."""
    dev = require_cuda(x1, x3, idx, w2, w2_scales, w2_zeros, nbits, w_strides)
    require(x1.shape == x3.shape and x1.dim() == 2 and x1.shape[0] == 1, "x1 / x3 must be [1, A*K]")
    require(x1.dtype == torch.float16 and x3.dtype == torch.float16, "x1 / x3 must be float16")
    require(idx.dtype == torch.int64 and idx.dim() == 1, "idx must be int64 [A]")
    _check_stacked(w2, w2_scales, w2_zeros, nbits, w_strides)
    A = idx.shape[0]
    require(x1.shape[1] % A == 0, "x1 length must be a multiple of len(idx)")
    K = x1.shape[1] // A
    N = w2.shape[1]
    x1 = x1.contiguous()
    x3 = x3.contiguous()
    x2 = torch.empty((1, A * N), dtype=torch.float16, device=dev)
    ws = gemv_workspace(dev, A * N, K, 1)
    s2 = _capi.stacked(w2, w2_scales, w2_zeros, nbits, w_strides)
    _capi.check("gemq_fused_down_proj", _capi.lib.gemq_fused_down_proj(
        x1.data_ptr(), x3.data_ptr(), idx.data_ptr(), A, ctypes.byref(s2), x2.data_ptr(), N, K, group_size,
        ws.data_ptr(), ws.numel(), stream_ptr(dev)))
    return x2


fused_dequant_up_proj_triton = fused_dequant_up_proj
fused_dequant_down_proj_triton = fused_dequant_down_proj
