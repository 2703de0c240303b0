"""Dequant-fused GEMV; same call signatures as gemq/triton_kernels/dequant_gemv.py."""
from __future__ import annotations

import ctypes

import torch
from torch import Tensor

from .. import _capi
from ._ops import library_op
from ._runtime import check_kernel_form, gemv_workspace, require, require_cuda, stream_ptr


def _fake_rows(x, w_q, scales, zeros, nbits, group_size):
    return x.new_empty((x.shape[0], w_q.shape[1]), dtype=torch.float16)


@library_op("dequant_gemv_rows", _fake_rows)
def dequant_gemv_rows(x: Tensor, w_q: Tensor, scales: Tensor, zeros: Tensor, nbits: int, group_size: int) -> Tensor:
    """``x[M, K] @ deq(w_q)`` for a few rows (decode batch); fp16 in, fp16 out."""
    dev = require_cuda(x, w_q, scales, zeros)
    require(x.dim() == 2 and x.dtype == torch.float16, "x must be float16 [M, K]")
    M, K = x.shape
    N = w_q.shape[1]
    check_kernel_form(w_q, scales, zeros, K, N, nbits, group_size)
    x = x if x.stride(1) == 1 else x.contiguous()
    out = torch.empty((M, N), dtype=torch.float16, device=dev)
    ws = gemv_workspace(dev, N, K, M)
    _capi.check("gemq_dequant_gemv", _capi.lib.gemq_dequant_gemv(
        x.data_ptr(), x.stride(0), w_q.data_ptr(), scales.data_ptr(), zeros.data_ptr(),
        out.data_ptr(), N, M, N, K, nbits, group_size, ws.data_ptr(), ws.numel(), stream_ptr(dev)))
    return out


@library_op("dequant_splitk_gemv", _fake_rows)
def dequant_splitk_gemv(x: Tensor, w_q: Tensor, scales: Tensor, zeros: Tensor, nbits: int, group_size: int) -> Tensor:
    """``output[1, N] = x[1, K] @ dequantize(w_q, scales, zeros)``
    (gemq/triton_kernels/dequant_gemv.py:118-156).  Unlike the reference's fp16 atomics the
    split-K sum is formed in a fixed order, so the result is reproducible."""
    require(x.dim() == 2 and x.shape[0] == 1, "dequant_splitk_gemv takes exactly one row (M == 1)")
    return dequant_gemv_rows._init_fn(x, w_q, scales, zeros, nbits, group_size)


@library_op("dequant_sel_splitk_gemv",
            lambda x, idx, w_q, scales, zeros, nbits, wq_strides, group_size:
            x.new_empty((1, w_q.shape[1]), dtype=torch.float16))
def dequant_sel_splitk_gemv(x: Tensor, idx: Tensor, w_q: Tensor, scales: Tensor, zeros: Tensor,
                            nbits: Tensor, wq_strides: Tensor, group_size: int) -> Tensor:
    """GEMV against expert ``idx[0]`` of stacked tensors (gemq/triton_kernels/dequant_gemv.py:225-270)."""
    dev = require_cuda(x, idx, w_q, scales, zeros, nbits, wq_strides)
    require(x.dim() == 2 and x.shape[0] == 1 and x.dtype == torch.float16, "x must be float16 [1, K]")
    require(idx.dtype == torch.int64 and idx.numel() >= 1, "idx must be an int64 tensor")
    require(nbits.dtype == torch.int32 and wq_strides.dtype == torch.int32, "nbits / wq_strides must be int32")
    require(w_q.dtype == torch.int32 and w_q.is_contiguous(), "w_q must be contiguous int32")
    require(scales.dtype == torch.float16 and zeros.dtype == torch.float16, "scales / zeros must be float16")
    K = x.shape[1]
    N = w_q.shape[1]
    x = x.contiguous()
    out = torch.empty((1, N), dtype=torch.float16, device=dev)
    ws = gemv_workspace(dev, N, K, 1)
    scales, zeros = scales.contiguous(), zeros.contiguous()
    st = _capi.stacked(w_q, scales, zeros, nbits, wq_strides)
    _capi.check("gemq_dequant_sel_gemv", _capi.lib.gemq_dequant_sel_gemv(
        x.data_ptr(), idx.data_ptr(), ctypes.byref(st), out.data_ptr(), N, K, group_size,
        ws.data_ptr(), ws.numel(), stream_ptr(dev)))
    return out


dequant_splitk_gemv_triton = dequant_splitk_gemv
dequant_sel_splitk_gemv_triton = dequant_sel_splitk_gemv
