"""Grouped dequant GEMM over selected experts; same call signature as
gemq/triton_kernels/dequant_group_gemm.py."""
from __future__ import annotations

import ctypes

import torch
from torch import Tensor

from .. import _capi
from ._ops import library_op
from ._runtime import error_word, gemv_workspace, require, require_cuda, stream_ptr, tc_gemm_ok

_ROW_BLOCK = 64
_group_size_cache: dict = {}


def _uniform_group_size(group_sizes: Tensor) -> int:
    """The block-wide group size (gemq/inference/moe_block.py:130-134 asserts it is uniform).
    Read from the device once per tensor."""
    key = (group_sizes.data_ptr(), group_sizes.numel())
    g = _group_size_cache.get(key)
    if g is None:
        vals = torch.unique(group_sizes).tolist()
        require(len(vals) == 1, "Group sizes must be the same across all experts.")
        g = int(vals[0])
        _group_size_cache[key] = g
    return g


def dequant_group_gemm(x: Tensor, indices: Tensor, wq: Tensor, scales: Tensor, zeros: Tensor,
                       nbits: Tensor, group_sizes: Tensor, wq_strides: Tensor, zs_strides: Tensor,
                       compute_dtype=torch.float16) -> Tensor:
    """``output[g] = x @ dequantize(W[indices[g]])`` -> ``[A, M, N]``
    (gemq/triton_kernels/dequant_group_gemm.py:155-202)."""
    require(compute_dtype == torch.float16, "only float16 is supported, as in the reference kernel")
    return _group_gemm(x, indices, wq, scales, zeros, nbits, group_sizes, wq_strides, zs_strides)


@library_op("dequant_group_gemm",
            lambda x, indices, wq, scales, zeros, nbits, group_sizes, wq_strides, zs_strides:
            x.new_empty((indices.numel(), x.shape[0], wq.shape[1]), dtype=torch.float16))
def _group_gemm(x: Tensor, indices: Tensor, wq: Tensor, scales: Tensor, zeros: Tensor,
                nbits: Tensor, group_sizes: Tensor, wq_strides: Tensor, zs_strides: Tensor) -> Tensor:
    dev = require_cuda(x, indices, wq, scales, zeros, nbits, group_sizes, wq_strides, zs_strides)
    require(x.dim() == 2 and x.dtype == torch.float16, "x must be float16 [M, K]")
    require(indices.dtype == torch.int64, "indices must be int64")
    indices = indices.reshape(-1)
    require(wq.dtype == torch.int32 and wq.is_contiguous(), "wq must be contiguous int32")
    require(scales.dtype == torch.float16 and zeros.dtype == torch.float16, "scales / zeros must be float16")
    for t in (nbits, group_sizes, wq_strides, zs_strides):
        require(t.dtype == torch.int32, "metadata tensors must be int32")
    G = _uniform_group_size(group_sizes)
    M, K = x.shape
    N = wq.shape[1]
    A = indices.shape[0]
    x = x if x.stride(1) == 1 else x.contiguous()
    scales = scales.contiguous()
    zeros = zeros.contiguous()
    out = torch.empty((A, M, N), dtype=torch.float16, device=dev)
    if tc_gemm_ok(M, N, K, G):
        x = x.contiguous()
        for g in range(A):
            _capi.check("gemq_dequant_gemm_tc", _capi.lib.gemq_dequant_gemm_tc(
                x.data_ptr(), indices[g:g + 1].data_ptr(), wq.data_ptr(), scales.data_ptr(), zeros.data_ptr(),
                nbits.data_ptr(), wq_strides.data_ptr(), zs_strides.data_ptr(), 0, out[g].data_ptr(), M, N, K, G, 0,
                error_word(dev).data_ptr(), stream_ptr(dev)))
        return out
    if M <= _ROW_BLOCK:
        blocks = [(0, M, out)]
    else:
        blocks = []
        for i in range(0, M, _ROW_BLOCK):
            m = min(_ROW_BLOCK, M - i)
            blocks.append((i, m, torch.empty((A, m, N), dtype=torch.float16, device=dev)))
    st = _capi.stacked(wq, scales, zeros, nbits, wq_strides, zs_strides)
    for i, m, dst in blocks:
        ws = gemv_workspace(dev, A * N, K, m)
        xs = x[i:i + m]
        _capi.check("gemq_dequant_group_gemv", _capi.lib.gemq_dequant_group_gemv(
            xs.data_ptr(), xs.stride(0), indices.data_ptr(), A, ctypes.byref(st), dst.data_ptr(), m, N, K, G,
            ws.data_ptr(), ws.numel(), stream_ptr(dev)))
        if dst is not out:
            out[:, i:i + m] = dst
    return out


dequant_group_gemm_triton = dequant_group_gemm
