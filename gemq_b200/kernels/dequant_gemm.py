"""Dequant-fused GEMM; same call signature as gemq/triton_kernels/dequant_gemm.py."""
from __future__ import annotations

import torch
from torch import Tensor

from .. import _capi
from ._ops import library_op
from ._runtime import check_kernel_form, error_word, require, require_cuda, stream_ptr, tc_gemm_ok
from .dequant_gemv import dequant_gemv_rows

_ROW_BLOCK = 64


def _fake_gemm(x, w_q, scales, zeros, nbits, group_size):
    M, K = x.shape
    N = w_q.shape[1]
    tc = tc_gemm_ok(M, N, K, group_size) and x.dtype in (torch.float16, torch.bfloat16)
    return x.new_empty((M, N), dtype=x.dtype if tc else torch.float16)


@library_op("dequant_gemm", _fake_gemm)
def dequant_gemm(x: Tensor, w_q: Tensor, scales: Tensor, zeros: Tensor, nbits: int, group_size: int) -> Tensor:
    """``output[M, N] = x[M, K] @ dequantize(w_q, scales, zeros)``, fp16
    (gemq/triton_kernels/dequant_gemm.py:150-193).  32 rows or more go to the tcgen05 GEMM when
    N % 128 == 0 and K % 64 == 0; otherwise rows are processed eight at a time by the decode
    kernel, in calls of at most 64 rows to bound the split-K workspace."""
    require(x.dim() == 2, "x must be [M, K]")
    M, K = x.shape
    N = w_q.shape[1]
    if tc_gemm_ok(M, N, K, group_size) and x.dtype in (torch.float16, torch.bfloat16):
        dev = require_cuda(x, w_q, scales, zeros)
        check_kernel_form(w_q, scales, zeros, K, N, nbits, group_size)
        x = x.contiguous()
        out = torch.empty((M, N), dtype=x.dtype, device=dev)
        _capi.check("gemq_dequant_gemm_tc", _capi.lib.gemq_dequant_gemm_tc(
            x.data_ptr(), None, w_q.data_ptr(), scales.data_ptr(), zeros.data_ptr(), None, None, None, nbits,
            out.data_ptr(), M, N, K, group_size, int(x.dtype == torch.bfloat16), error_word(dev).data_ptr(),
            stream_ptr(dev)))
        return out
    rows = dequant_gemv_rows._init_fn  # the plain function behind the operator
    if M <= _ROW_BLOCK:
        return rows(x, w_q, scales, zeros, nbits, group_size)
    return torch.cat([rows(x[i:i + _ROW_BLOCK], w_q, scales, zeros, nbits, group_size)
                      for i in range(0, M, _ROW_BLOCK)])


dequant_gemm_triton = dequant_gemm
