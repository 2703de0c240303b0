"""Packing format ops; same call signatures as gemq/triton_kernels/utils.py."""
from __future__ import annotations

import torch

from .. import _capi
from ._runtime import require, require_cuda, stream_ptr


def elements_per_sample(nbits: int, packing_bitwidth: int = 32) -> int:
    return packing_bitwidth // nbits


def pack_weights_over_cols(W_q: torch.Tensor, W_nbits: int, packing_bitwidth: int = 32, transpose: bool = True):
    """uint8 codes ``[out_features, in_features]`` -> int32 words, ``(packed, elements_per_sample)``.

    Mirrors pack_weights_over_cols_triton (gemq/triton_kernels/utils.py:74-113): with
    ``transpose=True`` the result is the ``.t()`` view ``[ceil(in/eps), out]`` of a row-major
    ``[out, ceil(in/eps)]`` buffer.
    """
    assert packing_bitwidth == 32, "Unsuported bitpacking width"
    assert W_nbits in (4, 3, 2, 1), f"Untested quantization bitwidth: {W_nbits}"
    dev = require_cuda(W_q)
    require(W_q.dim() == 2, "W_q must be 2-D")
    q = W_q.contiguous()
    if q.dtype != torch.uint8:
        q = q.to(torch.uint8)
    rows, cols = q.shape
    eps = 32 // W_nbits
    out = torch.empty((rows, -(-cols // eps)), dtype=torch.int32, device=dev)
    _capi.check("gemq_pack_over_cols",
                _capi.lib.gemq_pack_over_cols(q.data_ptr(), out.data_ptr(), rows, cols, W_nbits, stream_ptr(dev)))
    return (out.t() if transpose else out), eps


def pack_kernel_form(W_q: torch.Tensor, W_nbits: int) -> torch.Tensor:
    """uint8 codes ``[N, K]`` -> contiguous int32 ``[ceil(K/eps), N]`` (what the MoE blocks stack)."""
    dev = require_cuda(W_q)
    require(W_q.dim() == 2 and W_q.dtype == torch.uint8, "W_q must be 2-D uint8")
    require(W_nbits in (1, 2, 3, 4), f"unsupported bit-width {W_nbits}")
    q = W_q.contiguous()
    N, K = q.shape
    out = torch.empty((-(-K // (32 // W_nbits)), N), dtype=torch.int32, device=dev)
    _capi.check("gemq_pack_kernel_form",
                _capi.lib.gemq_pack_kernel_form(q.data_ptr(), out.data_ptr(), N, K, W_nbits, stream_ptr(dev)))
    return out


def unpack_over_cols(W_q_packed: torch.Tensor, W_nbits: int, packing_bitwidth: int, num_output_cols: int,
                     dtype: torch.dtype = torch.uint8) -> torch.Tensor:
    """Inverse of the row-major pack (gemq/triton_kernels/utils.py:149-189)."""
    assert packing_bitwidth == 32
    dev = require_cuda(W_q_packed)
    require(W_q_packed.dim() == 2 and W_q_packed.dtype == torch.int32, "packed words must be 2-D int32")
    p = W_q_packed.contiguous()
    rows, words = p.shape
    out = torch.empty((rows, num_output_cols), dtype=torch.uint8, device=dev)
    _capi.check("gemq_unpack_over_cols",
                _capi.lib.gemq_unpack_over_cols(p.data_ptr(), out.data_ptr(), rows, words, num_output_cols, W_nbits,
                                                stream_ptr(dev)))
    return out if dtype == torch.uint8 else out.to(dtype)


def dequantize(w_q: torch.Tensor, scales: torch.Tensor, zeros: torch.Tensor, nbits: int, group_size: int) -> torch.Tensor:
    """Kernel-form tensors -> fp16 ``W^T [K, N]``, the values ``dequantize``
    (gemq/triton_kernels/utils.py:192-212) produces: one fp16 fma per weight."""
    dev = require_cuda(w_q, scales, zeros)
    G, N = scales.shape
    K = G * group_size
    from ._runtime import check_kernel_form
    check_kernel_form(w_q, scales, zeros, K, N, nbits, group_size)
    out = torch.empty((K, N), dtype=torch.float16, device=dev)
    _capi.check("gemq_dequantize",
                _capi.lib.gemq_dequantize(w_q.data_ptr(), scales.data_ptr(), zeros.data_ptr(), out.data_ptr(),
                                          K, N, nbits, group_size, stream_ptr(dev)))
    return out


# Names the reference's callers import (gemq/inference/patch.py:17).
pack_weights_over_cols_triton = pack_weights_over_cols
unpack_over_cols_triton = unpack_over_cols
