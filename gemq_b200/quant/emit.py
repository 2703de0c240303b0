"""Quantise-side emit of the kernel-form layout and the packing self-check.

The reference's quantisation driver turns its fake-quantised ``nn.Linear`` modules into HQQ
layers (``replace_linears``, gemq/utils/quant_utils.py:131-156: ``Q = round(W.view(groups, -1) /
scale + zero).clamp(0, 2^b - 1)``) and later re-packs those for the kernels
(gemq/inference/patch.py:23-68).  ``emit_packed_linear`` goes from the same quantiser outputs
straight to the tensors the kernels consume, and ``check_packing`` is the assertion the
reference only prints (gemq/utils/quant_utils.py:159-173).  Plain torch, any device: this is
load-time code, not the inference path.
"""
from __future__ import annotations

import torch
from torch import Tensor


def _packed_linear_cls():
    from ..inference.packed_linear import PackedLinear  # imported late: the inference package imports this module
    return PackedLinear


def pack_kernel_form_torch(codes: Tensor, nbits: int) -> Tensor:
    """uint8 codes ``[N, K]`` -> int32 ``[ceil(K / eps), N]`` contiguous, ``eps = 32 // nbits``: code
    ``k`` of column ``n`` sits in word ``(k // eps, n)`` at bit ``(k % eps) * nbits``; missing lanes
    of the last word are zero (gemq/triton_kernels/utils.py:33-70 with ``transpose=True``)."""
    assert nbits in (1, 2, 3, 4) and codes.dim() == 2
    N, K = codes.shape
    eps = 32 // nbits
    rows = -(-K // eps)
    q = torch.zeros((N, rows * eps), dtype=torch.int64, device=codes.device)
    q[:, :K] = codes.to(torch.int64)
    shifts = (torch.arange(eps, device=codes.device, dtype=torch.int64) * nbits).view(1, 1, eps)
    words = (q.view(N, rows, eps) << shifts).sum(dim=2)          # < 2^32, disjoint bit fields
    words = torch.where(words >= 2 ** 31, words - 2 ** 32, words)  # two's complement int32
    return words.to(torch.int32).t().contiguous()


def unpack_kernel_form_torch(wq: Tensor, nbits: int, K: int) -> Tensor:
    """Inverse of ``pack_kernel_form_torch``: int32 ``[rows, N]`` -> uint8 codes ``[N, K]``."""
    eps = 32 // nbits
    w = wq.to(torch.int64) & 0xFFFFFFFF
    shifts = (torch.arange(eps, device=wq.device, dtype=torch.int64) * nbits).view(1, eps, 1)
    q = (w.unsqueeze(1) >> shifts) & ((1 << nbits) - 1)        # [rows, eps, N]
    return q.reshape(-1, wq.shape[1])[:K].t().contiguous().to(torch.uint8)


def dequantize_torch(p) -> Tensor:
    """fp16 ``W [out, in]`` the kernels see: ``fp16(q * scale + offset)`` with one rounding
    (gemq/triton_kernels/utils.py:206-210), computed in float64."""
    q = unpack_kernel_form_torch(p.W_q, p.W_nbits, p.in_features).to(torch.float64)     # [N, K]
    s = p.scales.to(torch.float64).repeat_interleave(p.group_size, dim=0).t()          # [N, K]
    z = p.zeros.to(torch.float64).repeat_interleave(p.group_size, dim=0).t()
    return (q * s + z).to(torch.float16)


def quantise_codes(W: Tensor, scale: Tensor, zero: Tensor, nbits: int) -> Tensor:
    """Codes of a weight ``W [out, in]`` for per-group parameters given as ``[out * in / G, 1]``
    (groups run along the input dimension inside each output row):
    ``round(W.view(groups, -1) / scale + zero).clamp(0, 2^b - 1)``
    (gemq/utils/quant_utils.py:142-147)."""
    groups = scale.shape[0]
    q = torch.round(W.reshape(groups, -1).float() / scale.float() + zero.float()).clamp(0, 2 ** nbits - 1)
    return q.reshape(W.shape).to(torch.uint8)


def emit_packed_linear(codes: Tensor, scale: Tensor, zero: Tensor, nbits: int, group_size: int):
    """Quantiser output -> kernel form.  ``codes`` uint8 ``[out, in]``; ``scale`` / ``zero`` (the
    zero-point of ``W = (Q - zero) * scale``, gemq/quantizers/gptq.py:446-450) either
    ``[out * in / G, 1]`` as the quantisers keep them or already ``[in / G, out]``."""
    out_f, in_f = codes.shape
    ng = in_f // group_size
    if scale.shape == (out_f * ng, 1) or scale.dim() == 1:
        scale = scale.reshape(out_f, ng).t()
        zero = zero.reshape(out_f, ng).t()
    assert tuple(scale.shape) == (ng, out_f) == tuple(zero.shape)
    s16 = scale.to(torch.float16).contiguous()
    offset = (-(zero.float() * s16.float())).to(torch.float16).contiguous()
    return _packed_linear_cls()(pack_kernel_form_torch(codes, nbits), s16, offset, nbits, group_size, in_f, out_f)


def check_packing(p, codes: Tensor = None, weight: Tensor = None, tol: float = None) -> float:
    """Assert that a packed layer holds what it was made from.  With ``codes``: the unpacked
    integers must be identical.  With ``weight`` (the fake-quantised ``W``): the mean absolute
    reconstruction error must stay below ``tol`` (default: one fp16 rounding of the largest
    weight).  Returns the mean absolute error (0.0 without ``weight``)."""
    if codes is not None:
        got = unpack_kernel_form_torch(p.W_q, p.W_nbits, p.in_features)
        if not torch.equal(got.cpu(), codes.to(torch.uint8).cpu()):
            raise AssertionError("packed codes differ from the quantiser's codes")
    err = 0.0
    if weight is not None:
        w = dequantize_torch(p).float().cpu()
        err = float((w - weight.float().cpu()).abs().mean())
        bound = tol if tol is not None else float(weight.abs().max()) * 2.0 ** -10 + 1e-6
        if err > bound:
            raise AssertionError(f"mean reconstruction error {err:.3e} above {bound:.3e}")
    return err
