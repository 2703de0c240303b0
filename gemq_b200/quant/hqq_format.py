"""HQQ-format quantised layers -> kernel form, without hqq or gemlite installed.

The reference loads its checkpoints with hqq (>= 0.2.8) and converts every ``HQQLinear`` with
gemlite (>= 0.5.1) (``create_gemlite_from_hqq``, gemq/inference/patch.py:23-68): unpack the
codes to ``[out, in]``, hand gemlite the per-group ``scale`` / ``zero`` of shape
``[out * in / G, 1]`` and let it pack.  Neither package is available to this build, so the bit
packing below restates hqq's published scheme (the ``bit_to_packing`` table the reference
uses at gemq/utils/quant_utils.py:76 selects ``4bit_u8``, ``2bit_u8``, ``1bit_u8`` and
``3bit_32``), and the metadata conversion follows what the reference's kernels index:
``scales`` / ``zeros`` as ``[in / G, out]`` with the additive offset ``-zero * scale``
(gemq/triton_kernels/utils.py:196, dequant_gemv.py:97-98).  NOT pinned against real hqq /
gemlite objects: the tests build their fixture with ``hqq_pack`` from this file.

HQQ packs along dim 0 of the ``[groups_total, G]`` code matrix: the rows are cut into ``n``
equal steps (2, 4, 8 or 10 codes per storage element) and step ``j`` lands in bit field ``j``
counted from the top.
"""
from __future__ import annotations

import torch
from torch import Tensor

from .emit import emit_packed_linear

_PER_ELEMENT = {4: 2, 2: 4, 1: 8, 3: 10}


def hqq_pack(codes: Tensor, nbits: int) -> Tensor:
    """``[rows, G]`` codes -> HQQ storage: uint8 ``[rows / n, G]`` for 4/2/1 bits (n = 2/4/8),
    int32 ``[ceil(rows / 10), G]`` for 3 bits (rows zero-padded to a multiple of 10)."""
    n = _PER_ELEMENT[nbits]
    if nbits == 3:
        step = -(-codes.shape[0] // n)
        q = torch.zeros((n * step, codes.shape[1]), dtype=torch.int32, device=codes.device)
        q[:codes.shape[0]] = codes.to(torch.int32)
        out = torch.zeros((step, codes.shape[1]), dtype=torch.int32, device=codes.device)
        for j in range(n):
            out |= q[j * step:(j + 1) * step] << (3 * (n - 1 - j))
        return out
    assert codes.shape[0] % n == 0, "row count must be a multiple of the codes per byte"
    step = codes.shape[0] // n
    out = torch.zeros((step, codes.shape[1]), dtype=torch.uint8, device=codes.device)
    for j in range(n):
        out |= (codes[j * step:(j + 1) * step].to(torch.uint8) << (nbits * (n - 1 - j))).to(torch.uint8)
    return out


def hqq_unpack(packed: Tensor, nbits: int) -> Tensor:
    """Inverse of ``hqq_pack``: uint8 codes ``[n * rows_packed, G]`` (3-bit: including the padding rows)."""
    n = _PER_ELEMENT[nbits]
    mask = (1 << nbits) - 1
    p = packed.to(torch.int32)
    parts = [((p >> (nbits * (n - 1 - j))) & mask).to(torch.uint8) for j in range(n)]
    return torch.cat(parts, dim=0)


def packed_linear_from_hqq(W_q: Tensor, meta: dict):
    """One HQQ layer (its packed ``W_q`` and ``meta`` dict with ``shape``, ``nbits``,
    ``group_size``, ``axis``, ``scale``, ``zero``) -> kernel form.  Follows
    gemq/inference/patch.py:26-37: only ``axis == 1``; the unpacked codes are cut to
    ``out * in / G`` rows (3-bit padding) and viewed as ``[out, in]``."""
    assert meta["axis"] == 1, "Only axis==1 is supported."
    out_f, in_f = meta["shape"]
    nbits, G = int(meta["nbits"]), int(meta["group_size"])
    codes = hqq_unpack(W_q, nbits)[: out_f * in_f // G].reshape(out_f, in_f)
    return emit_packed_linear(codes, meta["scale"], meta["zero"], nbits, G)
