"""Loader side on the GPU: an HQQ-format layer (gemq/inference/patch.py:23-68) converted to the
kernel form and run as a quantised linear, against fp32 math on the de-quantised weight
W = (Q - zero) * scale (gemq/quantizers/gptq.py:446-450)."""
import pytest
import torch

from conftest import MAX_ABS_TOL, REL_FRO_TOL, max_abs, rel_fro

pytestmark = pytest.mark.gpu


def _hqq_layer(seed, out_f, in_f, nbits, G):
    from gemq_b200.quant.hqq_format import hqq_pack
    g = torch.Generator().manual_seed(seed)
    codes = torch.randint(0, 2 ** nbits, (out_f, in_f), generator=g, dtype=torch.uint8)
    groups = out_f * in_f // G
    scale = (torch.randn(groups, 1, generator=g).abs() * 0.01 + 1e-3).half()
    zero = (torch.rand(groups, 1, generator=g) * (2 ** nbits - 1)).half()
    meta = dict(shape=(out_f, in_f), nbits=nbits, group_size=G, axis=1, scale=scale, zero=zero)
    return hqq_pack(codes.reshape(groups, G), nbits), meta, codes, scale, zero


@pytest.mark.parametrize("nbits", [1, 2, 3, 4])
@pytest.mark.parametrize("rows", [1, 64])
def test_hqq_layer_as_quant_linear(nbits, rows):
    from gemq_b200.inference import QuantLinear
    from gemq_b200.quant.emit import check_packing
    from gemq_b200.quant.hqq_format import packed_linear_from_hqq
    out_f, in_f, G = 384, 512, 128
    W_q, meta, codes, scale, zero = _hqq_layer(10 * nbits + rows, out_f, in_f, nbits, G)
    packed = packed_linear_from_hqq(W_q, meta)
    check_packing(packed, codes=codes)          # the integers survive the conversion bit-exactly
    lin = QuantLinear(packed)
    for name in ("W_q", "scales", "zeros"):
        setattr(lin, name, getattr(lin, name).cuda())
    x = torch.randn(rows, in_f, generator=torch.Generator().manual_seed(3)).half()
    y = lin(x.cuda()).float().cpu().numpy()
    s = scale.float().reshape(out_f, in_f // G).repeat_interleave(G, dim=1)
    z = zero.float().reshape(out_f, in_f // G).repeat_interleave(G, dim=1)
    W = (codes.float() - z) * s
    ref = (x.float() @ W.t()).numpy()
    assert y.shape == (rows, out_f)
    assert rel_fro(y, ref) < REL_FRO_TOL, rel_fro(y, ref)
    assert max_abs(y, ref) < MAX_ABS_TOL, max_abs(y, ref)
