"""Load-time tools: quantise-side emit, the packing check, the HQQ-format reader (CPU, plain torch)."""
import numpy as np
import pytest
import torch

from oracle import gemq_oracle as O
from gemq_b200.quant import (check_packing, dequantize_torch, emit_packed_linear, hqq_pack, hqq_unpack,
                             pack_kernel_form_torch, packed_linear_from_hqq, quantise_codes, unpack_kernel_form_torch)


@pytest.mark.parametrize("nbits,K", [(1, 256), (2, 384), (3, 1408), (3, 4096), (4, 200)])
def test_torch_packer_matches_the_oracle_and_the_golden_layout(nbits, K):
    rng = np.random.default_rng(nbits * 1000 + K)
    q = rng.integers(0, 2 ** nbits, (24, K), dtype=np.uint8)
    wq = pack_kernel_form_torch(torch.from_numpy(q), nbits)
    assert np.array_equal(wq.numpy(), O.pack_kernel_form(q, nbits))
    assert np.array_equal(unpack_kernel_form_torch(wq, nbits, K).numpy(), q)


def test_torch_packer_matches_reference_kernel_output(golden):
    for b in (1, 2, 3, 4):
        q = golden[f"pack{b}_q"]  # [rows, cols] codes and the reference kernel's [rows, ceil(cols / eps)] words
        assert np.array_equal(pack_kernel_form_torch(torch.from_numpy(q), b).numpy().T, golden[f"pack{b}_w"])


@pytest.mark.parametrize("nbits", [1, 2, 3, 4])
def test_emit_and_check_packing(nbits):
    g = torch.Generator().manual_seed(nbits)
    out_f, in_f, G = 48, 512, 128
    W = torch.randn(out_f, in_f, generator=g) * 0.05
    groups = out_f * in_f // G
    wg = W.view(groups, G)
    scale = ((wg.max(1, keepdim=True).values - wg.min(1, keepdim=True).values) / (2 ** nbits - 1)).clamp_min(1e-5)
    zero = torch.round(-wg.min(1, keepdim=True).values / scale)
    codes = quantise_codes(W, scale, zero, nbits)
    fake = ((codes.view(groups, G).float() - zero) * scale).view(out_f, in_f)      # the quantiser's W
    p = emit_packed_linear(codes, scale, zero, nbits, G)
    assert p.W_q.shape == (-(-in_f // (32 // nbits)), out_f) and p.scales.shape == (in_f // G, out_f)
    err = check_packing(p, codes=codes, weight=fake)
    assert err < 1e-4
    # a corrupted word is caught
    bad = emit_packed_linear(codes, scale, zero, nbits, G)
    bad.W_q[0, 0] ^= 1
    with pytest.raises(AssertionError):
        check_packing(bad, codes=codes)
    # the kernel-form dequantisation equals the oracle's bit for bit
    want = O.dequantize(p.W_q.numpy(), p.scales.numpy(), p.zeros.numpy(), nbits, G, in_f)  # [K, N]
    assert np.array_equal(dequantize_torch(p).numpy().view(np.uint16), np.ascontiguousarray(want.T).view(np.uint16))


@pytest.mark.parametrize("nbits", [1, 2, 3, 4])
def test_hqq_format_round_trip_and_conversion(nbits):
    g = torch.Generator().manual_seed(10 + nbits)
    out_f, in_f, G = 40, 384, 128
    groups = out_f * in_f // G
    codes = torch.randint(0, 2 ** nbits, (groups, G), generator=g, dtype=torch.uint8)   # HQQ's [groups, G] view
    packed = hqq_pack(codes, nbits)
    assert packed.dtype == (torch.int32 if nbits == 3 else torch.uint8)
    assert torch.equal(hqq_unpack(packed, nbits)[:groups], codes)
    scale = torch.rand(groups, 1, generator=g) * 0.02 + 1e-3
    zero = torch.rand(groups, 1, generator=g) * (2 ** nbits - 1)
    meta = dict(shape=(out_f, in_f), nbits=nbits, group_size=G, axis=1, scale=scale.half(), zero=zero.half())
    p = packed_linear_from_hqq(packed, meta)
    # HQQ's own dequantisation: (W_q - zero) * scale on the [groups, G] view, reshaped to [out, in]
    want = ((codes.float() - zero.half().float()) * scale.half().float()).view(out_f, in_f)
    got = dequantize_torch(p).float()
    assert float((got - want).abs().max()) < 2e-3 * float(want.abs().max()) + 1e-4
    check_packing(p, codes=codes.view(out_f, in_f))


def test_prepare_for_inference_swaps_linears_and_blocks():
    """A toy Mixtral-shaped model whose linears are HQQ-format stand-ins: after
    prepare_for_inference every expert linear is in kernel form and every layer's MoE block is
    the fused quantised one, with the stacked tensors the kernels expect."""
    import torch.nn as nn
    from types import SimpleNamespace
    from gemq_b200.inference import QuantFusedMixtralMoEBlock, QuantLinear, prepare_for_inference
    D, Fd, E, G = 256, 384, 4, 128
    g = torch.Generator().manual_seed(5)

    class FakeHQQ(nn.Module):
        def __init__(self, out_f, in_f, nbits):
            super().__init__()
            groups = out_f * in_f // G
            self.codes = torch.randint(0, 2 ** nbits, (groups, G), generator=g, dtype=torch.uint8)
            self.W_q = hqq_pack(self.codes, nbits)
            self.meta = dict(shape=(out_f, in_f), nbits=nbits, group_size=G, axis=1,
                             scale=(torch.rand(groups, 1, generator=g) * 0.02 + 1e-3).half(),
                             zero=(torch.rand(groups, 1, generator=g) * (2 ** nbits - 1)).half())
            self.bias = None

    class Expert(nn.Module):
        def __init__(self, b):
            super().__init__()
            self.w1, self.w2, self.w3 = FakeHQQ(Fd, D, b), FakeHQQ(D, Fd, b), FakeHQQ(Fd, D, b)

    class Moe(nn.Module):
        def __init__(self):
            super().__init__()
            self.gate = nn.Linear(D, E, bias=False)
            self.experts = nn.ModuleList([Expert(b) for b in (1, 2, 3, 4)])

    class Layer(nn.Module):
        def __init__(self):
            super().__init__()
            self.block_sparse_moe = Moe()

    class Model(nn.Module):
        def __init__(self):
            super().__init__()
            self.model = nn.Module()
            self.model.layers = nn.ModuleList([Layer(), Layer()])
            self.config = SimpleNamespace(hidden_size=D, intermediate_size=Fd, num_local_experts=E, num_experts_per_tok=2)

    m = Model()
    codes_e2_w1 = m.model.layers[1].block_sparse_moe.experts[2].w1.codes.clone()
    prepare_for_inference(m, "mixtral-8x7b")
    for layer in m.model.layers:
        blk = layer.block_sparse_moe
        assert isinstance(blk, QuantFusedMixtralMoEBlock)
        assert blk.w1_nbits.tolist() == [1, 2, 3, 4] and blk.w1_scales.shape == (E * D // G, Fd)
        rows = [-(-D // (32 // b)) for b in (1, 2, 3, 4)]
        assert blk.w1_wq.shape == (sum(rows), Fd)
        assert blk.w1_wq_strides.tolist() == [0] + list(np.cumsum([r * Fd for r in rows])[:-1])
    blk = m.model.layers[1].block_sparse_moe
    off, r3 = int(blk.w1_wq_strides[2]), -(-D // 10)
    got = unpack_kernel_form_torch(blk.w1_wq.view(-1)[off:off + r3 * Fd].view(r3, Fd), 3, D)
    assert torch.equal(got, codes_e2_w1.view(Fd, D))
