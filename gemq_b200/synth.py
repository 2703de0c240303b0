"""Seeded synthetic weights and inputs with the shapes and value distributions of the
benchmark configurations (there are no checkpoints or datasets in the build environment).

Codes are uniform in ``[0, 2^b)``, the per-group fp16 scale is ``|N(0,1)| * 0.01 + 1e-3`` and
the fp16 zero-point is uniform in ``[0, 2^b - 1]``; the kernels receive the additive offset
``-zero * scale``.
"""
from __future__ import annotations

from types import SimpleNamespace

import torch

from .inference.moe_block import QuantFusedDeepseekV2MoEBlock, QuantFusedMixtralMoEBlock
from .inference.packed_linear import PackedLinear
from .synth_bits import draw_expert_bits  # noqa: F401  (re-exported)

MIXTRAL_8X7B = dict(hidden_size=4096, intermediate_size=14336, num_local_experts=8, num_experts_per_tok=2)
DEEPSEEK_V2_LITE = dict(hidden_size=2048, moe_intermediate_size=1408, n_routed_experts=64, n_shared_experts=2,
                        num_experts_per_tok=6, norm_topk_prob=False)


def generator(seed: int, device) -> torch.Generator:
    g = torch.Generator(device=device)
    g.manual_seed(seed)
    return g


def draw_codes_meta(out_f: int, in_f: int, nbits: int, group: int, gen: torch.Generator, device):
    """codes uint8 [out, in], scale fp16 [in/group, out], zero-point fp16 [in/group, out]."""
    codes = torch.randint(0, 2 ** nbits, (out_f, in_f), dtype=torch.uint8, device=device, generator=gen)
    scale = (torch.randn(in_f // group, out_f, device=device, generator=gen).abs() * 0.01 + 1e-3).to(torch.float16)
    zero = (torch.rand(in_f // group, out_f, device=device, generator=gen) * (2 ** nbits - 1)).to(torch.float16)
    return codes, scale, zero


def make_linear(out_f: int, in_f: int, nbits: int, group: int, gen: torch.Generator, device) -> PackedLinear:
    codes, scale, zero = draw_codes_meta(out_f, in_f, nbits, group, gen, device)
    return PackedLinear.from_codes(codes, scale, zero, nbits, group)


def mixtral_block(seed: int = 0, device="cuda", bits=None, group: int = 128, **overrides) -> QuantFusedMixtralMoEBlock:
    cfg = SimpleNamespace(**{**MIXTRAL_8X7B, **overrides})
    E, D, Fd = cfg.num_local_experts, cfg.hidden_size, cfg.intermediate_size
    bits = bits or draw_expert_bits(E, seed)
    gen = generator(seed, device)
    gate = (torch.randn(E, D, device=device, generator=gen) * 0.02).to(torch.float16)
    w1 = [make_linear(Fd, D, b, group, gen, device) for b in bits]
    w3 = [make_linear(Fd, D, b, group, gen, device) for b in bits]
    w2 = [make_linear(D, Fd, b, group, gen, device) for b in bits]
    return QuantFusedMixtralMoEBlock.from_linears(cfg, gate, w1, w2, w3)


def deepseek_block(seed: int = 0, device="cuda", bits=None, shared_bits: int = 4, group: int = 128,
                   **overrides) -> QuantFusedDeepseekV2MoEBlock:
    cfg = SimpleNamespace(**{**DEEPSEEK_V2_LITE, **overrides})
    E, D, Fd = cfg.n_routed_experts, cfg.hidden_size, cfg.moe_intermediate_size
    SF = cfg.n_shared_experts * Fd
    bits = bits or draw_expert_bits(E, seed)
    gen = generator(seed, device)
    gate = (torch.randn(E, D, device=device, generator=gen) / D ** 0.5).to(torch.float16)  # logits ~ N(0, 1)
    w1 = [make_linear(Fd, D, b, group, gen, device) for b in bits]
    w3 = [make_linear(Fd, D, b, group, gen, device) for b in bits]
    w2 = [make_linear(D, Fd, b, group, gen, device) for b in bits]
    shared = (make_linear(SF, D, shared_bits, group, gen, device), make_linear(D, SF, shared_bits, group, gen, device),
              make_linear(SF, D, shared_bits, group, gen, device))
    return QuantFusedDeepseekV2MoEBlock.from_linears(cfg, gate, w1, w2, w3, shared)


def mixtral_expert_parallel(rank: int, world: int, seed: int = 0, device="cuda", bits=None, group: int = 128,
                            process_group=None, routed_rows=None, replicate=True, placement=None, **overrides):
    """This rank's shard of a Mixtral-shaped layer.  Without ``routed_rows`` rank r holds experts
    ``[r*E/world, (r+1)*E/world)``; with it (rows each expert receives, e.g. from calibration) the
    experts are placed so that the rows per rank even out, an expert above a rank's fair share
    being held by several ranks when ``replicate``.  Every expert is drawn from its own seed, so
    all ranks agree on the full layer.  ``placement`` gives the table directly.  Returns (layer, bits, [(expert, rank, share), ...])."""
    from .inference.expert_parallel import (ExpertParallelMixtralMoE, Placement, balanced_placement, contiguous_placement,
                                            replicated_placement)
    cfg = {**MIXTRAL_8X7B, **overrides}
    E, D, Fd, A = cfg["num_local_experts"], cfg["hidden_size"], cfg["intermediate_size"], cfg["num_experts_per_tok"]
    bits = bits or draw_expert_bits(E, seed)
    gate = (torch.randn(E, D, device=device, generator=generator(seed, device)) * 0.02).to(torch.float16)
    if placement is not None:
        place = placement
    elif routed_rows is None:
        place = Placement.from_expert_to_rank(contiguous_placement(E, world), world)
    elif replicate:
        place = replicated_placement(routed_rows, world)
    else:
        place = Placement.from_expert_to_rank(balanced_placement(routed_rows, world), world)
    mine = place.experts_of[rank]
    w1, w2, w3 = [], [], []
    for e in mine:
        gen = generator(seed * 1000 + 17 * e + 1, device)
        w1.append(make_linear(Fd, D, bits[e], group, gen, device))
        w3.append(make_linear(Fd, D, bits[e], group, gen, device))
        w2.append(make_linear(D, Fd, bits[e], group, gen, device))
    local = None
    if mine:
        local_cfg = SimpleNamespace(hidden_size=D, intermediate_size=Fd, num_local_experts=len(mine), num_experts_per_tok=1)
        local = QuantFusedMixtralMoEBlock.from_linears(local_cfg, gate[mine].clone(), w1, w2, w3)
    layer = ExpertParallelMixtralMoE(local, gate, E, A, process_group, expert_to_rank=place)
    return layer, bits, [list(i) for i in place.instances]
