"""Build the same seeded quantised MoE layer twice: as oracle tensors and as a GPU block."""
from types import SimpleNamespace

import numpy as np
import torch

from oracle import gemq_oracle as O


def draw_linear(rng, out_f, in_f, b, G=128):
    q = rng.integers(0, 2 ** b, (out_f, in_f), dtype=np.uint8)
    s = (np.abs(rng.standard_normal((in_f // G, out_f))) * 0.01 + 1e-3).astype(np.float16)
    zp = (rng.random((in_f // G, out_f)) * (2 ** b - 1)).astype(np.float16)
    return dict(wq=O.pack_kernel_form(q, b), s=s, z=O.kernel_form_offset(s, zp), b=b, G=G, i=in_f, o=out_f)


def to_packed(lin, device):
    from gemq_b200.inference import PackedLinear
    t = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(device)
    return PackedLinear(t(lin["wq"]), t(lin["s"]), t(lin["z"]), lin["b"], lin["G"], lin["i"], lin["o"])


def stacked(lins):
    return O.StackedExperts([l["wq"] for l in lins], [l["s"] for l in lins], [l["z"] for l in lins],
                            [l["b"] for l in lins], lins[0]["G"])


def make_layer(family, D, Fd, E, A, bits, seed, gate_std, n_shared=0, shared_bits=4, norm_topk_prob=False):
    rng = np.random.default_rng(seed)
    gate = (rng.standard_normal((E, D)) * gate_std).astype(np.float16)
    w1 = [draw_linear(rng, Fd, D, b) for b in bits]
    w3 = [draw_linear(rng, Fd, D, b) for b in bits]
    w2 = [draw_linear(rng, D, Fd, b) for b in bits]
    shared = None
    if n_shared:
        SF = n_shared * Fd
        shared = (draw_linear(rng, SF, D, shared_bits), draw_linear(rng, D, SF, shared_bits),
                  draw_linear(rng, SF, D, shared_bits))  # gate_proj, down_proj, up_proj
    if family == "mixtral":
        cfg = SimpleNamespace(hidden_size=D, intermediate_size=Fd, num_local_experts=E, num_experts_per_tok=A)
    else:
        cfg = SimpleNamespace(hidden_size=D, moe_intermediate_size=Fd, n_routed_experts=E, n_shared_experts=n_shared,
                              num_experts_per_tok=A, norm_topk_prob=norm_topk_prob)
    return dict(family=family, cfg=cfg, gate=gate, w1=w1, w2=w2, w3=w3, shared=shared, A=A)


def oracle_parts(layer):
    sh = None
    if layer["shared"]:
        s1, s2, s3 = layer["shared"]
        trip = lambda l: (l["wq"], l["s"], l["z"])
        sh = (trip(s1), trip(s3), trip(s2), s1["b"], s1["G"])
    return stacked(layer["w1"]), stacked(layer["w3"]), stacked(layer["w2"]), sh


def gpu_block(layer, device="cuda"):
    from gemq_b200.inference import QuantFusedDeepseekV2MoEBlock, QuantFusedMixtralMoEBlock
    gate = torch.from_numpy(layer["gate"]).to(device)
    p = lambda lins: [to_packed(l, device) for l in lins]
    if layer["family"] == "mixtral":
        return QuantFusedMixtralMoEBlock.from_linears(layer["cfg"], gate, p(layer["w1"]), p(layer["w2"]), p(layer["w3"]))
    s1, s2, s3 = layer["shared"]
    return QuantFusedDeepseekV2MoEBlock.from_linears(layer["cfg"], gate, p(layer["w1"]), p(layer["w2"]), p(layer["w3"]),
                                                     (to_packed(s1, device), to_packed(s2, device), to_packed(s3, device)))
