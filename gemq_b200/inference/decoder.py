"""A Mixtral-architecture decoder around the quantised MoE blocks, and the generate loop.

The reference drives a Hugging Face model: ``prefill`` (eager), then ``decode_one_token`` under
``torch.compile(mode="reduce-overhead")`` in ``decode_n_tokens``, with a static cache
(gemq/benchmark_generate.py:46-63, :92-134, :158-168).  No checkpoint exists in the build
environment, so ``MixtralDecoder`` is a random-initialised model of the same architecture
(RMSNorm, grouped-query attention with rotary embeddings in bf16, one quantised MoE block per
layer, tied to nothing) whose decode step is captured in a CUDA graph; the functions keep the
reference's names and roles.  Sampling is greedy.
"""
from __future__ import annotations

import time
from types import SimpleNamespace
from typing import List, Tuple

import torch
import torch.nn as nn
import torch.nn.functional as F
from torch import Tensor

from .kv_cache import StaticCache

MIXTRAL_8X7B_CONFIG = dict(hidden_size=4096, intermediate_size=14336, num_local_experts=8, num_experts_per_tok=2,
                           num_hidden_layers=32, num_attention_heads=32, num_key_value_heads=8, head_dim=128,
                           vocab_size=32000, rms_norm_eps=1e-5, rope_theta=1e6)


class RMSNorm(nn.Module):
    def __init__(self, dim: int, eps: float):
        super().__init__()
        self.weight = nn.Parameter(torch.ones(dim))
        self.eps = eps

    def forward(self, x: Tensor) -> Tensor:
        v = x.float()
        return (v * torch.rsqrt(v.pow(2).mean(-1, keepdim=True) + self.eps)).to(x.dtype) * self.weight


def rotary(x: Tensor, pos: Tensor, theta: float) -> Tensor:
    """x [B, H, S, hd], pos [S] -> rotated (half-split convention)."""
    hd = x.shape[-1]
    inv = 1.0 / (theta ** (torch.arange(0, hd, 2, device=x.device, dtype=torch.float32) / hd))
    ang = pos.float()[:, None] * inv[None, :]
    cos, sin = torch.cat([ang.cos(), ang.cos()], -1), torch.cat([ang.sin(), ang.sin()], -1)
    x1, x2 = x[..., : hd // 2], x[..., hd // 2:]
    return (x.float() * cos + torch.cat([-x2, x1], -1).float() * sin).to(x.dtype)


class Attention(nn.Module):
    def __init__(self, cfg, layer_idx: int, make_linear):
        super().__init__()
        self.cfg, self.layer_idx = cfg, layer_idx
        H, Hkv, hd, D = cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim, cfg.hidden_size
        self.q_proj, self.k_proj = make_linear(H * hd, D), make_linear(Hkv * hd, D)
        self.v_proj, self.o_proj = make_linear(Hkv * hd, D), make_linear(D, H * hd)

    def forward(self, x: Tensor, cache: StaticCache, pos: Tensor) -> Tensor:
        B, S, _ = x.shape
        c = self.cfg
        q = self.q_proj(x).view(B, S, c.num_attention_heads, c.head_dim).transpose(1, 2)
        k = self.k_proj(x).view(B, S, c.num_key_value_heads, c.head_dim).transpose(1, 2)
        v = self.v_proj(x).view(B, S, c.num_key_value_heads, c.head_dim).transpose(1, 2)
        q, k = rotary(q, pos, c.rope_theta), rotary(k, pos, c.rope_theta)
        keys, values = cache.update(k, v, self.layer_idx, {"cache_position": pos})
        # a query at position p sees cache slots 0..p; the mask is built on the device from `pos`
        mask = torch.arange(keys.shape[2], device=x.device)[None, :] <= pos[:, None]
        y = F.scaled_dot_product_attention(q, keys, values, attn_mask=mask[None, None], enable_gqa=True)
        return self.o_proj(y.transpose(1, 2).reshape(B, S, -1))


class DecoderLayer(nn.Module):
    def __init__(self, cfg, layer_idx: int, moe_block, make_linear):
        super().__init__()
        self.input_layernorm = RMSNorm(cfg.hidden_size, cfg.rms_norm_eps)
        self.self_attn = Attention(cfg, layer_idx, make_linear)
        self.post_attention_layernorm = RMSNorm(cfg.hidden_size, cfg.rms_norm_eps)
        self.block_sparse_moe = moe_block

    def forward(self, x: Tensor, cache: StaticCache, pos: Tensor) -> Tensor:
        x = x + self.self_attn(self.input_layernorm(x), cache, pos)
        h = self.post_attention_layernorm(x)
        B, S, D = h.shape
        if B * S == 1:
            y, _ = self.block_sparse_moe(h.view(1, 1, D))          # one-token path
        else:
            y, _ = self.block_sparse_moe(h.reshape(1, B * S, D))   # n-token path over all rows
        return x + y.reshape(B, S, D).to(x.dtype)


class MixtralDecoder(nn.Module):
    """Random-initialised Mixtral-architecture decoder; every MoE block is quantised with mixed
    bits (mean ``mean_bits`` per layer), attention stays in bf16 unless ``attn_bits`` is given
    (then its linears are quantised too and run on the same kernels)."""

    def __init__(self, device="cuda", dtype=torch.bfloat16, seed: int = 0, mean_bits: float = 2.0, attn_bits: int = 0,
                 **overrides):
        super().__init__()
        from .. import synth
        from .quant_linear import QuantLinear
        cfg = SimpleNamespace(**{**MIXTRAL_8X7B_CONFIG, **overrides})
        self.config, self.dtype_, self.device_ = cfg, dtype, torch.device(device)
        gen = synth.generator(seed, device)

        def make_linear(out_f: int, in_f: int):
            if attn_bits:
                return QuantLinear(synth.make_linear(out_f, in_f, attn_bits, 128, gen, device))
            lin = nn.Linear(in_f, out_f, bias=False, device=device, dtype=dtype)
            lin.weight.data = (torch.randn(out_f, in_f, device=device, generator=gen) * in_f ** -0.5).to(dtype)
            return lin

        self.embed_tokens = nn.Embedding(cfg.vocab_size, cfg.hidden_size, device=device, dtype=dtype)
        layers = []
        for i in range(cfg.num_hidden_layers):
            bits = synth.draw_expert_bits(cfg.num_local_experts, seed * 1000 + i, mean_bits - 0.01, mean_bits + 0.01)
            moe = synth.mixtral_block(seed=seed * 1000 + i, device=device, bits=bits, hidden_size=cfg.hidden_size,
                                      intermediate_size=cfg.intermediate_size, num_local_experts=cfg.num_local_experts,
                                      num_experts_per_tok=cfg.num_experts_per_tok)
            layers.append(DecoderLayer(cfg, i, moe, make_linear))
        self.layers = nn.ModuleList(layers)
        self.norm = RMSNorm(cfg.hidden_size, cfg.rms_norm_eps).to(device=device, dtype=dtype)
        self.lm_head = nn.Linear(cfg.hidden_size, cfg.vocab_size, bias=False, device=device, dtype=dtype)
        self.lm_head.weight.data = (torch.randn(cfg.vocab_size, cfg.hidden_size, device=device, generator=gen)
                                    * cfg.hidden_size ** -0.5).to(dtype)
        for m in self.modules():
            if isinstance(m, RMSNorm):
                m.to(device=device, dtype=dtype)

    @torch.no_grad()
    def forward(self, input_ids: Tensor, past_key_values: StaticCache, cache_position: Tensor) -> Tensor:
        """input_ids [B, S], cache_position [S] -> logits of the last position [B, vocab]."""
        x = self.embed_tokens(input_ids)
        for layer in self.layers:
            x = layer(x, past_key_values, cache_position)
        return self.lm_head(self.norm(x[:, -1]))

    def expert_bytes_per_token(self) -> float:
        """Algorithmic bytes of the expert weights one decoded token streams (two experts per layer
        at the layer's mean bit width, (b + 0.25) / 8 bytes per weight)."""
        c = self.config
        per_expert = 3 * c.hidden_size * c.intermediate_size
        total = 0.0
        for layer in self.layers:
            bits = layer.block_sparse_moe._nbits_host
            total += c.num_experts_per_tok * per_expert * (sum(bits) / len(bits) + 0.25) / 8
        return total

    def attention_bytes_per_token(self, context: int, batch: int = 1) -> float:
        """Attention and head weights (read once per step) plus the cached keys / values a token reads."""
        c = self.config
        w = c.num_hidden_layers * (2 * c.num_attention_heads + 2 * c.num_key_value_heads) * c.head_dim * c.hidden_size
        w += c.vocab_size * c.hidden_size
        kv = c.num_hidden_layers * 2 * c.num_key_value_heads * c.head_dim * context * batch
        return 2.0 * (w + kv)


def prefill(model: MixtralDecoder, x: Tensor, kv_cache: StaticCache, input_pos: Tensor) -> Tensor:
    """gemq/benchmark_generate.py:46-48 with greedy sampling: next token per sequence [B]."""
    return model(x, kv_cache, input_pos).argmax(dim=-1)


def decode_one_token(model: MixtralDecoder, x: Tensor, kv_cache: StaticCache, input_pos: Tensor) -> Tensor:
    """gemq/benchmark_generate.py:51-53."""
    return model(x, kv_cache, input_pos).argmax(dim=-1)


class GraphedDecodeStep:
    """``decode_one_token`` captured once in a CUDA graph (the role of
    ``torch.compile(mode="reduce-overhead")`` at gemq/benchmark_generate.py:158-160): token and
    position live in static buffers, a step is a copy into them and a replay."""

    def __init__(self, model: MixtralDecoder, kv_cache: StaticCache, batch: int):
        dev = model.device_
        self.tok = torch.zeros((batch, 1), dtype=torch.long, device=dev)
        # the warm-up steps write the cache at `pos`: use the last slot, which a real step fills before any
        # query can see it, so that the prefilled context stays intact
        self.pos = torch.full((1,), kv_cache.max_cache_len - 1, dtype=torch.long, device=dev)
        self.model, self.cache = model, kv_cache
        side = torch.cuda.Stream(device=dev)
        with torch.cuda.stream(side):
            for _ in range(2):
                decode_one_token(model, self.tok, kv_cache, self.pos)
            torch.cuda.synchronize()
            self.graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(self.graph, stream=side):
                self.out = decode_one_token(model, self.tok, kv_cache, self.pos)
        torch.cuda.synchronize()

    def __call__(self, tok: Tensor, pos: Tensor) -> Tensor:
        self.tok.copy_(tok)
        self.pos.copy_(pos)
        self.graph.replay()
        return self.out


def decode_n_tokens(step, cur_token: Tensor, input_pos: Tensor, num_new_tokens: int) -> List[Tensor]:
    """gemq/benchmark_generate.py:56-63; ``step(token [B, 1], pos [1]) -> next token [B]``."""
    new_tokens = []
    for _ in range(num_new_tokens):
        nxt = step(cur_token, input_pos)
        input_pos = input_pos + 1
        new_tokens.append(nxt.clone())
        cur_token = nxt.clone().view(-1, 1)
    return new_tokens


@torch.no_grad()
def generate(model: MixtralDecoder, prompt: Tensor, max_new_tokens: int, kv_cache: StaticCache,
             graphed: bool = True) -> Tuple[Tensor, dict]:
    """Prefill the prompt ``[B, T]``, then decode greedily (gemq/benchmark_generate.py:92-134).
    Returns the sequences ``[B, T + max_new_tokens]`` and the timing stats the reference prints
    (prefill / decode latency and tokens per second, summed over the batch)."""
    dev = prompt.device
    B, T = prompt.shape
    seq = torch.empty((B, T + max_new_tokens), dtype=prompt.dtype, device=dev)
    seq[:, :T] = prompt
    stats = {}
    input_pos = torch.arange(0, T, device=dev)
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    nxt = prefill(model, prompt, kv_cache, input_pos)
    torch.cuda.synchronize()
    stats["prefill_latency"] = time.perf_counter() - t0
    stats["prefill_throughput"] = B * T / stats["prefill_latency"]
    seq[:, T] = nxt
    step = GraphedDecodeStep(model, kv_cache, B) if graphed else (
        lambda tok, pos: decode_one_token(model, tok, kv_cache, pos))
    input_pos = torch.tensor([T], device=dev, dtype=torch.long)
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    new = decode_n_tokens(step, nxt.view(-1, 1), input_pos, max_new_tokens - 1)
    torch.cuda.synchronize()
    stats["decode_latency"] = time.perf_counter() - t0
    stats["decode_throughput"] = B * (max_new_tokens - 1) / stats["decode_latency"]
    if new:
        seq[:, T + 1:] = torch.stack(new, dim=1)
    return seq, stats
