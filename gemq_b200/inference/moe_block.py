"""Quantised fused MoE blocks for Mixtral and DeepSeek-V2 on the gemq_b200 kernels.

Same constructor / ``from_hf`` / ``forward`` surface and attribute names as
``QuantFusedMixtralMoEBlock`` and ``QuantFusedDeepseekV2MoEBlock`` in
gemq/inference/moe_block.py, so ``replace_moe_blocks`` (gemq/inference/patch.py:82-125)
can swap them in.  A one-token forward is a single library call (router, fused
gate/up, SiLU*mul + down, combine); the routing result never reaches the host.
"""
from __future__ import annotations

import ctypes as C
import itertools
import weakref
from typing import Tuple

import torch
import torch.nn as nn
import torch.nn.functional as F
from torch import Tensor

from .. import _capi
from ..kernels import dequant_gemm, dequant_group_gemm
from ..kernels._ops import library_op
from ..kernels._runtime import require_cuda, stream_ptr
from .packed_linear import is_packed_linear

ROUTE_FP16, ROUTE_FP32_SOFTMAX, ROUTE_FP32 = 0, 1, 2
# Decode batches up to this many rows run the one-launch layer kernel row by row; larger ones go through the
# expert-sorted grouped GEMM, which reads every distinct expert (and the shared experts) once per call and is
# faster from about six rows on (measured on the DeepSeek-V2-Lite shape: 360 vs 275 us at 8 rows, 779 vs 333 at 16).
_MAX_LOOPED_TOKENS = 4


def _excl_cumsum(vals, device):
    t = torch.tensor([0] + list(vals), dtype=torch.int64).cumsum(0)[:-1]
    assert int(t.max()) < 2 ** 31, "stacked tensor too large for int32 offsets"
    return t.to(torch.int32).to(device)


# The block-level library calls take a ctypes description of the layer; as custom operators
# they receive an integer handle of the block instead (dynamo treats it as a constant).
_BLOCKS: "weakref.WeakValueDictionary[int, _QuantFusedMoEBase]" = weakref.WeakValueDictionary()
_HANDLES = itertools.count(1)


def _fake_route(x, gate_weight, top_k, mode, renorm):
    T = x.shape[0]
    return (x.new_empty((T, top_k)), x.new_empty((T, top_k), dtype=torch.int64),
            x.new_empty((T, gate_weight.shape[0]), dtype=torch.float32))


@library_op("moe_route", _fake_route)
def route_tokens(x: Tensor, gate_weight: Tensor, top_k: int, mode: int, renorm: bool) -> Tuple[Tensor, Tensor, Tensor]:
    """Router on the device: ``(weights [T, A] in x.dtype, indices int64 [T, A], logits fp32 [T, E])``."""
    dev = require_cuda(x, gate_weight)
    T, D = x.shape
    E = gate_weight.shape[0]
    idx = torch.empty((T, top_k), dtype=torch.int64, device=dev)
    w = torch.empty((T, top_k), dtype=x.dtype, device=dev)
    logits = torch.empty((T, E), dtype=torch.float32, device=dev)
    gate = gate_weight if gate_weight.dtype == x.dtype else gate_weight.to(x.dtype)
    _capi.check("gemq_moe_route", _capi.lib.gemq_moe_route(
        x.data_ptr(), gate.contiguous().data_ptr(), T, D, E, top_k, mode, int(renorm),
        int(x.dtype == torch.bfloat16), idx.data_ptr(), w.data_ptr(), logits.data_ptr(), stream_ptr(dev)))
    return w, idx, logits


class _QuantFusedMoEBase(nn.Module):
    """State and dispatch shared by the two model families."""

    _projections = ("w1", "w2", "w3")

    def __init__(self) -> None:
        super().__init__()
        for p in self._projections:
            for suffix in ("wq", "scales", "zeros", "nbits", "group_sizes", "wq_strides", "zs_strides"):
                setattr(self, f"{p}_{suffix}", None)
        self.block_group_size = None
        self._layer = None       # ctypes struct handed to the library
        self._scratch = None
        self._prefill_scratch = None
        self._nbits_host = None

    # -- construction ---------------------------------------------------------------
    def _stack(self, name: str, linears) -> None:
        """Concatenate per-expert packed tensors and build the metadata tensors
        (gemq/inference/moe_block.py:111-142)."""
        dev = linears[0].W_q.device
        setattr(self, f"{name}_wq", torch.cat([l.W_q.data.contiguous() for l in linears]))
        setattr(self, f"{name}_scales", torch.cat([l.scales.data for l in linears]).contiguous())
        setattr(self, f"{name}_zeros", torch.cat([l.zeros.data for l in linears]).contiguous())
        setattr(self, f"{name}_nbits", torch.tensor([l.W_nbits for l in linears], dtype=torch.int32, device=dev))
        setattr(self, f"{name}_group_sizes",
                torch.tensor([l.group_size for l in linears], dtype=torch.int32, device=dev))
        setattr(self, f"{name}_wq_strides", _excl_cumsum([l.W_q.numel() for l in linears], dev))
        setattr(self, f"{name}_zs_strides", _excl_cumsum([l.scales.numel() for l in linears], dev))

    def _check_group_sizes(self, experts_w1, experts_w2, experts_w3) -> None:
        sizes = {l.group_size for l in (*experts_w1, *experts_w2, *experts_w3)}
        assert len(sizes) == 1, "Group sizes must be the same across all experts."
        self.block_group_size = int(sizes.pop())
        bits = [(a.W_nbits, b.W_nbits) for a, b in zip(experts_w1, experts_w3)]
        assert all(a == b for a, b in bits), "w1 and w3 of an expert must share a bit-width"
        self._nbits_host = [int(l.W_nbits) for l in experts_w1]

    def _stacked_struct(self, name: str) -> _capi.Stacked:
        g = lambda s: getattr(self, f"{name}_{s}")
        return _capi.stacked(g("wq"), g("scales"), g("zeros"), g("nbits"), g("wq_strides"), g("zs_strides"))

    def _single_struct(self, name: str) -> _capi.Single:
        g = lambda s: getattr(self, f"shared_{name}_{s}").data_ptr()
        return _capi.Single(g("wq"), g("scales"), g("zeros"), int(self.shared_nbits), int(self.shared_group_size))

    def _build_layer(self, route_mode: int, renorm: bool, shared_ffn: int) -> None:
        dev = self.w1_wq.device
        self.gate.to(device=dev, dtype=torch.float16)
        L = _capi.MoeLayer()
        L.hidden, L.ffn, L.n_experts, L.top_k = self.hidden_dim, self.ffn_dim, self.num_experts, self.top_k
        L.group_size, L.route_mode, L.renorm, L.shared_ffn = self.block_group_size, route_mode, int(renorm), shared_ffn
        L.gate = self.gate.weight.data_ptr()
        L.w1, L.w3, L.w2 = self._stacked_struct("w1"), self._stacked_struct("w3"), self._stacked_struct("w2")
        if shared_ffn:
            L.s1, L.s3, L.s2 = self._single_struct("w1"), self._single_struct("w3"), self._single_struct("w2")
        self._layer = L
        nbytes = _capi.lib.gemq_moe_decode_scratch_bytes(C.byref(L))
        self._scratch = torch.zeros(nbytes, dtype=torch.uint8, device=dev)
        self._handle = next(_HANDLES)
        _BLOCKS[self._handle] = self

    # -- forward pieces ----------------------------------------------------------------
    def _decode(self, x: Tensor, route_mode: int):
        """``x [T, D]`` fp16 -> ``out [T, D]``, routing weights and indices, all on the device."""
        return _moe_decode(x, self._handle, route_mode)

    def _decode_impl(self, x: Tensor, route_mode: int):
        dev = require_cuda(x)
        T = x.shape[0]
        out = torch.empty_like(x)
        idx = torch.empty((T, self.top_k), dtype=torch.int64, device=dev)
        w = torch.empty((T, self.top_k), dtype=torch.float16, device=dev)
        _capi.check("gemq_moe_decode", _capi.lib.gemq_moe_decode(
            C.byref(self._layer), x.data_ptr(), out.data_ptr(), idx.data_ptr(), w.data_ptr(), T, 1, route_mode,
            self._scratch.data_ptr(), self._scratch.numel(), stream_ptr(dev)))
        return out, w, idx

    def _scratch_word(self, fn) -> Tensor:
        off = fn(self._scratch.data_ptr()) - self._scratch.data_ptr()
        return self._scratch[off:off + 4].view(torch.int32)

    def decode_error_code(self, clear: bool = True) -> int:
        """Error word of the decode scratch (0 = every bounded wait was met and every expert id was
        in range); synchronises.  After a non-zero code call ``reset_decode_scratch``."""
        word = self._scratch_word(_capi.lib.gemq_workspace_error_word)
        code = int(word.item())
        if clear and code:
            word.zero_()
        return code

    def reset_decode_scratch(self) -> None:
        """Put the decode scratch back into its resting state (all zero)."""
        self._scratch.zero_()

    def _route(self, x: Tensor, mode: int, renorm: bool):
        return route_tokens(x, self.gate.weight, self.top_k, mode, renorm)

    def _prefill_ok(self) -> bool:
        D, Fd, G = self.hidden_dim, self.ffn_dim, self.block_group_size
        ok = D % 128 == 0 and Fd % 128 == 0 and G % 64 == 0 and self.top_k <= 8 and self.num_experts <= 256
        sf = self._layer.shared_ffn
        return ok and (sf == 0 or (sf % 128 == 0 and self.shared_group_size % 64 == 0))

    def _prefill(self, x: Tensor, route_mode: int, renorm: bool, routing=None):
        """``x [T, D]`` fp16/bf16 -> ``(out, weights, indices, logits)`` through the expert-sorted
        tcgen05 grouped GEMM; no host synchronisation.  ``routing = (weights [T, A] in x.dtype,
        indices int64 [T, A])`` skips the router."""
        if routing is None:
            return _moe_prefill(x, self._handle, route_mode, renorm)
        out = _moe_prefill_routed(x, routing[0], routing[1], self._handle, route_mode, renorm)
        return out, routing[0], routing[1], None

    def _prefill_impl(self, x: Tensor, route_mode: int, renorm: bool, routing=None):
        dev = require_cuda(x)
        x = x.contiguous()
        T = x.shape[0]
        bf = x.dtype == torch.bfloat16
        nbytes = _capi.lib.gemq_moe_prefill_scratch_bytes(C.byref(self._layer), T)
        if self._prefill_scratch is None or self._prefill_scratch.numel() < nbytes:
            self._prefill_scratch = torch.empty(nbytes, dtype=torch.uint8, device=dev)
        out = torch.empty_like(x)
        if routing is not None:
            w, idx = routing[0].contiguous(), routing[1].contiguous()
            logits = torch.empty((T, self.num_experts), dtype=torch.float32, device=dev)
            do_route = 0
        elif bf:  # the library's router reads the fp16 gate of the layer: route here with a bf16 copy
            w, idx, logits = self._route(x, route_mode, renorm)
            do_route = 0
        else:
            idx = torch.empty((T, self.top_k), dtype=torch.int64, device=dev)
            w = torch.empty((T, self.top_k), dtype=x.dtype, device=dev)
            logits = torch.empty((T, self.num_experts), dtype=torch.float32, device=dev)
            do_route = 1
        sc = self._prefill_scratch
        _capi.check("gemq_moe_prefill", _capi.lib.gemq_moe_prefill(
            C.byref(self._layer), x.data_ptr(), out.data_ptr(), idx.data_ptr(), w.data_ptr(), logits.data_ptr(),
            T, do_route, route_mode, int(bf), sc.data_ptr(), sc.numel(), stream_ptr(dev)))
        return out, w, idx, logits

    def prefill_error_code(self, tokens: int) -> int:
        """Error word of the last prefill with this many tokens (0 = no bounded wait expired); syncs."""
        p = _capi.lib.gemq_moe_prefill_error_word(C.byref(self._layer), tokens, self._prefill_scratch.data_ptr())
        off = p - self._prefill_scratch.data_ptr()
        return int(self._prefill_scratch[off:off + 4].view(torch.int32).item())

    def forward_single_expert(self, expert_idx: Tensor, hidden_states: Tensor) -> Tensor:
        """Expert FFN on ``[T, D]`` rows (gemq/inference/moe_block.py:146-163)."""
        x = hidden_states
        x1 = dequant_group_gemm(x, expert_idx, self.w1_wq, self.w1_scales, self.w1_zeros,
                                self.w1_nbits, self.w1_group_sizes, self.w1_wq_strides, self.w1_zs_strides)[0]
        x3 = dequant_group_gemm(x, expert_idx, self.w3_wq, self.w3_scales, self.w3_zeros,
                                self.w3_nbits, self.w3_group_sizes, self.w3_wq_strides, self.w3_zs_strides)[0]
        return dequant_group_gemm(F.silu(x1) * x3, expert_idx, self.w2_wq, self.w2_scales, self.w2_zeros,
                                  self.w2_nbits, self.w2_group_sizes, self.w2_wq_strides, self.w2_zs_strides)[0]

    def _unsupported(self, x: Tensor) -> ValueError:
        return ValueError(
            f"n-token forward needs hidden / intermediate sizes that are multiples of 128, a group size that is a "
            f"multiple of 64, at most 8 experts per token and 256 experts, and fp16 or bf16 activations; got hidden="
            f"{self.hidden_dim}, intermediate={self.ffn_dim}, group={self.block_group_size}, top_k={self.top_k}, "
            f"experts={self.num_experts}, dtype={x.dtype}")


def _fake_decode(x, handle, route_mode):
    k = _BLOCKS[handle].top_k
    return (torch.empty_like(x), x.new_empty((x.shape[0], k), dtype=torch.float16),
            x.new_empty((x.shape[0], k), dtype=torch.int64))


@library_op("moe_decode", _fake_decode)
def _moe_decode(x: Tensor, handle: int, route_mode: int) -> Tuple[Tensor, Tensor, Tensor]:
    return _BLOCKS[handle]._decode_impl(x, route_mode)


def _fake_prefill(x, handle, route_mode, renorm):
    blk = _BLOCKS[handle]
    T = x.shape[0]
    return (torch.empty_like(x), x.new_empty((T, blk.top_k)), x.new_empty((T, blk.top_k), dtype=torch.int64),
            x.new_empty((T, blk.num_experts), dtype=torch.float32))


@library_op("moe_prefill", _fake_prefill)
def _moe_prefill(x: Tensor, handle: int, route_mode: int, renorm: bool) -> Tuple[Tensor, Tensor, Tensor, Tensor]:
    return _BLOCKS[handle]._prefill_impl(x, route_mode, renorm)


@library_op("moe_prefill_routed", lambda x, w, idx, handle, route_mode, renorm: torch.empty_like(x))
def _moe_prefill_routed(x: Tensor, w: Tensor, idx: Tensor, handle: int, route_mode: int, renorm: bool) -> Tensor:
    return _BLOCKS[handle]._prefill_impl(x, route_mode, renorm, routing=(w, idx))[0]


class QuantFusedMixtralMoEBlock(_QuantFusedMoEBase):
    """Drop-in for gemq/inference/moe_block.py:73-240."""

    def __init__(self, config) -> None:
        super().__init__()
        self.hidden_dim = config.hidden_size
        self.ffn_dim = config.intermediate_size
        self.num_experts = config.num_local_experts
        self.top_k = config.num_experts_per_tok
        self.gate = nn.Linear(self.hidden_dim, self.num_experts, bias=False)

    @classmethod
    def from_hf(cls, config, hf_block):
        experts = list(hf_block.experts)
        if not is_packed_linear(experts[0].w1):
            raise ValueError("Expected linears in MixtralSparseMoeBlock. Please patch and replace them first.")
        return cls.from_linears(config, hf_block.gate.weight.data,
                                [e.w1 for e in experts], [e.w2 for e in experts], [e.w3 for e in experts])

    @classmethod
    def from_linears(cls, config, gate_weight: Tensor, w1, w2, w3):
        """Build from per-expert packed linears (lists of length ``num_local_experts``)."""
        blk = cls(config)
        blk.gate.weight.data = gate_weight.detach().clone()
        blk._check_group_sizes(w1, w2, w3)
        blk._stack("w1", w1)
        blk._stack("w2", w2)
        blk._stack("w3", w3)
        blk._build_layer(ROUTE_FP16, True, 0)
        return blk

    def forward_n_tokens(self, hidden_states: Tensor):
        """gemq/inference/moe_block.py:165-198."""
        b, s, d = hidden_states.shape
        x = hidden_states.reshape(-1, d)
        if self._prefill_ok() and x.dtype in (torch.float16, torch.bfloat16):
            out, _, _, logits = self._prefill(x, ROUTE_FP32_SOFTMAX, True)
            return out.reshape(b, s, d), logits.to(hidden_states.dtype)
        raise self._unsupported(x)

    def forward_one_token(self, hidden_states: Tensor):
        """gemq/inference/moe_block.py:200-235."""
        b, s, d = hidden_states.shape
        x = hidden_states.reshape(-1, self.hidden_dim)
        assert x.shape[0] == 1, f"This function only supports single token forward. But got {x.shape[0]} tokens."
        xh = x if x.dtype == torch.float16 else x.to(torch.float16)
        out, _, _ = self._decode(xh.contiguous(), ROUTE_FP16)
        return out.to(hidden_states.dtype).reshape(b, s, d), None

    def forward(self, hidden_states: Tensor):
        if hidden_states.shape[0] == hidden_states.shape[1] == 1:
            return self.forward_one_token(hidden_states)
        return self.forward_n_tokens(hidden_states)


class QuantFusedDeepseekV2MoEBlock(_QuantFusedMoEBase):
    """Drop-in for gemq/inference/moe_block.py:321-536."""

    def __init__(self, config) -> None:
        super().__init__()
        self.hidden_dim = config.hidden_size
        self.ffn_dim = config.moe_intermediate_size
        self.num_experts = config.n_routed_experts
        self.num_shared_experts = config.n_shared_experts
        self.top_k = config.num_experts_per_tok
        self.norm_topk_prob = config.norm_topk_prob
        self.gate = nn.Linear(self.hidden_dim, self.num_experts, bias=False)
        for p in self._projections:
            for suffix in ("wq", "scales", "zeros"):
                setattr(self, f"shared_{p}_{suffix}", None)
        self.shared_nbits, self.shared_group_size = None, None

    @classmethod
    def from_hf(cls, config, hf_block):
        experts = list(hf_block.experts)
        if not is_packed_linear(experts[0].gate_proj):
            raise ValueError("Expected linears in DeepseekV2MoE. Please patch and replace them first.")
        sh = hf_block.shared_experts
        return cls.from_linears(config, hf_block.gate.weight.data,
                                [e.gate_proj for e in experts], [e.down_proj for e in experts],
                                [e.up_proj for e in experts], (sh.gate_proj, sh.down_proj, sh.up_proj))

    @classmethod
    def from_linears(cls, config, gate_weight: Tensor, w1, w2, w3, shared):
        """``shared`` = (gate_proj, down_proj, up_proj) packed linears of the merged shared experts."""
        blk = cls(config)
        blk.gate.weight.data = gate_weight.detach().clone()
        blk._check_group_sizes(w1, w2, w3)
        blk._stack("w1", w1)
        blk._stack("w2", w2)
        blk._stack("w3", w3)
        s1, s2, s3 = shared
        for name, lin in (("w1", s1), ("w2", s2), ("w3", s3)):
            setattr(blk, f"shared_{name}_wq", lin.W_q.data.contiguous().clone())
            setattr(blk, f"shared_{name}_scales", lin.scales.data.contiguous().clone())
            setattr(blk, f"shared_{name}_zeros", lin.zeros.data.contiguous().clone())
        # the shared projections are assumed to share nbits and group size (moe_block.py:410-412)
        blk.shared_nbits, blk.shared_group_size = int(s1.W_nbits), int(s1.group_size)
        blk._build_layer(ROUTE_FP32, bool(blk.norm_topk_prob), blk.shared_w1_wq.shape[1])
        return blk

    def _shared_ffn(self, x: Tensor) -> Tensor:
        """gemq/inference/moe_block.py:419-430."""
        b, g = self.shared_nbits, self.shared_group_size
        x1 = dequant_gemm(x, self.shared_w1_wq, self.shared_w1_scales, self.shared_w1_zeros, b, g)
        x3 = dequant_gemm(x, self.shared_w3_wq, self.shared_w3_scales, self.shared_w3_zeros, b, g)
        return dequant_gemm(F.silu(x1) * x3, self.shared_w2_wq, self.shared_w2_scales, self.shared_w2_zeros, b, g)

    def forward_n_tokens(self, hidden_states: Tensor) -> Tensor:
        """gemq/inference/moe_block.py:448-486.  A handful of rows (decode batches) run the
        fused one-token kernels row by row with this path's fp32 routing."""
        b, s, d = hidden_states.shape
        x = hidden_states.reshape(-1, d)
        grouped = self._prefill_ok() and x.dtype in (torch.float16, torch.bfloat16)
        if x.shape[0] <= _MAX_LOOPED_TOKENS or (not grouped and x.shape[0] <= 16):
            xh = x if x.dtype == torch.float16 else x.to(torch.float16)
            out, _, _ = self._decode(xh.contiguous(), ROUTE_FP32)
            return out.to(hidden_states.dtype).reshape(b, s, d)
        if grouped:
            out, _, _, _ = self._prefill(x, ROUTE_FP32, bool(self.norm_topk_prob))
            return out.reshape(b, s, d)
        raise self._unsupported(x)

    def forward_one_token(self, hidden_states: Tensor) -> Tensor:
        """gemq/inference/moe_block.py:488-531."""
        b, s, d = hidden_states.shape
        x = hidden_states.reshape(-1, self.hidden_dim)
        assert x.shape[0] == 1, f"Only supports single token forward. Got {x.shape[0]} tokens."
        xh = x if x.dtype == torch.float16 else x.to(torch.float16)
        out, _, _ = self._decode(xh.contiguous(), ROUTE_FP32)
        return out.to(hidden_states.dtype).reshape(b, s, d)

    def forward(self, hidden_states: Tensor) -> Tensor:
        if hidden_states.shape[0] == hidden_states.shape[1] == 1:
            return self.forward_one_token(hidden_states)
        return self.forward_n_tokens(hidden_states)
