"""Swap a loaded model's HQQ linears and MoE blocks for this library's, by the reference's names.

Same entry points as gemq/inference/patch.py: ``create_gemlite_from_hqq`` (here it returns a
``QuantLinear`` on this library's kernels; gemlite is not involved), ``replace_linear_recursive``,
``replace_moe_blocks`` and ``prepare_for_inference``.  An HQQ linear is recognised by what the
reference reads from it (gemq/inference/patch.py:26-37): packed ``W_q``, a ``meta`` dict with
``shape / nbits / group_size / axis / scale / zero`` and an optional ``bias``; hqq itself is not
imported.  Only the quantised path exists: ``is_fp=True`` (the reference's un-quantised fused
blocks) raises.
"""
from __future__ import annotations

import gc

import torch

from ..quant.hqq_format import packed_linear_from_hqq
from .moe_block import QuantFusedDeepseekV2MoEBlock, QuantFusedMixtralMoEBlock
from .quant_linear import QuantLinear

_MIXTRAL_NAMES = ("mixtral",)
_DEEPSEEK_NAMES = ("deepseek",)


def is_hqq_linear(m) -> bool:
    meta = getattr(m, "meta", None)
    return hasattr(m, "W_q") and isinstance(meta, dict) and all(k in meta for k in ("shape", "nbits", "group_size", "axis"))


def create_gemlite_from_hqq(hqq_layer, **kwargs) -> QuantLinear:
    """One HQQ linear -> a quantised linear in kernel form (gemq/inference/patch.py:23-68)."""
    device = kwargs.get("device", hqq_layer.W_q.device)
    meta = hqq_layer.meta
    packed = packed_linear_from_hqq(hqq_layer.W_q.to(device), {**meta, "scale": meta["scale"].to(device),
                                                                "zero": meta["zero"].to(device)})
    bias = getattr(hqq_layer, "bias", None)
    return QuantLinear(packed, bias.clone().to(device) if bias is not None else None)


def replace_linear_recursive(module, **kwargs) -> None:
    """Replace all HQQ linears below ``module`` (gemq/inference/patch.py:71-79)."""
    for name, child in list(module.named_children()):
        if is_hqq_linear(child):
            setattr(module, name, create_gemlite_from_hqq(child, **kwargs))
        else:
            replace_linear_recursive(child, **kwargs)


def _decoder_layers(model):
    inner = getattr(model, "model", model)
    return inner.layers


def replace_moe_blocks(model, model_name: str, config, is_fp: bool = False) -> None:
    """Replace the MoE blocks of a Mixtral or DeepSeek-V2 model (gemq/inference/patch.py:82-125)."""
    if is_fp:
        raise NotImplementedError("only the quantised blocks exist in this library")
    name = model_name.lower()
    layers = _decoder_layers(model)
    for i, layer in enumerate(layers):
        if any(k in name for k in _MIXTRAL_NAMES):
            org = layer.block_sparse_moe
            layer.block_sparse_moe = QuantFusedMixtralMoEBlock.from_hf(config, org)
        elif any(k in name for k in _DEEPSEEK_NAMES):
            if i == 0:  # the first layer of this model is dense (gemq/inference/patch.py:122-123)
                continue
            org = layer.mlp
            layer.mlp = QuantFusedDeepseekV2MoEBlock.from_hf(config, org)
        else:
            raise NotImplementedError(model_name)
        del org
        gc.collect()
        if torch.cuda.is_available():
            torch.cuda.empty_cache()


def prepare_for_inference(model, model_name: str, is_fp: bool = False):
    """HQQ linears -> quantised linears, then fused MoE blocks (gemq/inference/patch.py:128-144)."""
    if is_fp:
        raise NotImplementedError("only the quantised blocks exist in this library")
    replace_linear_recursive(model)
    replace_moe_blocks(model, model_name, model.config, is_fp=False)
    gc.collect()
    if torch.cuda.is_available():
        torch.cuda.empty_cache()
    return model
