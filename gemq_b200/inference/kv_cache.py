"""Static key/value cache for the decode loop.

Same role and class names as gemq/inference/kv_cache.py:10-114 (``StaticLayer``,
``StaticCache(config, max_cache_len)``): buffers of the full length allocated on first use,
``update`` writes the new positions with ``index_copy_`` and returns the whole buffers, key and
value head sizes may differ (DeepSeek-V2's attention).  The buffers keep their addresses, so a
decode step can be captured in a CUDA graph.  This version stands on plain torch instead of the
transformers cache base classes.
"""
from __future__ import annotations

from typing import Any, Optional, Tuple

import torch
from torch import Tensor


class StaticLayer:
    is_compileable = True
    is_sliding = False

    def __init__(self, max_cache_len: int):
        self.max_cache_len = max_cache_len
        self.is_initialized = False
        self.keys: Optional[Tensor] = None
        self.values: Optional[Tensor] = None

    def lazy_initialization(self, key_states: Tensor, value_states: Tensor) -> None:
        b, h, _, kd = key_states.shape
        vd = value_states.shape[-1]
        self.keys = torch.zeros((b, h, self.max_cache_len, kd), dtype=key_states.dtype, device=key_states.device)
        self.values = torch.zeros((b, h, self.max_cache_len, vd), dtype=value_states.dtype, device=value_states.device)
        self.is_initialized = True

    def update(self, key_states: Tensor, value_states: Tensor,
               cache_kwargs: Optional[dict[str, Any]] = None) -> Tuple[Tensor, Tensor]:
        if not self.is_initialized:
            self.lazy_initialization(key_states, value_states)
        pos = cache_kwargs.get("cache_position") if cache_kwargs is not None else None
        if pos is None:
            pos = torch.arange(key_states.shape[-2], device=key_states.device)
        self.keys.index_copy_(2, pos, key_states)
        self.values.index_copy_(2, pos, value_states)
        return self.keys, self.values

    def get_mask_sizes(self, cache_position: Tensor) -> Tuple[int, int]:
        return self.max_cache_len, 0

    def get_seq_length(self) -> int:
        return int(self.keys[0, 0].any(dim=-1).sum()) if self.is_initialized else 0

    def get_max_cache_shape(self) -> int:
        return self.max_cache_len


class StaticCache:
    """One ``StaticLayer`` per decoder layer (``config.num_hidden_layers``)."""

    def __init__(self, config, max_cache_len: int, **kwargs):
        self.layers = [StaticLayer(max_cache_len) for _ in range(config.num_hidden_layers)]
        self.max_cache_len = max_cache_len

    def update(self, key_states: Tensor, value_states: Tensor, layer_idx: int,
               cache_kwargs: Optional[dict[str, Any]] = None) -> Tuple[Tensor, Tensor]:
        return self.layers[layer_idx].update(key_states, value_states, cache_kwargs)

    def get_seq_length(self, layer_idx: int = 0) -> int:
        return self.layers[layer_idx].get_seq_length()
