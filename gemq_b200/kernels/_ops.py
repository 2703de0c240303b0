"""Registration of the library calls as ``torch.library`` custom operators.

The reference runs its decode step under ``torch.compile(mode="reduce-overhead",
fullgraph=True)`` (gemq/benchmark_generate.py:158-160).  A ctypes call is opaque to dynamo, so
every public op is a custom operator with a fake (meta) implementation: tracing sees an
operator with known output shapes and dtypes, and the real implementation -- argument checks
plus the C-ABI call on the current stream -- runs at execution (and CUDA-graph capture) time.
"""
from __future__ import annotations

import torch

NAMESPACE = "gemq_b200"


def library_op(name: str, fake):
    """``@library_op("name", fake_fn)``: register ``fn`` as ``gemq_b200::name`` (no argument is
    mutated, outputs are fresh tensors) with ``fake_fn`` as its shape/dtype propagation."""
    def deco(fn):
        op = torch.library.custom_op(f"{NAMESPACE}::{name}", mutates_args=())(fn)
        op.register_fake(fake)
        return op
    return deco
