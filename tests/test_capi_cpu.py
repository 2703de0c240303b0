"""Host-side checks that need no GPU: the library loads, exports what the header declares,
and the wrappers refuse CPU tensors instead of falling back."""
import os
import re

import pytest
import torch

from conftest import ROOT


def _declared():
    text = open(os.path.join(ROOT, "include", "gemq_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(gemq_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    from gemq_b200 import _capi
    names = _declared()
    assert len(names) >= 10
    for n in names:
        assert hasattr(_capi.lib, n), f"{n} declared in include/gemq_b200.h but not exported"
    assert sorted(_capi.EXPORTED) == names, "ctypes signature table and header disagree"
    assert b"sm_100a" in _capi.lib.gemq_version()


def test_workspace_size_is_monotone():
    from gemq_b200 import _capi
    f = _capi.lib.gemq_gemv_workspace_bytes
    assert f(0, 128, 1) == 0
    assert f(4096, 4096, 1) < f(8192, 4096, 1) < f(8192, 14336, 1) < f(8192, 14336, 2)


def test_ops_refuse_cpu_tensors():
    from gemq_b200.kernels import dequant_splitk_gemv, pack_weights_over_cols
    with pytest.raises(RuntimeError, match="CUDA"):
        pack_weights_over_cols(torch.zeros(4, 32, dtype=torch.uint8), 2)
    with pytest.raises(RuntimeError, match="CUDA"):
        dequant_splitk_gemv(torch.zeros(1, 128, dtype=torch.float16), torch.zeros(8, 32, dtype=torch.int32),
                            torch.zeros(1, 32, dtype=torch.float16), torch.zeros(1, 32, dtype=torch.float16), 2, 128)


def test_expert_bit_draw_respects_mean():
    from gemq_b200.synth import draw_expert_bits
    for seed in range(5):
        bits = draw_expert_bits(8, seed)
        assert set(bits) <= {1, 2, 3, 4} and 1.5 <= sum(bits) / 8 <= 2.5
    assert draw_expert_bits(64, 3) == draw_expert_bits(64, 3)
