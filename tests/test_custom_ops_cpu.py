"""The library calls are torch.library custom operators: their fake implementations must give
the shapes and dtypes the real ones produce, so that torch.compile can trace through them
without a GPU in sight."""
import torch
from torch._subclasses.fake_tensor import FakeTensorMode

from gemq_b200 import kernels as K

E, D, Fd, A = 8, 4096, 14336, 2


def fake_inputs():
    h, i32, i64 = torch.float16, torch.int32, torch.int64
    x = torch.empty(1, D, dtype=h)
    wq = torch.empty(256, Fd, dtype=i32)
    sz = torch.empty(32, Fd, dtype=h)
    meta = torch.empty(E, dtype=i32)
    idx = torch.empty(A, dtype=i64)
    return x, wq, sz, meta, idx


def test_every_op_is_registered():
    for name in ("dequant_gemv_rows", "dequant_splitk_gemv", "dequant_sel_splitk_gemv", "fused_dequant_up_proj",
                 "fused_dequant_down_proj", "dequant_gemm", "dequant_group_gemm", "moe_route", "moe_decode",
                 "moe_prefill", "moe_prefill_routed"):
        assert hasattr(torch.ops.gemq_b200, name), name


def test_fake_shapes_and_dtypes():
    with FakeTensorMode():
        x, wq, sz, meta, idx = fake_inputs()
        y = K.dequant_splitk_gemv(x, wq, sz, sz, 2, 128)
        assert y.shape == (1, Fd) and y.dtype == torch.float16
        y = K.dequant_sel_splitk_gemv(x, idx[:1], wq, sz, sz, meta, meta, 128)
        assert y.shape == (1, Fd)
        x1, x3 = K.fused_dequant_up_proj(x, idx, wq, wq, sz, sz, sz, sz, meta, meta, 128)
        assert x1.shape == x3.shape == (1, A * Fd) and x1.dtype == torch.float16
        w2 = torch.empty(Fd // 16, D, dtype=torch.int32)
        s2 = torch.empty(Fd // 128, D, dtype=torch.float16)
        x2 = K.fused_dequant_down_proj(x1, x3, idx, w2, s2, s2, meta, meta, 128)
        assert x2.shape == (1, A * D)
        for M, dt, want in ((7, torch.float16, torch.float16), (200, torch.float16, torch.float16),
                            (200, torch.bfloat16, torch.bfloat16)):
            y = K.dequant_gemm(torch.empty(M, D, dtype=dt), wq, sz, sz, 2, 128)
            assert y.shape == (M, Fd) and y.dtype == want
        y = K.dequant_group_gemm(torch.empty(50, D, dtype=torch.float16), idx, wq, sz, sz, meta, meta, meta, meta)
        assert y.shape == (A, 50, Fd) and y.dtype == torch.float16
        from gemq_b200.inference.moe_block import route_tokens
        w, i, logits = route_tokens(torch.empty(5, D, dtype=torch.bfloat16), torch.empty(E, D, dtype=torch.bfloat16), A, 1, True)
        assert w.shape == (5, A) and w.dtype == torch.bfloat16 and i.dtype == torch.int64 and logits.shape == (5, E)
