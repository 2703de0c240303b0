"""The CPU oracle against the golden vectors produced by the reference's own kernels."""
import numpy as np
import pytest

from oracle import gemq_oracle as O
from conftest import rel_fro, max_abs

# The reference kernels round to fp16 at the end and (for split-K) through fp16
# atomics, so agreement with the oracle is to fp16 resolution, not bit-exact.
TOL_FRO = 1.5e-3
TOL_ABS = 8e-3


@pytest.mark.parametrize("b", [1, 2, 3, 4])
def test_pack_unpack_bit_exact(golden, b):
    q = golden[f"pack{b}_q"]
    assert np.array_equal(O.pack_over_cols(q, b), golden[f"pack{b}_w"])
    assert np.array_equal(O.unpack_over_cols(golden[f"pack{b}_w"], b, q.shape[1]), golden[f"unpack{b}_q"])


@pytest.mark.parametrize("b", [1, 2, 3, 4])
@pytest.mark.parametrize("G", [128, 64])
def test_gemv(golden, b, G):
    k = f"gemv{b}_g{G}"
    w = golden[k + "_w"]
    assert np.array_equal(O.pack_kernel_form(golden[k + "_q"], b), w)
    K = golden[k + "_x"].shape[1]
    assert np.array_equal(O.unpack_kernel_form(w, b, K), golden[k + "_q"].T)
    y = O.dequant_gemv(golden[k + "_x"], w, golden[k + "_s"], golden[k + "_z"], b, G)
    assert rel_fro(y, golden[k + "_y"]) < TOL_FRO
    assert max_abs(y, golden[k + "_y"]) < TOL_ABS


def test_dequantize_single_rounding():
    # q*s+z where double rounding (f64 -> f32 -> f16) would differ from one rounding
    rng = np.random.default_rng(0)
    K, N, b, G = 128, 32, 4, 128
    q = rng.integers(0, 16, (N, K), dtype=np.uint8)
    s = rng.standard_normal((1, N)).astype(np.float16)
    z = rng.standard_normal((1, N)).astype(np.float16)
    w = O.dequantize(O.pack_kernel_form(q, b), s, z, b, G, K)
    exact = q.T.astype(np.float64) * s.astype(np.float64) + z.astype(np.float64)
    assert np.array_equal(w, exact.astype(np.float16))
    assert w.dtype == np.float16


@pytest.mark.parametrize("e", [0, 1, 2, 3])
def test_sel_gemv(golden, e):
    g = golden
    y = O.dequant_sel_gemv(g["stk_x"], np.array([e]), g["stk_w1"], g["stk_s1"], g["stk_z1"],
                           g["stk_nbits"], g["stk_w1_str"], 128)
    assert rel_fro(y, g[f"stk_sel{e}_y"]) < TOL_FRO


@pytest.mark.parametrize("tag", ["a", "b"])
def test_fused_up_down(golden, tag):
    g = golden
    idx = g[f"stk_{tag}_idx"]
    x1, x3 = O.fused_up_proj(g["stk_x"], idx, g["stk_w1"], g["stk_w3"], g["stk_s1"], g["stk_z1"],
                             g["stk_s3"], g["stk_z3"], g["stk_nbits"], g["stk_w1_str"], 128)
    assert rel_fro(x1, g[f"stk_{tag}_x1"]) < TOL_FRO
    assert rel_fro(x3, g[f"stk_{tag}_x3"]) < TOL_FRO
    # down projection from the reference's own x1/x3 so only this op is compared
    x2 = O.fused_down_proj(g[f"stk_{tag}_x1"], g[f"stk_{tag}_x3"], idx, g["stk_w2"], g["stk_s2"], g["stk_z2"],
                           g["stk_nbits"], g["stk_w2_str"], 128)
    assert rel_fro(x2, g[f"stk_{tag}_x2"]) < TOL_FRO
    assert max_abs(x2, g[f"stk_{tag}_x2"]) < TOL_ABS


def test_group_gemm(golden):
    g = golden
    y = O.dequant_group_gemm(g["stk_xm"], g["stk_gg_idx"], g["stk_w1"], g["stk_s1"], g["stk_z1"], g["stk_nbits"],
                             g["stk_gsz"], g["stk_w1_str"], g["stk_z1_str"])
    assert y.shape == g["stk_gg_y"].shape
    assert rel_fro(y, g["stk_gg_y"]) < TOL_FRO


@pytest.mark.parametrize("b", [3, 4])
def test_gemm(golden, b):
    k = f"gemm{b}"
    y = O.dequant_gemm(golden[k + "_x"], golden[k + "_w"], golden[k + "_s"], golden[k + "_z"], b, 128)
    assert rel_fro(y, golden[k + "_y"]) < TOL_FRO
