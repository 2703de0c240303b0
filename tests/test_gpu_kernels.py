"""Parity of the CUDA kernels (through the C ABI) with the golden vectors of the reference
kernels and with the CPU oracle.  Integer / de-quantised results are bit-exact; GEMV-type
outputs are within max-abs 2e-2 and relative Frobenius 5e-3 of fp32-accumulated results."""
import numpy as np
import pytest
import torch

from oracle import gemq_oracle as O
from conftest import MAX_ABS_TOL, REL_FRO_TOL, max_abs, rel_fro

pytestmark = pytest.mark.gpu
DEV = "cuda"


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).to(DEV)


def close(got, want):
    got = got.float().cpu().numpy() if isinstance(got, torch.Tensor) else got
    assert rel_fro(got, want) < REL_FRO_TOL, f"rel-Frobenius {rel_fro(got, want):.3e}"
    assert max_abs(got, want) < MAX_ABS_TOL, f"max-abs {max_abs(got, want):.3e}"


def rand_matrix(rng, N, K, b, G):
    q = rng.integers(0, 2 ** b, (N, K), dtype=np.uint8)
    s = (np.abs(rng.standard_normal((K // G, N))) * 0.01 + 1e-3).astype(np.float16)
    zp = (rng.random((K // G, N)) * (2 ** b - 1)).astype(np.float16)
    return q, O.pack_kernel_form(q, b), s, O.kernel_form_offset(s, zp)


@pytest.mark.parametrize("b", [1, 2, 3, 4])
def test_pack_unpack_golden(golden, b):
    from gemq_b200.kernels import pack_weights_over_cols, unpack_over_cols
    q = golden[f"pack{b}_q"]
    w, eps = pack_weights_over_cols(dev(q), b, 32, transpose=False)
    assert eps == 32 // b
    assert np.array_equal(w.cpu().numpy(), golden[f"pack{b}_w"])
    wt, _ = pack_weights_over_cols(dev(q), b)
    assert wt.shape == (w.shape[1], w.shape[0]) and torch.equal(wt.contiguous(), w.t().contiguous())
    back = unpack_over_cols(dev(golden[f"pack{b}_w"]), b, 32, q.shape[1])
    assert np.array_equal(back.cpu().numpy(), golden[f"unpack{b}_q"])


@pytest.mark.parametrize("b", [1, 2, 3, 4])
@pytest.mark.parametrize("shape", [(64, 256), (96, 1408), (33, 70)])
def test_pack_kernel_form_and_roundtrip(b, shape):
    from gemq_b200.kernels import pack_kernel_form, unpack_over_cols
    N, K = shape
    rng = np.random.default_rng(b * 100 + N)
    q = rng.integers(0, 2 ** b, (N, K), dtype=np.uint8)
    w = pack_kernel_form(dev(q), b)
    assert np.array_equal(w.cpu().numpy(), O.pack_kernel_form(q, b))
    back = unpack_over_cols(w.t().contiguous(), b, 32, K)
    assert np.array_equal(back.cpu().numpy(), q)


@pytest.mark.parametrize("b", [1, 2, 3, 4])
@pytest.mark.parametrize("G", [128, 64])
def test_dequantize_bit_exact(b, G):
    from gemq_b200.kernels import dequantize
    rng = np.random.default_rng(7 + b)
    N, K = 96, 640
    q, w, s, z = rand_matrix(rng, N, K, b, G)
    # wide-range metadata so that rounding of q*s+z is exercised
    s = rng.standard_normal((K // G, N)).astype(np.float16)
    z = rng.standard_normal((K // G, N)).astype(np.float16)
    got = dequantize(dev(w), dev(s), dev(z), b, G).cpu().numpy()
    want = O.dequantize(w, s, z, b, G, K)
    assert np.array_equal(got.view(np.uint16), want.view(np.uint16))


@pytest.mark.parametrize("b", [1, 2, 3, 4])
@pytest.mark.parametrize("G", [128, 64])
def test_gemv_golden(golden, b, G):
    from gemq_b200.kernels import dequant_splitk_gemv
    k = f"gemv{b}_g{G}"
    y = dequant_splitk_gemv(dev(golden[k + "_x"]), dev(golden[k + "_w"]), dev(golden[k + "_s"]),
                            dev(golden[k + "_z"]), b, G)
    close(y, golden[k + "_y"].astype(np.float32))
    close(y, O.dequant_gemv(golden[k + "_x"], golden[k + "_w"], golden[k + "_s"], golden[k + "_z"], b, G))


@pytest.mark.parametrize("b", [1, 2, 3, 4])
@pytest.mark.parametrize("NK", [(2816, 2048), (2048, 1408), (160, 4096), (4096, 14336)])
@pytest.mark.parametrize("M", [1, 2, 3, 7, 9])
def test_gemv_rows_vs_oracle(b, NK, M):
    from gemq_b200.kernels import dequant_gemv_rows
    N, K = NK
    if M > 1 and K > 4096:
        pytest.skip("large-K multi-row case covered by smaller K")
    rng = np.random.default_rng(b * 1000 + N + M)
    q, w, s, z = rand_matrix(rng, N, K, b, 128)
    x = rng.standard_normal((M, K)).astype(np.float16)
    wd, sd, zd, xd = dev(w), dev(s), dev(z), dev(x)
    y = dequant_gemv_rows(xd, wd, sd, zd, b, 128)
    want = O.dequant_gemv(x, w, s, z, b, 128) if M == 1 else O.dequant_gemm(x, w, s, z, b, 128)
    close(y, want)
    y2 = dequant_gemv_rows(xd, wd, sd, zd, b, 128)
    assert torch.equal(y, y2), "split-K reduction must be deterministic"


def test_gemv_config0_full_size():
    """Single 2-bit expert GEMV, 14336 x 4096, group 128, seed 0."""
    from gemq_b200.kernels import dequant_splitk_gemv
    rng = np.random.default_rng(0)
    N, K, b = 14336, 4096, 2
    q, w, s, z = rand_matrix(rng, N, K, b, 128)
    x = rng.standard_normal((1, K)).astype(np.float16)
    y = dequant_splitk_gemv(dev(x), dev(w), dev(s), dev(z), b, 128)
    close(y, O.dequant_gemv(x, w, s, z, b, 128))


def test_gemv_small_and_large_activations():
    """The per-slice power-of-two scaling keeps precision for tiny and huge activations."""
    from gemq_b200.kernels import dequant_splitk_gemv
    rng = np.random.default_rng(5)
    N, K, b = 64, 1024, 2
    q, w, s, z = rand_matrix(rng, N, K, b, 128)
    for scale in (1e-4, 3e2):
        x = (rng.standard_normal((1, K)) * scale).astype(np.float16)
        y = dequant_splitk_gemv(dev(x), dev(w), dev(s), dev(z), b, 128).float().cpu().numpy()
        want = O.dequant_gemv(x, w, s, z, b, 128).astype(np.float32)
        assert rel_fro(y, want) < REL_FRO_TOL


@pytest.mark.parametrize("e", [0, 1, 2, 3])
def test_sel_gemv_golden(golden, e):
    from gemq_b200.kernels import dequant_sel_splitk_gemv
    g = golden
    y = dequant_sel_splitk_gemv(dev(g["stk_x"]), torch.tensor([e], device=DEV), dev(g["stk_w1"]), dev(g["stk_s1"]),
                                dev(g["stk_z1"]), dev(g["stk_nbits"]), dev(g["stk_w1_str"]), 128)
    close(y, g[f"stk_sel{e}_y"].astype(np.float32))


@pytest.mark.parametrize("tag", ["a", "b"])
def test_fused_up_down_golden(golden, tag):
    from gemq_b200.kernels import fused_dequant_down_proj, fused_dequant_up_proj
    g = golden
    idx = dev(g[f"stk_{tag}_idx"])
    x1, x3 = fused_dequant_up_proj(dev(g["stk_x"]), idx, dev(g["stk_w1"]), dev(g["stk_w3"]), dev(g["stk_s1"]),
                                   dev(g["stk_z1"]), dev(g["stk_s3"]), dev(g["stk_z3"]), dev(g["stk_nbits"]),
                                   dev(g["stk_w1_str"]), 128)
    close(x1, g[f"stk_{tag}_x1"].astype(np.float32))
    close(x3, g[f"stk_{tag}_x3"].astype(np.float32))
    x2 = fused_dequant_down_proj(dev(g[f"stk_{tag}_x1"]), dev(g[f"stk_{tag}_x3"]), idx, dev(g["stk_w2"]),
                                 dev(g["stk_s2"]), dev(g["stk_z2"]), dev(g["stk_nbits"]), dev(g["stk_w2_str"]), 128)
    close(x2, g[f"stk_{tag}_x2"].astype(np.float32))


def test_group_gemm_and_gemm_golden(golden):
    from gemq_b200.kernels import dequant_gemm, dequant_group_gemm
    g = golden
    y = dequant_group_gemm(dev(g["stk_xm"]), dev(g["stk_gg_idx"]), dev(g["stk_w1"]), dev(g["stk_s1"]),
                           dev(g["stk_z1"]), dev(g["stk_nbits"]), dev(g["stk_gsz"]), dev(g["stk_w1_str"]),
                           dev(g["stk_z1_str"]))
    assert tuple(y.shape) == g["stk_gg_y"].shape
    close(y, g["stk_gg_y"].astype(np.float32))
    for b in (3, 4):
        k = f"gemm{b}"
        y = dequant_gemm(dev(g[k + "_x"]), dev(g[k + "_w"]), dev(g[k + "_s"]), dev(g[k + "_z"]), b, 128)
        close(y, g[k + "_y"].astype(np.float32))


def test_gemm_many_rows_vs_oracle():
    from gemq_b200.kernels import dequant_gemm
    rng = np.random.default_rng(11)
    N, K, b, M = 256, 512, 3, 150
    q, w, s, z = rand_matrix(rng, N, K, b, 128)
    x = rng.standard_normal((M, K)).astype(np.float16)
    close(dequant_gemm(dev(x), dev(w), dev(s), dev(z), b, 128), O.dequant_gemm(x, w, s, z, b, 128))
