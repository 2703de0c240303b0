"""Generate golden vectors by running the reference's own Triton kernels on the CPU.

Run once, in a container that has the reference checkout (it is not needed at
test time):

    python tests/golden/make_golden.py /path/to/reference

The reference kernels (gemq/triton_kernels/*.py) import with torch+triton only
and execute on CPU tensors under ``TRITON_INTERPRET=1`` once every autotuner is
pinned to a single configuration.  Inputs are seeded and stored together with
the outputs in ``tests/golden/reference_kernels.npz`` so the tests need neither
the reference nor triton.
"""
import os
import sys

os.environ["TRITON_INTERPRET"] = "1"
sys.dont_write_bytecode = True
if len(sys.argv) < 2:
    sys.exit("usage: python tests/golden/make_golden.py <path to a GEMQ checkout>")
ref_root = sys.argv[1]
sys.path.insert(0, ref_root)

import numpy as np  # noqa: E402
import torch  # noqa: E402
import triton  # noqa: E402

from gemq.triton_kernels import utils as U  # noqa: E402
from gemq.triton_kernels import dequant_gemv as GV  # noqa: E402
from gemq.triton_kernels import dequant_gemm as GM  # noqa: E402
from gemq.triton_kernels import dequant_group_gemm as GG  # noqa: E402
from gemq.triton_kernels import fused_dequant_bmm as FB  # noqa: E402

GV.dequant_splitk_gemv_kernel.configs = [triton.Config({"BLOCK_SIZE_N": 64, "BLOCK_SIZE_K": 64})]
GV.dequant_sel_splitk_gemv_kernel.configs = [triton.Config({"BLOCK_SIZE_N": 64, "BLOCK_SIZE_K": 64})]
GM.dequant_gemm_kernel.configs = [triton.Config({"BLOCK_SIZE_M": 32, "BLOCK_SIZE_N": 32, "BLOCK_SIZE_K": 32})]
GG.dequant_group_gemm_kernel.configs = [
    triton.Config({"BLOCK_SIZE_M": 16, "BLOCK_SIZE_N": 32, "BLOCK_SIZE_K": 32, "NUM_SM": 4})]
FB.fused_dequant_up_proj_kernel.configs = [triton.Config({"BLOCK_SIZE_N": 32, "BLOCK_SIZE_K": 128})]
FB.fused_dequant_down_proj_kernel.configs = [triton.Config({"BLOCK_SIZE_N": 32, "BLOCK_SIZE_K": 128})]

out = {}
gen = torch.Generator().manual_seed(1234)


def rand_codes(n, k, b):
    return torch.randint(0, 2 ** b, (n, k), dtype=torch.uint8, generator=gen)


def rand_meta(groups, n, b):
    scale = (torch.randn(groups, n, generator=gen).abs() * 0.01 + 1e-3).half()
    zero_point = (torch.rand(groups, n, generator=gen) * (2 ** b - 1)).half()
    offset = (-(zero_point.float() * scale.float())).half()
    return scale, offset


def packed(q, b):
    w, _ = U.pack_weights_over_cols_triton(q, b, 32, True)
    return w.contiguous()


# 1. pack / unpack, including non-divisible column counts
for b in (1, 2, 3, 4):
    q = rand_codes(16, 50, b)
    w, eps = U.pack_weights_over_cols_triton(q, b, 32, False)
    out[f"pack{b}_q"] = q.numpy()
    out[f"pack{b}_w"] = w.numpy()
    back = U.unpack_over_cols_triton(w, b, 32, 50)
    out[f"unpack{b}_q"] = back.numpy()
    assert torch.equal(back, q)

# 2. split-K GEMV, every bit-width, two group sizes
for b in (1, 2, 3, 4):
    for G in (128, 64):
        N, K = 64, 256
        q = rand_codes(N, K, b)
        s, z = rand_meta(K // G, N, b)
        x = torch.randn(1, K, generator=gen).half()
        w = packed(q, b)
        y = GV.dequant_splitk_gemv_triton(x, w, s, z, b, G)
        key = f"gemv{b}_g{G}"
        out.update({key + "_q": q.numpy(), key + "_w": w.numpy(), key + "_s": s.numpy(),
                    key + "_z": z.numpy(), key + "_x": x.numpy(), key + "_y": y.numpy()})

# 3. stacked experts with mixed bits: selected GEMV, fused up/down, grouped GEMM
bits = [1, 2, 3, 4]
E, A, K, N, G = 4, 2, 256, 128, 128


def stack(kdim, ndim):
    ws, ss, zs = [], [], []
    for b in bits:
        q = rand_codes(ndim, kdim, b)
        s, z = rand_meta(kdim // G, ndim, b)
        ws.append(packed(q, b)); ss.append(s); zs.append(z)
    wq = torch.cat(ws); sc = torch.cat(ss); ze = torch.cat(zs)
    cs = lambda v: torch.tensor([0] + v, dtype=torch.int32).cumsum(0)[:-1].to(torch.int32)
    return wq, sc, ze, cs([w.numel() for w in ws]), cs([s.numel() for s in ss])


nb = torch.tensor(bits, dtype=torch.int32)
gs = torch.full((E,), G, dtype=torch.int32)
w1, s1, z1, w1_str, z1_str = stack(K, N)
w3, s3, z3, _, _ = stack(K, N)
w2, s2, z2, w2_str, z2_str = stack(N, K)      # down projection: in=N(ffn), out=K(hidden)
x = torch.randn(1, K, generator=gen).half()
for name, v in dict(w1=w1, s1=s1, z1=z1, w3=w3, s3=s3, z3=z3, w2=w2, s2=s2, z2=z2, w1_str=w1_str,
                    z1_str=z1_str, w2_str=w2_str, z2_str=z2_str, nbits=nb, gsz=gs, x=x).items():
    out["stk_" + name] = v.numpy()

for e in range(E):
    idx1 = torch.tensor([e], dtype=torch.int64)
    out[f"stk_sel{e}_y"] = GV.dequant_sel_splitk_gemv_triton(x, idx1, w1, s1, z1, nb, w1_str, G).numpy()

for tag, sel in (("a", [3, 0]), ("b", [1, 2])):
    idx = torch.tensor(sel, dtype=torch.int64)
    x1, x3 = FB.fused_dequant_up_proj_triton(x, idx, w1, w3, s1, z1, s3, z3, nb, w1_str, G)
    x2 = FB.fused_dequant_down_proj_triton(x1, x3, idx, w2, s2, z2, nb, w2_str, G)
    out[f"stk_{tag}_idx"] = idx.numpy()
    out[f"stk_{tag}_x1"] = x1.numpy(); out[f"stk_{tag}_x3"] = x3.numpy(); out[f"stk_{tag}_x2"] = x2.numpy()

xm = torch.randn(7, K, generator=gen).half()
out["stk_xm"] = xm.numpy()
idx = torch.tensor([2, 1], dtype=torch.int64)
out["stk_gg_idx"] = idx.numpy()
out["stk_gg_y"] = GG.dequant_group_gemm_triton(xm, idx, w1, s1, z1, nb, gs, w1_str, z1_str).numpy()

# 4. dense GEMM
for b in (3, 4):
    M, N2, K2 = 5, 64, 256
    q = rand_codes(N2, K2, b)
    s, z = rand_meta(K2 // G, N2, b)
    xx = torch.randn(M, K2, generator=gen).half()
    w = packed(q, b)
    y = GM.dequant_gemm_triton(xx, w, s, z, b, G)
    key = f"gemm{b}"
    out.update({key + "_w": w.numpy(), key + "_s": s.numpy(), key + "_z": z.numpy(),
                key + "_x": xx.numpy(), key + "_y": y.numpy()})

dst = os.path.join(os.path.dirname(os.path.abspath(__file__)), "reference_kernels.npz")
np.savez_compressed(dst, **out)
print("wrote", dst, os.path.getsize(dst), "bytes,", len(out), "arrays")
