"""gemq_dequant_gemv_static: the GEMV entry point for hosts that cannot allocate.

A serving process with a frozen memory pool, or a plugin inside a runtime that forbids
cudaMalloc once the model is loaded, cannot hand the library the zero-filled workspace that
gemq_dequant_gemv needs.  The static variant keeps that scratch in a fixed 2 MiB device array
inside the library.  This test drives it through the C ABI, twice in a row (the array keeps the
first call's leftovers), and compares with gemq_dequant_gemv on a caller-provided workspace.
It lives in the file pytest collects last so that a failure here cannot hide another test.
"""
import numpy as np
import pytest
import torch

from oracle import gemq_oracle as O
from conftest import MAX_ABS_TOL, REL_FRO_TOL, max_abs, rel_fro

pytestmark = pytest.mark.gpu


def _problem(seed, N, K, b):
    rng = np.random.default_rng(seed)
    q = rng.integers(0, 2 ** b, (N, K), dtype=np.uint8)
    s = (np.abs(rng.standard_normal((K // 128, N))) * 0.01 + 1e-3).astype(np.float16)
    z = O.kernel_form_offset(s, (rng.random((K // 128, N)) * (2 ** b - 1)).astype(np.float16))
    x = rng.standard_normal((1, K)).astype(np.float16)
    dev = lambda a: torch.from_numpy(np.ascontiguousarray(a)).cuda()
    return dev(O.pack_kernel_form(q, b)), dev(s), dev(z), dev(x)


def test_static_scratch_gemv_matches_workspace_gemv_twice():
    from gemq_b200 import _capi
    from gemq_b200.kernels import dequant_splitk_gemv
    lib = _capi.lib
    stream = torch.cuda.current_stream().cuda_stream
    assert lib.gemq_static_scratch_bytes() == 2 << 20
    # two different problems back to back: the second call finds the first call's leftovers
    for seed, (N, K, b) in enumerate([(2048, 4096, 2), (4096, 1408, 3)]):
        wq, s, z, x = _problem(seed, N, K, b)
        want = dequant_splitk_gemv(x, wq, s, z, b, 128)          # existing entry point, own workspace
        got = torch.empty((1, N), dtype=torch.float16, device="cuda")
        rc = lib.gemq_dequant_gemv_static(x.data_ptr(), wq.data_ptr(), s.data_ptr(), z.data_ptr(), got.data_ptr(),
                                          N, K, b, 128, stream)
        assert rc == 0
        torch.cuda.synchronize()
        g, w = got.float().cpu().numpy(), want.float().cpu().numpy()
        assert rel_fro(g, w) < REL_FRO_TOL and max_abs(g, w) < MAX_ABS_TOL
        assert torch.equal(got, want)  # same kernel, same fixed summation order
        ref = O.dequant_gemv(x.cpu().numpy(), wq.cpu().numpy(), s.cpu().numpy(), z.cpu().numpy(), b, 128)
        assert rel_fro(g, ref) < REL_FRO_TOL and max_abs(g, ref) < MAX_ABS_TOL  # and the oracle agrees


@pytest.mark.parametrize("case", ["unaligned_x", "n_not_multiple_of_32", "group_64"])
def test_static_scratch_gemv_fallback_shapes(case):
    """Shapes the persistent kernel does not take reach the other kernels behind the same entry
    point: an activation that is not 16-byte aligned, an N that is not a multiple of 32, a group
    size of 64.  Each must match gemq_dequant_gemv on a caller workspace."""
    from gemq_b200 import _capi
    from gemq_b200.kernels._runtime import gemv_workspace
    lib = _capi.lib
    stream = torch.cuda.current_stream().cuda_stream
    N, K, b, G = (2048, 1024, 2, 128)
    if case == "n_not_multiple_of_32":
        N = 2000
    if case == "group_64":
        G = 64
    rng = np.random.default_rng(7)
    q = rng.integers(0, 2 ** b, (N, K), dtype=np.uint8)
    s = (np.abs(rng.standard_normal((K // G, N))) * 0.01 + 1e-3).astype(np.float16)
    z = O.kernel_form_offset(s, (rng.random((K // G, N)) * (2 ** b - 1)).astype(np.float16))
    dev = lambda a: torch.from_numpy(np.ascontiguousarray(a)).cuda()
    wq, s, z = dev(O.pack_kernel_form(q, b)), dev(s), dev(z)
    xbuf = dev(rng.standard_normal(K + 8).astype(np.float16))
    x = xbuf[1:1 + K] if case == "unaligned_x" else xbuf[:K]
    assert (x.data_ptr() % 16 != 0) == (case == "unaligned_x")
    got = torch.empty((1, N), dtype=torch.float16, device="cuda")
    want = torch.empty((1, N), dtype=torch.float16, device="cuda")
    ws = gemv_workspace(got.device, N, K, 1)
    rc = lib.gemq_dequant_gemv(x.data_ptr(), K, wq.data_ptr(), s.data_ptr(), z.data_ptr(), want.data_ptr(), N, 1, N, K, b, G,
                               ws.data_ptr(), ws.numel(), stream)
    assert rc == 0
    rc = lib.gemq_dequant_gemv_static(x.data_ptr(), wq.data_ptr(), s.data_ptr(), z.data_ptr(), got.data_ptr(), N, K, b, G,
                                      stream)
    assert rc == 0
    torch.cuda.synchronize()
    assert torch.equal(got, want)
    ref = O.dequant_gemv(x.cpu().numpy()[None, :], wq.cpu().numpy(), s.cpu().numpy(), z.cpu().numpy(), b, G)
    g = got.float().cpu().numpy()
    assert rel_fro(g, ref) < REL_FRO_TOL and max_abs(g, ref) < MAX_ABS_TOL


def test_static_scratch_rejects_oversized_problem():
    from gemq_b200 import _capi
    lib = _capi.lib
    N, K = 14336 * 4, 14336  # needs far more than the 2 MiB array
    assert lib.gemq_gemv_workspace_bytes(N, K, 1) > lib.gemq_static_scratch_bytes()
    dummy = torch.zeros(16, dtype=torch.int32, device="cuda")
    rc = lib.gemq_dequant_gemv_static(dummy.data_ptr(), dummy.data_ptr(), dummy.data_ptr(), dummy.data_ptr(),
                                      dummy.data_ptr(), N, K, 2, 128, torch.cuda.current_stream().cuda_stream)
    assert rc == -3
