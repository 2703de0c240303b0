"""Host-side plumbing shared by the op wrappers: argument checks, streams, workspace."""
from __future__ import annotations

import torch

from .. import _capi

_workspaces: dict = {}


def require_cuda(*tensors: torch.Tensor) -> torch.device:
    dev = None
    for t in tensors:
        if not isinstance(t, torch.Tensor):
            raise TypeError(f"expected a torch.Tensor, got {type(t).__name__}")
        if not t.is_cuda:
            raise RuntimeError("gemq_b200 ops run on CUDA tensors only (there is no CPU path)")
        if dev is None:
            dev = t.device
        elif t.device != dev:
            raise RuntimeError(f"tensors on different devices: {dev} and {t.device}")
    return dev


def require(cond: bool, msg: str) -> None:
    if not cond:
        raise ValueError(msg)


def stream_ptr(dev: torch.device) -> int:
    return torch.cuda.current_stream(dev).cuda_stream


def workspace(dev: torch.device, nbytes: int) -> torch.Tensor:
    """Zero-initialised uint8 scratch of at least ``nbytes`` on ``dev``.

    The arrival counters at its head are left at zero by every kernel, so the buffer is
    zeroed only when it is (re)allocated.  One buffer per device: calls that share it must
    be ordered on one stream.
    """
    key = (dev.type, dev.index if dev.index is not None else torch.cuda.current_device())
    ws = _workspaces.get(key)
    if ws is None or ws.numel() < nbytes:
        ws = torch.zeros(max(nbytes, 1 << 20), dtype=torch.uint8, device=dev)
        _workspaces[key] = ws
    return ws


def gemv_workspace(dev: torch.device, total_cols: int, max_k: int, tokens: int) -> torch.Tensor:
    return workspace(dev, _capi.lib.gemq_gemv_workspace_bytes(total_cols, max_k, tokens))


def check_kernel_form(wq, scales, zeros, K: int, N: int, nbits: int, group_size: int) -> None:
    require(nbits in (1, 2, 3, 4), f"unsupported bit-width {nbits}")
    require(wq.dtype == torch.int32 and wq.is_contiguous(), "w_q must be contiguous int32 [ceil(K/eps), N]")
    eps = 32 // nbits
    require(tuple(wq.shape) == (-(-K // eps), N), f"w_q shape {tuple(wq.shape)} != {(-(-K // eps), N)}")
    require(K % group_size == 0, "K must be a multiple of group_size")
    for name, t in (("scales", scales), ("zeros", zeros)):
        require(t.dtype == torch.float16 and t.is_contiguous(), f"{name} must be contiguous float16")
        require(tuple(t.shape) == (K // group_size, N), f"{name} shape {tuple(t.shape)} != {(K // group_size, N)}")


_err_words: dict = {}


def error_word(dev: torch.device) -> torch.Tensor:
    """One int32 per device that kernels with bounded waits set when a wait expires."""
    key = (dev.type, dev.index if dev.index is not None else torch.cuda.current_device())
    t = _err_words.get(key)
    if t is None:
        t = torch.zeros(1, dtype=torch.int32, device=dev)
        _err_words[key] = t
    return t


def tc_gemm_ok(M: int, N: int, K: int, group_size: int) -> bool:
    """Shapes the tcgen05 GEMM takes; smaller row counts stay on the decode kernel."""
    return M >= 32 and N % 128 == 0 and K % 64 == 0 and group_size % 64 == 0 and K % group_size == 0
