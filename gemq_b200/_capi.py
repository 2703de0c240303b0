"""ctypes binding of libgemq_b200.so (the C ABI declared in include/gemq_b200.h).

There is no fallback: importing this module without the built library raises.
Build it with ``python -m gemq_b200.csrc.build`` (needs nvcc).
"""
from __future__ import annotations

import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.environ.get("GEMQ_B200_LIB") or os.path.join(_HERE, "libgemq_b200.so")

ERRORS = {
    -1: "bad argument (null pointer, non-positive extent or unsupported bit-width)",
    -2: "unsupported shape",
    -3: "workspace missing or too small",
    -4: "CUDA launch error",
    -5: "pointer not 16-byte aligned",
}


class GemqError(RuntimeError):
    def __init__(self, fn: str, code: int):
        super().__init__(f"{fn} failed with code {code}: {ERRORS.get(code, 'unknown error')}")
        self.code = code


class Stacked(C.Structure):
    _fields_ = [("wq", C.c_void_p), ("scales", C.c_void_p), ("zeros", C.c_void_p),
                ("nbits", C.c_void_p), ("wq_strides", C.c_void_p), ("zs_strides", C.c_void_p),
                ("wq_rows", C.c_int64), ("zs_rows", C.c_int64), ("n_experts", C.c_int32)]


class Single(C.Structure):
    _fields_ = [("wq", C.c_void_p), ("scales", C.c_void_p), ("zeros", C.c_void_p),
                ("nbits", C.c_int), ("group_size", C.c_int)]


class MoeLayer(C.Structure):
    _fields_ = [("hidden", C.c_int), ("ffn", C.c_int), ("n_experts", C.c_int), ("top_k", C.c_int),
                ("group_size", C.c_int), ("route_mode", C.c_int), ("renorm", C.c_int), ("shared_ffn", C.c_int),
                ("gate", C.c_void_p), ("w1", Stacked), ("w3", Stacked), ("w2", Stacked),
                ("s1", Single), ("s3", Single), ("s2", Single)]


_P, _I, _Z = C.c_void_p, C.c_int, C.c_size_t

_SIGNATURES = {
    "gemq_version": (C.c_char_p, []),
    "gemq_gemv_workspace_bytes": (_Z, [_I, _I, _I]),
    "gemq_pack_over_cols": (_I, [_P, _P, _I, _I, _I, _P]),
    "gemq_pack_kernel_form": (_I, [_P, _P, _I, _I, _I, _P]),
    "gemq_unpack_over_cols": (_I, [_P, _P, _I, _I, _I, _I, _P]),
    "gemq_dequantize": (_I, [_P, _P, _P, _P, _I, _I, _I, _I, _P]),
    "gemq_dequant_gemv": (_I, [_P, _I, _P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _P, _Z, _P]),
    "gemq_dequant_sel_gemv": (_I, [_P, _P, C.POINTER(Stacked), _P, _I, _I, _I, _P, _Z, _P]),
    "gemq_fused_up_proj": (_I, [_P, _P, _I, C.POINTER(Stacked), C.POINTER(Stacked), _P, _P, _I, _I, _I, _P, _Z, _P]),
    "gemq_fused_down_proj": (_I, [_P, _P, _P, _I, C.POINTER(Stacked), _P, _I, _I, _I, _P, _Z, _P]),
    "gemq_dequant_group_gemv": (_I, [_P, _I, _P, _I, C.POINTER(Stacked), _P, _I, _I, _I, _I, _P, _Z, _P]),
    "gemq_moe_route": (_I, [_P, _P, _I, _I, _I, _I, _I, _I, _I, _P, _P, _P, _P]),
    "gemq_moe_decode_scratch_bytes": (_Z, [C.POINTER(MoeLayer)]),
    "gemq_dequant_gemm_tc": (_I, [_P, _P, _P, _P, _P, _P, _P, _P, _I, _P, _I, _I, _I, _I, _I, _P, _P]),
    "gemq_moe_prefill_scratch_bytes": (_Z, [C.POINTER(MoeLayer), _I]),
    "gemq_moe_prefill": (_I, [C.POINTER(MoeLayer), _P, _P, _P, _P, _P, _I, _I, _I, _I, _P, _Z, _P]),
    "gemq_moe_prefill_error_word": (_P, [C.POINTER(MoeLayer), _I, _P]),
    "gemq_ep_plan_scratch_bytes": (_Z, [_I]),
    "gemq_ep_plan": (_I, [_P, _I, _I, _I, _I, _P, _P, _P, _P, _P, _P, _P, _P, _Z, _P]),
    "gemq_ep_pack_rows": (_I, [_P, _P, _P, _P, _I, _I, _I, _P, _P]),
    "gemq_ep_unpack_rows": (_I, [_P, _I, _I, _P, _P, _P, _P]),
    "gemq_ep_combine": (_I, [_P, _P, _P, _I, _I, _I, _I, _P, _P]),
    "gemq_dequant_gemv_static": (_I, [_P, _P, _P, _P, _P, _I, _I, _I, _I, _P]),
    "gemq_static_scratch_bytes": (_Z, []),
    "gemq_workspace_error_word": (_P, [_P]),
    "gemq_workspace_wait_limit_word": (_P, [_P]),
    "gemq_moe_decode": (_I, [C.POINTER(MoeLayer), _P, _P, _P, _P, _I, _I, _I, _P, _Z, _P]),
}

EXPORTED = tuple(_SIGNATURES)


def _load() -> C.CDLL:
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            f"{LIB_PATH} is missing: gemq_b200 has no CPU or Triton fallback. "
            "Build it with `python -m gemq_b200.csrc.build`.")
    lib = C.CDLL(LIB_PATH)
    for name, (res, args) in _SIGNATURES.items():
        fn = getattr(lib, name)
        fn.restype = res
        fn.argtypes = args
    return lib


lib = _load()


def stacked(wq, scales, zeros, nbits, wq_strides, zs_strides=None) -> Stacked:
    """Describe stacked-expert torch tensors for the library (borrowed pointers)."""
    return Stacked(wq.data_ptr(), scales.data_ptr(), zeros.data_ptr(), nbits.data_ptr(), wq_strides.data_ptr(),
                   zs_strides.data_ptr() if zs_strides is not None else None, wq.shape[0], scales.shape[0],
                   int(nbits.numel()))


def check(fn: str, code: int) -> None:
    if code != 0:
        raise GemqError(fn, code)
