"""CPU restatement of the GEMQ packed-weight kernels and quantized MoE blocks.

TEST INFRASTRUCTURE ONLY (see the package docstring).  The restatement follows
the reference's Python/Triton sources; citations are ``path:line`` inside the
reference project.  Parity of this file is pinned by ``tests/golden``: the
fixtures there were produced by running the reference's own Triton kernels on
the CPU through the Triton interpreter (``tests/golden/make_golden.py``), and
``tests/test_oracle.py`` checks every function below against them.

Conventions ("kernel form", what every reference kernel consumes):

* ``wq``      int32 ``[ceil(K / eps), N]`` contiguous, ``eps = 32 // nbits``; the
  word at ``(r, n)`` holds the codes of ``k = r * eps + j`` at bit ``j * nbits``
  (gemq/triton_kernels/utils.py:47-70, made contiguous by the ``torch.cat`` of
  gemq/inference/moe_block.py:111-119).
* ``scales``, ``zeros`` fp16 ``[K / G, N]``; a weight is
  ``fp16(fma(fp16(q), scale, zero))`` (gemq/triton_kernels/utils.py:206-210), so
  ``zeros`` is an additive offset.
"""
from __future__ import annotations

import numpy as np
import torch
import torch.nn.functional as F

SUPPORTED_BITS = (1, 2, 3, 4)


def elements_per_word(nbits: int) -> int:
    """Codes per int32 word (gemq/triton_kernels/utils.py:85)."""
    return 32 // nbits


def cdiv(a: int, b: int) -> int:
    return -(-a // b)


# --------------------------------------------------------------------------
# packing format
# --------------------------------------------------------------------------
def pack_over_cols(q: np.ndarray, nbits: int) -> np.ndarray:
    """uint8 codes ``[rows, cols]`` -> int32 ``[rows, ceil(cols/eps)]``.

    Follows pack_weights_over_cols_kernel (gemq/triton_kernels/utils.py:33-70)
    with ``transpose=False``: lane ``j`` of a word is shifted by ``j*nbits``, the
    tail of the last word is zero padded (``other=0`` at :63).
    """
    assert nbits in SUPPORTED_BITS
    q = np.ascontiguousarray(q, dtype=np.uint8)
    rows, cols = q.shape
    eps = elements_per_word(nbits)
    words = cdiv(cols, eps)
    padded = np.zeros((rows, words * eps), dtype=np.uint32)
    padded[:, :cols] = q
    padded = padded.reshape(rows, words, eps)
    shifts = (np.arange(eps, dtype=np.uint32) * nbits).reshape(1, 1, eps)
    out = np.bitwise_or.reduce(padded << shifts, axis=2).astype(np.uint32)
    return out.view(np.int32)


def pack_kernel_form(q: np.ndarray, nbits: int) -> np.ndarray:
    """uint8 codes ``[N, K]`` -> contiguous int32 ``[ceil(K/eps), N]``.

    ``pack_weights_over_cols_triton(..., transpose=True)`` returns the ``.t()``
    view (gemq/triton_kernels/utils.py:110-111); the MoE blocks make it
    contiguous when stacking experts (gemq/inference/moe_block.py:111-119).
    """
    return np.ascontiguousarray(pack_over_cols(q, nbits).T)


def unpack_over_cols(packed: np.ndarray, nbits: int, num_output_cols: int) -> np.ndarray:
    """int32 ``[rows, words]`` -> uint8 ``[rows, num_output_cols]``.

    Follows unpack_over_cols_kernel (gemq/triton_kernels/utils.py:116-146).
    """
    assert nbits in SUPPORTED_BITS
    eps = elements_per_word(nbits)
    w = np.ascontiguousarray(packed).view(np.uint32)
    cols = np.arange(num_output_cols)
    words = w[:, cols // eps]
    shifts = ((cols % eps) * nbits).astype(np.uint32)
    return ((words >> shifts) & np.uint32((1 << nbits) - 1)).astype(np.uint8)


def unpack_kernel_form(wq: np.ndarray, nbits: int, K: int) -> np.ndarray:
    """Kernel-form words ``[ceil(K/eps), N]`` -> uint8 codes ``[K, N]``."""
    return np.ascontiguousarray(unpack_over_cols(np.ascontiguousarray(wq.T), nbits, K).T)


def dequantize(wq: np.ndarray, scales: np.ndarray, zeros: np.ndarray,
               nbits: int, group_size: int, K: int) -> np.ndarray:
    """Kernel-form tensors -> fp16 ``W^T [K, N]``, bit-exact.

    ``dequantize`` (gemq/triton_kernels/utils.py:192-212) is ``tl.fma`` on fp16
    operands: one rounding of ``q*s+z``.  The product and sum are exact in
    float64, and numpy rounds float64 -> float16 once (round to nearest even).
    """
    q = unpack_kernel_form(wq, nbits, K).astype(np.float64)
    g = np.arange(K) // group_size
    s = scales.astype(np.float64)[g]
    z = zeros.astype(np.float64)[g]
    return (q * s + z).astype(np.float16)


def kernel_form_offset(scale: np.ndarray, zero_point: np.ndarray) -> np.ndarray:
    """Additive offset ``z' = fp16(-zero_point * scale)`` for ``W=(Q-zero)*scale``.

    The quantizers define ``W = (Q - zero) * scale``
    (gemq/quantizers/gptq.py:446-450, gemq/quantizers/rtn.py:57-61); the kernels
    compute ``q*s + z'`` (gemq/triton_kernels/utils.py:196,210).
    """
    return (-(zero_point.astype(np.float32)) * scale.astype(np.float32)).astype(np.float16)


# --------------------------------------------------------------------------
# single-matrix ops
# --------------------------------------------------------------------------
def _t(a) -> torch.Tensor:
    return a if isinstance(a, torch.Tensor) else torch.from_numpy(np.ascontiguousarray(a))


def _n(a) -> np.ndarray:
    return a.detach().cpu().numpy() if isinstance(a, torch.Tensor) else np.asarray(a)


def _matmul_f32acc(x: np.ndarray, w: np.ndarray) -> np.ndarray:
    """``x[M,K] @ w[K,N]`` with fp32 operands/accumulation (``tl.dot``/``tl.sum`` in fp32)."""
    return (_t(x.astype(np.float32)) @ _t(w.astype(np.float32))).numpy()


def dequant_gemv(x, wq, scales, zeros, nbits: int, group_size: int) -> np.ndarray:
    """``y[1,N] = x[1,K] @ deq(wq)`` -> fp16 (gemq/triton_kernels/dequant_gemv.py:118-156).

    The reference sums split-K fp32 partials with fp16 atomics (:115); the order
    is not defined on a GPU, so this oracle keeps fp32 until one final rounding.
    """
    x, wq, scales, zeros = map(_n, (x, wq, scales, zeros))
    K = x.shape[1]
    w = dequantize(wq, scales, zeros, nbits, group_size, K)
    return _matmul_f32acc(x, w).astype(np.float16)


def dequant_gemm(x, wq, scales, zeros, nbits: int, group_size: int) -> np.ndarray:
    """``Y[M,N] = X[M,K] @ deq(wq)`` -> fp16 (gemq/triton_kernels/dequant_gemm.py:150-193)."""
    x, wq, scales, zeros = map(_n, (x, wq, scales, zeros))
    K = x.shape[1]
    w = dequantize(wq, scales, zeros, nbits, group_size, K)
    return _matmul_f32acc(x, w).astype(np.float16)


# --------------------------------------------------------------------------
# stacked-expert ops
# --------------------------------------------------------------------------
def _expert_view(wq, scales, zeros, e: int, nbits, K: int, N: int, group_size: int,
                 wq_strides, zs_strides=None):
    """Slice expert ``e`` out of stacked tensors.

    Word offset ``wq_strides[e]`` counts int32 elements
    (gemq/inference/moe_block.py:136-142).  The fused and selected-GEMV kernels
    locate scales at ``e * (K // G)`` rows (gemq/triton_kernels/fused_dequant_bmm.py:62,
    dequant_gemv.py:203); the grouped GEMM uses ``zs_strides[e]`` elements
    (gemq/triton_kernels/dequant_group_gemm.py:75,80-81).
    """
    b = int(nbits[e])
    rows = cdiv(K, elements_per_word(b))
    off = int(wq_strides[e])
    w = wq.reshape(-1)[off: off + rows * N].reshape(rows, N)
    groups = K // group_size
    if zs_strides is None:
        zoff = e * groups * N
    else:
        zoff = int(zs_strides[e])
    s = scales.reshape(-1)[zoff: zoff + groups * N].reshape(groups, N)
    z = zeros.reshape(-1)[zoff: zoff + groups * N].reshape(groups, N)
    return w, s, z, b


def dequant_sel_gemv(x, idx, wq, scales, zeros, nbits, wq_strides, group_size: int) -> np.ndarray:
    """GEMV against the expert chosen by ``idx[0]`` (gemq/triton_kernels/dequant_gemv.py:225-270)."""
    x, idx, wq, scales, zeros, nbits, wq_strides = map(_n, (x, idx, wq, scales, zeros, nbits, wq_strides))
    K = x.shape[1]
    N = wq.shape[1]
    w, s, z, b = _expert_view(wq, scales, zeros, int(idx[0]), nbits, K, N, group_size, wq_strides)
    return dequant_gemv(x, w, s, z, b, group_size)


def fused_up_proj(x, idx, w1, w3, w1_scales, w1_zeros, w3_scales, w3_zeros,
                  nbits, w_strides, group_size: int):
    """``x1, x3 [1, A*N]`` for the experts in ``idx`` (gemq/triton_kernels/fused_dequant_bmm.py:122-173).

    ``w1`` and ``w3`` share ``nbits`` and ``w_strides`` (:56-57,80,98); outputs are
    stored as fp16 (:152-153).
    """
    x, idx, nbits, w_strides = map(_n, (x, idx, nbits, w_strides))
    w1, w3, w1_scales, w1_zeros, w3_scales, w3_zeros = map(_n, (w1, w3, w1_scales, w1_zeros, w3_scales, w3_zeros))
    K = x.shape[1]
    N = w1.shape[1]
    o1, o3 = [], []
    for e in idx.tolist():
        a, s, z, b = _expert_view(w1, w1_scales, w1_zeros, e, nbits, K, N, group_size, w_strides)
        o1.append(dequant_gemv(x, a, s, z, b, group_size))
        a, s, z, b = _expert_view(w3, w3_scales, w3_zeros, e, nbits, K, N, group_size, w_strides)
        o3.append(dequant_gemv(x, a, s, z, b, group_size))
    return np.concatenate(o1, axis=1), np.concatenate(o3, axis=1)


def silu_mul_f32(x1: np.ndarray, x3: np.ndarray) -> np.ndarray:
    """``silu(x1) * x3`` in fp32 from fp16 inputs (gemq/triton_kernels/fused_dequant_bmm.py:237-239)."""
    a = x1.astype(np.float32)
    return (a * (1.0 / (1.0 + np.exp(-a)))).astype(np.float32) * x3.astype(np.float32)


def fused_down_proj(x1, x3, idx, w2, w2_scales, w2_zeros, nbits, w_strides, group_size: int) -> np.ndarray:
    """``x2[1, A*N]``, slot ``a`` uses ``x1/x3[a*K:(a+1)*K]`` (gemq/triton_kernels/fused_dequant_bmm.py:264-312).

    The activation is indexed by slot, not expert id (:230-234), and stays fp32
    into the dot product (:255).
    """
    x1, x3, idx, w2, w2_scales, w2_zeros, nbits, w_strides = map(
        _n, (x1, x3, idx, w2, w2_scales, w2_zeros, nbits, w_strides))
    A = idx.shape[0]
    K = x1.shape[1] // A
    N = w2.shape[1]
    outs = []
    for a, e in enumerate(idx.tolist()):
        act = silu_mul_f32(x1[:, a * K:(a + 1) * K], x3[:, a * K:(a + 1) * K])
        w, s, z, b = _expert_view(w2, w2_scales, w2_zeros, e, nbits, K, N, group_size, w_strides)
        wd = dequantize(w, s, z, b, group_size, K)
        outs.append(_matmul_f32acc(act, wd).astype(np.float16))
    return np.concatenate(outs, axis=1)


def dequant_group_gemm(x, indices, wq, scales, zeros, nbits, group_sizes, wq_strides, zs_strides,
                       out_dtype=np.float16) -> np.ndarray:
    """``Y[A,M,N]``, ``Y[g] = X @ deq(W[indices[g]])`` (gemq/triton_kernels/dequant_group_gemm.py:155-202)."""
    x, indices, wq, scales, zeros, nbits, group_sizes, wq_strides, zs_strides = map(
        _n, (x, indices, wq, scales, zeros, nbits, group_sizes, wq_strides, zs_strides))
    K = x.shape[1]
    N = wq.shape[1]
    outs = []
    for e in indices.reshape(-1).tolist():
        G = int(group_sizes[e])
        w, s, z, b = _expert_view(wq, scales, zeros, e, nbits, K, N, G, wq_strides, zs_strides)
        wd = dequantize(w, s, z, b, G, K)
        outs.append(_matmul_f32acc(x.astype(np.float32), wd).astype(out_dtype))
    return np.stack(outs)


# --------------------------------------------------------------------------
# layer restatements
# --------------------------------------------------------------------------
class StackedExperts:
    """Stacked kernel-form tensors and metadata of one projection (w1, w2 or w3).

    Mirrors the attributes ``w?_wq, w?_scales, w?_zeros, w?_nbits,
    w?_group_sizes, w?_wq_strides, w?_zs_strides`` built at
    gemq/inference/moe_block.py:111-142.
    """

    def __init__(self, wq_list, scales_list, zeros_list, nbits_list, group_size: int):
        self.wq = np.concatenate([np.asarray(w) for w in wq_list], axis=0)
        self.scales = np.concatenate([np.asarray(s) for s in scales_list], axis=0)
        self.zeros = np.concatenate([np.asarray(z) for z in zeros_list], axis=0)
        self.nbits = np.asarray(nbits_list, dtype=np.int32)
        self.group_sizes = np.full(len(nbits_list), group_size, dtype=np.int32)
        self.wq_strides = np.cumsum([0] + [w.size for w in wq_list])[:-1].astype(np.int32)
        self.zs_strides = np.cumsum([0] + [s.size for s in scales_list])[:-1].astype(np.int32)
        self.group_size = group_size


def route_fp16(x: torch.Tensor, gate_w: torch.Tensor, top_k: int):
    """Mixtral one-token routing, all in the model dtype (gemq/inference/moe_block.py:211-214)."""
    scores = F.linear(x, gate_w)
    w = F.softmax(scores, dim=-1)
    w, idx = torch.topk(w, top_k, dim=-1)
    w = w / w.sum(dim=-1, keepdim=True)
    return w, idx, scores


def route_fp32(x: torch.Tensor, gate_w: torch.Tensor, top_k: int, renorm: bool, logits_fp32: bool):
    """fp32-softmax routing then cast back.

    Mixtral n-token: logits in the model dtype, softmax in fp32
    (gemq/inference/moe_block.py:174-180).  DeepSeek-V2 (both paths): logits from
    fp32 copies of ``x`` and the gate, renormalise only if ``norm_topk_prob``
    (:457-464, :499-505).
    """
    if logits_fp32:
        logits = F.linear(x.float(), gate_w.float())
    else:
        logits = F.linear(x, gate_w)
    w = F.softmax(logits, dim=1, dtype=torch.float)
    w, idx = torch.topk(w, top_k, dim=-1)
    if renorm:
        w = w / w.sum(dim=-1, keepdim=True)
    return w.to(x.dtype), idx, logits


def _expert_ffn_tokens(x: np.ndarray, e: int, w1: StackedExperts, w3: StackedExperts, w2: StackedExperts) -> np.ndarray:
    """Single-expert FFN on ``x[M,D]`` via three grouped GEMMs (gemq/inference/moe_block.py:146-163)."""
    ie = np.array([e], dtype=np.int64)
    x1 = dequant_group_gemm(x, ie, w1.wq, w1.scales, w1.zeros, w1.nbits, w1.group_sizes, w1.wq_strides, w1.zs_strides)[0]
    x3 = dequant_group_gemm(x, ie, w3.wq, w3.scales, w3.zeros, w3.nbits, w3.group_sizes, w3.wq_strides, w3.zs_strides)[0]
    h = (F.silu(_t(x1)) * _t(x3)).numpy()
    return dequant_group_gemm(h, ie, w2.wq, w2.scales, w2.zeros, w2.nbits, w2.group_sizes, w2.wq_strides, w2.zs_strides)[0]


def moe_one_token(x: torch.Tensor, gate_w: torch.Tensor, top_k: int,
                  w1: StackedExperts, w3: StackedExperts, w2: StackedExperts,
                  family: str = "mixtral", norm_topk_prob: bool = True, shared=None):
    """One-token forward of the quantized fused blocks.

    Mixtral: gemq/inference/moe_block.py:200-235.  DeepSeek-V2: :488-531, with the
    shared experts added through three single-matrix GEMVs (:525-528).
    ``shared`` is ``(w1, w3, w2, nbits, group_size)`` with each ``w?`` a
    ``(wq, scales, zeros)`` triple.  Returns ``(out[1,D], weights, indices)``.
    """
    assert x.shape[0] == 1
    if family == "mixtral":
        ew, ei, _ = route_fp16(x, gate_w, top_k)
    else:
        ew, ei, _ = route_fp32(x, gate_w, top_k, norm_topk_prob, logits_fp32=True)
    idx = ei[0].numpy()
    G = w1.group_size
    x1, x3 = fused_up_proj(x.numpy(), idx, w1.wq, w3.wq, w1.scales, w1.zeros, w3.scales, w3.zeros,
                           w1.nbits, w1.wq_strides, G)
    x2 = fused_down_proj(x1, x3, idx, w2.wq, w2.scales, w2.zeros, w2.nbits, w2.wq_strides, G)
    D = x.shape[1]
    outs = torch.einsum("tai,ta->ti", _t(x2).view(1, top_k, D), ew)
    if shared is not None:
        (s1, s3, s2, sb, sg) = shared
        a1 = dequant_gemv(x.numpy(), *s1, sb, sg)
        a3 = dequant_gemv(x.numpy(), *s3, sb, sg)
        h = (F.silu(_t(a1)) * _t(a3)).numpy()
        a2 = dequant_gemv(h, *s2, sb, sg)
        outs = outs + _t(a2)
    return outs, ew, ei


def moe_n_tokens(x: torch.Tensor, gate_w: torch.Tensor, top_k: int,
                 w1: StackedExperts, w3: StackedExperts, w2: StackedExperts,
                 family: str = "mixtral", norm_topk_prob: bool = True, shared=None):
    """n-token forward (gemq/inference/moe_block.py:165-198, DeepSeek-V2 :448-486).

    Each expert contribution is scaled by its routing weight in the model dtype
    and accumulated with ``index_add_`` in expert order (:191-195).
    Returns ``(out[T,D], weights, indices, router_logits)``.
    """
    T, D = x.shape
    E = gate_w.shape[0]
    rw, sel, logits = route_fp32(x, gate_w, top_k, True if family == "mixtral" else norm_topk_prob,
                                 logits_fp32=(family != "mixtral"))
    out = torch.zeros((T, D), dtype=x.dtype)
    xn = x.float().numpy().astype(np.float16) if x.dtype != torch.float16 else x.numpy()
    for e in range(E):
        tok, slot = torch.where(sel == e)
        if tok.numel() == 0:
            continue
        cur = xn[tok.numpy()]
        y = _t(_expert_ffn_tokens(cur, e, w1, w3, w2)).to(x.dtype) * rw[tok, slot, None]
        out.index_add_(0, tok, y.to(x.dtype))
    if shared is not None:
        (s1, s3, s2, sb, sg) = shared
        a1 = dequant_gemm(xn, *s1, sb, sg)
        a3 = dequant_gemm(xn, *s3, sb, sg)
        h = (F.silu(_t(a1)) * _t(a3)).numpy()
        out = out + _t(dequant_gemm(h, *s2, sb, sg)).to(x.dtype)
    return out, rw, sel, logits


def moe_reference_fp32(x: torch.Tensor, weights: torch.Tensor, indices: torch.Tensor,
                       w1: StackedExperts, w3: StackedExperts, w2: StackedExperts, shared=None) -> torch.Tensor:
    """fp32-accumulated layer output for given routing: no fp16 rounding of intermediates.

    Used as the tolerance anchor "fp32-accumulated reference" for layer outputs:
    weights are the exact fp16 dequantised values, everything else is float32.
    """
    T, D = x.shape
    out = torch.zeros((T, D), dtype=torch.float32)
    cache = {}

    def deq(st: StackedExperts, e: int, K: int):
        key = (id(st), e)
        if key not in cache:
            N = st.wq.shape[1]
            w, s, z, b = _expert_view(st.wq, st.scales, st.zeros, e, st.nbits, K, N, st.group_size,
                                      st.wq_strides, st.zs_strides)
            cache[key] = _t(dequantize(w, s, z, b, st.group_size, K).astype(np.float32))
        return cache[key]

    xf = x.float()
    F_dim = w1.wq.shape[1]
    for t in range(T):
        for a in range(indices.shape[1]):
            e = int(indices[t, a])
            h = F.silu(xf[t:t + 1] @ deq(w1, e, D)) * (xf[t:t + 1] @ deq(w3, e, D))
            out[t] += float(weights[t, a]) * (h @ deq(w2, e, F_dim))[0]
    if shared is not None:
        (s1, s3, s2, sb, sg) = shared
        d1 = _t(dequantize(*map(_n, s1), sb, sg, D).astype(np.float32))
        d3 = _t(dequantize(*map(_n, s3), sb, sg, D).astype(np.float32))
        d2 = _t(dequantize(*map(_n, s2), sb, sg, d1.shape[1]).astype(np.float32))
        out += (F.silu(xf @ d1) * (xf @ d3)) @ d2
    return out
