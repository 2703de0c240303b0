"""Parity at the benchmark configurations' real shapes, ragged expert loads, and the error paths.

The CPU oracle is affordable at full size only for a sample of rows, so the full-size prefill
test checks rows spread over all experts against the fp32-accumulated reference built from the
block's own packed tensors, plus bit-reproducibility of the whole output.
"""
import ctypes as C

import numpy as np
import pytest
import torch

from oracle import gemq_oracle as O
from conftest import MAX_ABS_TOL, REL_FRO_TOL, max_abs, rel_fro
import moe_fixtures as MF

pytestmark = pytest.mark.gpu

G = 128


def bf16_abs_bound(ref):
    """Max-abs bound for bf16 outputs: two roundings to 8 mantissa bits (the expert contribution and
    the sum) of values up to max|ref| -- 2^-7 of the largest magnitude, never below the fp16 bound."""
    return max(MAX_ABS_TOL, 2.0 ** -7 * float(np.abs(ref).max()))


def f16_abs_bound(ref):
    """The 2e-2 bound is stated for outputs of order one to ten; an fp16 result of magnitude m
    carries a rounding of up to m * 2^-11, so the bound grows with the largest magnitude beyond 16."""
    return MAX_ABS_TOL * max(1.0, float(np.abs(ref).max()) / 16.0)


def expert_matrix(blk, name, e, K, N, shared=False):
    """fp32 [K, N] de-quantised weights of expert ``e`` (or the shared expert) from the block's tensors."""
    if shared:
        b = int(blk.shared_nbits)
        wq = getattr(blk, f"shared_{name}_wq").cpu().numpy()
        s = getattr(blk, f"shared_{name}_scales").cpu().numpy()
        z = getattr(blk, f"shared_{name}_zeros").cpu().numpy()
        return O.dequantize(wq, s, z, b, G, K).astype(np.float32)
    b = blk._nbits_host[e]
    off = int(getattr(blk, f"{name}_wq_strides")[e])
    rows = -(-K // (32 // b))
    wq = getattr(blk, f"{name}_wq").view(-1)[off:off + rows * N].view(rows, N).cpu().numpy()
    zo = int(getattr(blk, f"{name}_zs_strides")[e])
    s = getattr(blk, f"{name}_scales").view(-1)[zo:zo + (K // G) * N].view(K // G, N).cpu().numpy()
    z = getattr(blk, f"{name}_zeros").view(-1)[zo:zo + (K // G) * N].view(K // G, N).cpu().numpy()
    return O.dequantize(wq, s, z, b, G, K).astype(np.float32)


def reference_rows(blk, x_rows, w_rows, sel_rows, D, Fd, shared_ffn=0):
    """fp32-accumulated layer output of the given rows, expert by expert (one expert's matrices
    in memory at a time)."""
    xf = x_rows.float().cpu().numpy()
    out = np.zeros((xf.shape[0], D), dtype=np.float64)
    sel = sel_rows.cpu().numpy()
    wts = w_rows.float().cpu().numpy()
    for e in np.unique(sel):
        rows, slots = np.nonzero(sel == e)
        w1, w3 = expert_matrix(blk, "w1", int(e), D, Fd), expert_matrix(blk, "w3", int(e), D, Fd)
        h1 = xf[rows] @ w1
        h = (h1 / (1.0 + np.exp(-h1))) * (xf[rows] @ w3)
        del w1, w3
        y = h @ expert_matrix(blk, "w2", int(e), Fd, D)
        out[rows] += wts[rows, slots][:, None] * y
    if shared_ffn:
        h1 = xf @ expert_matrix(blk, "w1", 0, D, shared_ffn, shared=True)
        h = (h1 / (1.0 + np.exp(-h1))) * (xf @ expert_matrix(blk, "w3", 0, D, shared_ffn, shared=True))
        out += h @ expert_matrix(blk, "w2", 0, shared_ffn, D, shared=True)
    return out


def test_config3_prefill_full_size_bf16():
    """Mixtral-8x7B-shaped layer, 4096 bf16 tokens, top-2 with Dirichlet(0.5) expert popularity, mixed bits."""
    from gemq_b200 import synth
    D, Fd, E, A, T = 4096, 14336, 8, 2, 4096
    blk = synth.mixtral_block(seed=0)
    g = torch.Generator().manual_seed(7)
    torch.manual_seed(7)
    pop = torch.distributions.Dirichlet(torch.full((E,), 0.5)).sample()
    sel = torch.multinomial(pop.expand(T, E), A, replacement=False, generator=g)
    w = torch.softmax(torch.randn(T, A, generator=g), -1).to(torch.bfloat16)
    x = torch.randn(T, D, generator=g).to(torch.bfloat16)
    out = blk._prefill(x.cuda(), 1, True, routing=(w.cuda(), sel.cuda()))[0]
    assert out.dtype == torch.bfloat16 and blk.prefill_error_code(T) == 0
    out2 = blk._prefill(x.cuda(), 1, True, routing=(w.cuda(), sel.cuda()))[0]
    assert torch.equal(out, out2)
    # 64 rows: for every expert the first rows that visit it
    rows = []
    for e in range(E):
        rows += torch.nonzero((sel == e).any(dim=1)).view(-1)[:8].tolist()
    rows = sorted(set(rows))
    ref = reference_rows(blk, x[rows], w[rows], sel[rows], D, Fd)
    got = out[rows].float().cpu().numpy()
    # bf16 output and bf16 per-expert contributions: 8 mantissa bits -> about 2.5e-3 relative
    assert rel_fro(got, ref) < REL_FRO_TOL, rel_fro(got, ref)
    assert max_abs(got, ref) < bf16_abs_bound(ref), (max_abs(got, ref), bf16_abs_bound(ref))


@pytest.mark.parametrize("B", [1, 4, 16])
def test_config2_deepseek_real_shape(B):
    """DeepSeek-V2-Lite-shaped layer: hidden 2048, intermediate 1408, 64 experts, top-6, two shared at 4-bit."""
    from gemq_b200 import synth
    D, Fd, SF = 2048, 1408, 2816
    blk = synth.deepseek_block(seed=0)
    x = torch.randn(B, D, generator=torch.Generator().manual_seed(B)).half()
    out = blk(x.cuda().view(B, 1, D)).view(B, D)
    assert blk.decode_error_code() == 0
    _, gw, gi = blk._decode(x.cuda(), 2)
    ref = reference_rows(blk, x, gw.cpu(), gi.cpu(), D, Fd, shared_ffn=SF)
    got = out.float().cpu().numpy()
    assert rel_fro(got, ref) < REL_FRO_TOL, rel_fro(got, ref)
    assert max_abs(got, ref) < f16_abs_bound(ref), (max_abs(got, ref), f16_abs_bound(ref))
    out2 = blk(x.cuda().view(B, 1, D)).view(B, D)
    assert torch.equal(out, out2)


@pytest.mark.parametrize("counts", [[300, 0, 0, 0], [0, 1, 0, 129], [128, 129, 256, 257], [1, 1, 1, 1], [0, 0, 513, 0]])
def test_prefill_ragged_expert_loads(counts):
    """Experts with no rows, one row, one expert taking everything, row counts around the 128-row tile."""
    layer = MF.make_layer("mixtral", D=256, Fd=512, E=4, A=1, bits=[4, 1, 3, 2], seed=21, gate_std=0.02)
    blk = MF.gpu_block(layer)
    w1, w3, w2, _ = MF.oracle_parts(layer)
    T = sum(counts)
    g = torch.Generator().manual_seed(T)
    sel = torch.cat([torch.full((c,), e, dtype=torch.int64) for e, c in enumerate(counts)])
    sel = sel[torch.randperm(T, generator=g)].view(T, 1)
    w = (torch.rand(T, 1, generator=g) * 0.5 + 0.5).half()
    x = torch.randn(T, 256, generator=g).half()
    out = blk._prefill(x.cuda(), 1, True, routing=(w.cuda(), sel.cuda()))[0]
    assert blk.prefill_error_code(T) == 0
    ref = O.moe_reference_fp32(x, w.float(), sel, w1, w3, w2).numpy()
    got = out.float().cpu().numpy()
    assert rel_fro(got, ref) < REL_FRO_TOL and max_abs(got, ref) < MAX_ABS_TOL


def test_mixtral_prefill_bf16_small():
    layer = MF.make_layer("mixtral", D=256, Fd=512, E=4, A=2, bits=[4, 1, 3, 2], seed=6, gate_std=0.02)
    blk = MF.gpu_block(layer)
    w1, w3, w2, _ = MF.oracle_parts(layer)
    T = 200
    x = torch.randn(T, 256, generator=torch.Generator().manual_seed(5)).to(torch.bfloat16)
    out, _ = blk(x.cuda().view(1, T, -1))
    assert out.dtype == torch.bfloat16 and blk.prefill_error_code(T) == 0
    _, gw, gi, _ = blk._prefill(x.cuda(), 1, True)
    ref = O.moe_reference_fp32(x.float(), gw.float().cpu(), gi.cpu(), w1, w3, w2).numpy()
    got = out.view(T, -1).float().cpu().numpy()
    assert rel_fro(got, ref) < REL_FRO_TOL, rel_fro(got, ref)
    assert max_abs(got, ref) < bf16_abs_bound(ref), (max_abs(got, ref), bf16_abs_bound(ref))


@pytest.mark.parametrize("D,Fd,bits", [(1280, 640, [3, 3, 3, 3]), (768, 1920, [3, 1, 3, 4]), (512, 384, [3, 3, 2, 3])])
def test_decode_three_bit_run_remainders(D, Fd, bits):
    """One-token layer with 3-bit experts whose reduction lengths leave every remainder of groups
    in the last 5-group run (10 and 5 groups: none; 6 and 15: one and none; 4 and 3), and packed rows that
    end inside a 16-row quad: the integer 3-bit path masks rows that straddle two groups and zero-fills
    rows past the end of the matrix."""
    layer = MF.make_layer("mixtral", D=D, Fd=Fd, E=4, A=2, bits=bits, seed=21, gate_std=0.02)
    blk = MF.gpu_block(layer)
    w1, w3, w2, _ = MF.oracle_parts(layer)
    for seed in (1, 2):
        x = torch.randn(1, D, generator=torch.Generator().manual_seed(seed)).half()
        out, _ = blk(x.cuda().view(1, 1, -1))
        assert blk.decode_error_code() == 0
        _, gw, gi = blk._decode(x.cuda(), 0)
        ref = O.moe_reference_fp32(x, gw.float().cpu(), gi.cpu(), w1, w3, w2)
        got = out.view(1, -1).float().cpu().numpy()
        ref = np.asarray(ref, dtype=np.float32)
        assert rel_fro(got, ref) < REL_FRO_TOL, rel_fro(got, ref)
        assert max_abs(got, ref) < f16_abs_bound(ref), (max_abs(got, ref), f16_abs_bound(ref))
        again, _ = blk(x.cuda().view(1, 1, -1))
        assert torch.equal(out, again)


def test_decode_layer_is_bit_reproducible_over_many_graph_replays():
    """The cross-CTA sums of the one-launch decode layer are formed in a fixed order whichever
    CTA completes a chunk: 60 replays of each of six captured layer calls (Mixtral config-1 shape
    and DeepSeek config-2 shape) give bit-identical outputs, and no wait runs out."""
    from gemq_b200 import synth
    dev = torch.device("cuda")
    gen = torch.Generator(device=dev).manual_seed(7)
    cases = [(synth.mixtral_block(seed=100, device=dev), 4096), (synth.mixtral_block(seed=103, device=dev), 4096),
             (synth.deepseek_block(seed=0, device=dev), 2048)]
    side = torch.cuda.Stream(device=dev)
    graphs, keep = [], []  # the graphs read their activations in place: keep them alive
    with torch.cuda.stream(side):
        for blk, D in cases:
            for _ in range(2):
                x = torch.randn(1, 1, D, device=dev, generator=gen).half()
                keep.append(x)
                blk(x)
                torch.cuda.synchronize()
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g, stream=side):
                    o = blk(x)
                    o = o[0] if isinstance(o, tuple) else o
                graphs.append((g, o))
    torch.cuda.synchronize()
    ref = []
    for g, o in graphs:
        g.replay()
        torch.cuda.synchronize()
        ref.append(o.clone())
    bad = torch.zeros((), dtype=torch.int64, device=dev)
    for _ in range(60):
        for (g, o), want in zip(graphs, ref):
            g.replay()
            bad += (o != want).any().to(torch.int64)
    torch.cuda.synchronize()
    assert int(bad) == 0
    assert all(blk.decode_error_code() == 0 for blk, _ in cases)
    assert not any(bool(torch.isnan(w).any()) for w in ref)


def test_group_gemm_tensor_core_branch():
    """dequant_group_gemm with M >= 32 rows: the tcgen05 GEMM with a device-side expert id and the
    stacked nbits / wq_strides / zs_strides of mixed-bit experts."""
    from gemq_b200.kernels import dequant_group_gemm
    from gemq_b200.kernels._runtime import error_word
    rng = np.random.default_rng(77)
    K, N, M = 512, 384, 150
    bits = [3, 1, 4, 2]
    lins = [MF.draw_linear(rng, N, K, b) for b in bits]
    st = MF.stacked(lins)
    x = rng.standard_normal((M, K)).astype(np.float16)
    idx = np.array([2, 0], dtype=np.int64)
    t = lambda a: torch.from_numpy(np.ascontiguousarray(a)).cuda()
    gs = np.full(len(bits), 128, dtype=np.int32)
    y = dequant_group_gemm(t(x), t(idx), t(st.wq), t(st.scales), t(st.zeros), t(st.nbits.astype(np.int32)), t(gs),
                           t(st.wq_strides.astype(np.int32)), t(st.zs_strides.astype(np.int32)))
    assert y.shape == (2, M, N) and int(error_word(y.device).item()) == 0
    want = O.dequant_group_gemm(x, idx, st.wq, st.scales, st.zeros, st.nbits, gs, st.wq_strides, st.zs_strides)
    got = y.float().cpu().numpy()
    assert rel_fro(got, want) < REL_FRO_TOL and max_abs(got, want) < MAX_ABS_TOL


def _set_word(blk, fn, value):
    off = fn(blk._scratch.data_ptr()) - blk._scratch.data_ptr()
    blk._scratch[off:off + 4].view(torch.int32).fill_(value)


def test_decode_wait_limit_expires_and_is_reported():
    """A wait limit of one poll makes the bounded waits of the layer kernel run out: the launch
    still returns, the error word says so, and after the scratch is reset the layer is correct again."""
    from gemq_b200 import _capi
    layer = MF.make_layer("mixtral", D=512, Fd=1024, E=4, A=2, bits=[1, 2, 3, 4], seed=31, gate_std=0.02)
    blk = MF.gpu_block(layer)
    w1, w3, w2, _ = MF.oracle_parts(layer)
    x = torch.randn(1, 512, generator=torch.Generator().manual_seed(31)).half()
    good, _ = blk(x.cuda().view(1, 1, -1))
    assert blk.decode_error_code() == 0
    _set_word(blk, _capi.lib.gemq_workspace_wait_limit_word, 1)
    codes = set()
    for _ in range(4):
        blk(x.cuda().view(1, 1, -1))
        codes.add(blk.decode_error_code())
        blk.reset_decode_scratch()
        _set_word(blk, _capi.lib.gemq_workspace_wait_limit_word, 1)
    assert codes - {0}, "no bounded wait ran out with a limit of one poll"
    blk.reset_decode_scratch()
    again, _ = blk(x.cuda().view(1, 1, -1))
    assert blk.decode_error_code() == 0
    assert torch.equal(good, again)


def test_expert_id_out_of_range_is_reported_not_used():
    """Caller-supplied routing with an id outside [0, E): decode clamps it and reports it; prefill
    leaves the pair out and reports it.  No access is made with the bad id."""
    from gemq_b200 import _capi
    from gemq_b200.kernels._runtime import stream_ptr
    layer = MF.make_layer("mixtral", D=256, Fd=512, E=4, A=2, bits=[1, 2, 3, 4], seed=41, gate_std=0.02)
    blk = MF.gpu_block(layer)
    dev = torch.device("cuda")
    x = torch.randn(1, 256, generator=torch.Generator().manual_seed(41)).half().cuda()
    out = torch.empty_like(x)
    idx = torch.tensor([[1, 99]], dtype=torch.int64, device=dev)
    w = torch.tensor([[0.5, 0.5]], dtype=torch.float16, device=dev)
    rc = _capi.lib.gemq_moe_decode(C.byref(blk._layer), x.data_ptr(), out.data_ptr(), idx.data_ptr(), w.data_ptr(), 1, 0, 0,
                                   blk._scratch.data_ptr(), blk._scratch.numel(), stream_ptr(dev))
    assert rc == 0
    assert blk.decode_error_code() == 7
    blk.reset_decode_scratch()
    T = 40
    xs = torch.randn(T, 256, generator=torch.Generator().manual_seed(42)).half().cuda()
    sel = torch.randint(0, 4, (T, 2), generator=torch.Generator().manual_seed(43))
    sel[:, 1] = (sel[:, 0] + 1) % 4
    sel[3, 1] = -5
    sel[7, 0] = 4
    ws = torch.full((T, 2), 0.5, dtype=torch.float16)
    out = blk._prefill(xs, 1, True, routing=(ws.cuda(), sel.cuda()))[0]
    assert blk.prefill_error_code(T) == 21
    w1, w3, w2, _ = MF.oracle_parts(layer)
    good = [t for t in range(T) if t not in (3, 7)]
    ref = O.moe_reference_fp32(xs.cpu()[good], ws[good].float(), sel[good], w1, w3, w2).numpy()
    got = out.float().cpu().numpy()[good]
    assert rel_fro(got, ref) < REL_FRO_TOL and max_abs(got, ref) < MAX_ABS_TOL


def test_torch_compile_traces_through_the_block():
    """torch.compile(mode="reduce-overhead", fullgraph=True) of the one-token forward, as the
    reference's decode step is compiled (gemq/benchmark_generate.py:158-160): no graph break,
    same bits as eager."""
    import torch._dynamo
    layer = MF.make_layer("mixtral", D=512, Fd=1024, E=4, A=2, bits=[1, 2, 3, 4], seed=51, gate_std=0.02)
    blk = MF.gpu_block(layer)
    x = torch.randn(1, 1, 512, generator=torch.Generator().manual_seed(51)).half().cuda()
    eager, _ = blk(x)

    def step(h):
        return blk(h)[0]

    explained = torch._dynamo.explain(step)(x)
    assert explained.graph_break_count == 0, explained.break_reasons
    compiled = torch.compile(step, mode="reduce-overhead", fullgraph=True)
    for _ in range(3):  # warm-up, capture, replay
        out = compiled(x)
    assert torch.equal(out, eager)
    torch._dynamo.reset()


TINY_DECODER = dict(hidden_size=256, intermediate_size=512, num_local_experts=4, num_experts_per_tok=2,
                    num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2, head_dim=64, vocab_size=512)


@pytest.mark.parametrize("batch,attn_bits", [(1, 0), (3, 0), (1, 4)])
def test_decoder_generate_graphed_equals_eager_and_cache_is_consistent(batch, attn_bits):
    """The decode/prefill driver on a tiny Mixtral-architecture model: the CUDA-graphed decode step
    produces the tokens of the eager one, and a cached decode step sees the same context as a
    prefill over the whole sequence."""
    from gemq_b200.inference import MixtralDecoder, StaticCache, generate
    model = MixtralDecoder(seed=3, attn_bits=attn_bits, **TINY_DECODER)
    T, new = 16, 6
    prompt = torch.randint(0, 512, (batch, T), generator=torch.Generator().manual_seed(batch)).cuda()
    seq_g, stats = generate(model, prompt, new, StaticCache(model.config, T + new), graphed=True)
    seq_e, _ = generate(model, prompt, new, StaticCache(model.config, T + new), graphed=False)
    assert seq_g.shape == (batch, T + new) and torch.equal(seq_g, seq_e)
    assert stats["prefill_throughput"] > 0 and stats["decode_throughput"] > 0
    # cached step vs recomputation: prefill T tokens, decode token T; compare with a prefill of T + 1 tokens
    cache = StaticCache(model.config, T + new)
    model(seq_g[:, :T], cache, torch.arange(T, device="cuda"))
    cached = model(seq_g[:, T:T + 1], cache, torch.tensor([T], device="cuda")).float()
    full = model(seq_g[:, :T + 1], StaticCache(model.config, T + new), torch.arange(T + 1, device="cuda")).float()
    # the two differ by the MoE path taken (one-token vs n-token roundings) and bf16 attention
    assert float((cached - full).norm() / full.norm()) < 5e-2
