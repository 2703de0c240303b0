"""Layer-level parity of the quantised MoE blocks with the CPU oracle."""
import numpy as np
import pytest
import torch

from oracle import gemq_oracle as O
from conftest import MAX_ABS_TOL, REL_FRO_TOL, max_abs, rel_fro
import moe_fixtures as MF

pytestmark = pytest.mark.gpu


def check(got, want):
    got = got.float().cpu().numpy()
    want = np.asarray(want, dtype=np.float32)
    assert rel_fro(got, want) < REL_FRO_TOL, f"rel-Frobenius {rel_fro(got, want):.3e}"
    assert max_abs(got, want) < MAX_ABS_TOL, f"max-abs {max_abs(got, want):.3e}"


def clear_margin(logits, k, eps=2e-2):
    v = np.sort(np.asarray(logits, dtype=np.float64).ravel())[::-1]
    return (v[k - 1] - v[k]) > eps * max(1.0, abs(v[k - 1]))


@pytest.mark.parametrize("seed", [0, 1, 2])
def test_mixtral_one_token_small(seed):
    layer = MF.make_layer("mixtral", D=256, Fd=512, E=4, A=2, bits=[1, 2, 3, 4], seed=seed, gate_std=0.02)
    blk = MF.gpu_block(layer)
    w1, w3, w2, _ = MF.oracle_parts(layer)
    x = torch.randn(1, 256, generator=torch.Generator().manual_seed(seed)).half()
    out, aux = blk(x.cuda().view(1, 1, -1))
    assert aux is None and out.shape == (1, 1, 256) and out.dtype == torch.float16
    _, gw, gi = blk._decode(x.cuda(), 0)
    ref_out, ew, ei = O.moe_one_token(x, torch.from_numpy(layer["gate"]), 2, w1, w3, w2, "mixtral")
    # against fp32-accumulated math with the routing the GPU chose
    check(out.view(1, -1), O.moe_reference_fp32(x, gw.float().cpu(), gi.cpu(), w1, w3, w2))
    scores = (x.float() @ torch.from_numpy(layer["gate"]).float().t()).numpy()
    if clear_margin(scores, 2):
        assert sorted(gi.cpu().view(-1).tolist()) == sorted(ei.view(-1).tolist())
        check(out.view(1, -1), ref_out.float().numpy())
        order = np.argsort(gi.cpu().view(-1).numpy()), np.argsort(ei.view(-1).numpy())
        assert np.allclose(gw.float().cpu().view(-1).numpy()[order[0]], ew.float().view(-1).numpy()[order[1]], atol=2e-3)


@pytest.mark.parametrize("norm", [False, True])
def test_deepseek_one_token_small(norm):
    layer = MF.make_layer("deepseek", D=256, Fd=384, E=16, A=6, bits=[1, 2, 3, 4] * 4, seed=3, gate_std=1 / 16.0,
                          n_shared=2, shared_bits=4, norm_topk_prob=norm)
    blk = MF.gpu_block(layer)
    w1, w3, w2, sh = MF.oracle_parts(layer)
    x = torch.randn(1, 256, generator=torch.Generator().manual_seed(9)).half()
    out = blk(x.cuda().view(1, 1, -1))
    assert isinstance(out, torch.Tensor) and out.shape == (1, 1, 256)
    _, gw, gi = blk._decode(x.cuda(), 2)
    check(out.view(1, -1), O.moe_reference_fp32(x, gw.float().cpu(), gi.cpu(), w1, w3, w2, sh))
    ref_out, ew, ei = O.moe_one_token(x, torch.from_numpy(layer["gate"]), 6, w1, w3, w2, "deepseek", norm, sh)
    logits = (x.float() @ torch.from_numpy(layer["gate"]).float().t()).numpy()
    if clear_margin(logits, 6):
        assert sorted(gi.cpu().view(-1).tolist()) == sorted(ei.view(-1).tolist())
        check(out.view(1, -1), ref_out.float().numpy())


def test_deepseek_decode_batch_rows():
    """[B, 1, D] decode batches take the n-token path of the reference (fp32 routing)."""
    layer = MF.make_layer("deepseek", D=256, Fd=384, E=16, A=6, bits=[1, 2, 3, 4] * 4, seed=4, gate_std=1 / 16.0,
                          n_shared=2)
    blk = MF.gpu_block(layer)
    w1, w3, w2, sh = MF.oracle_parts(layer)
    x = torch.randn(5, 256, generator=torch.Generator().manual_seed(1)).half()
    out = blk(x.cuda().view(5, 1, -1)).view(5, -1)
    _, gw, gi = blk._decode(x.cuda(), 2)
    check(out, O.moe_reference_fp32(x, gw.float().cpu(), gi.cpu(), w1, w3, w2, sh))


def test_mixtral_n_tokens_small():
    layer = MF.make_layer("mixtral", D=256, Fd=512, E=4, A=2, bits=[4, 1, 3, 2], seed=5, gate_std=0.02)
    blk = MF.gpu_block(layer)
    w1, w3, w2, _ = MF.oracle_parts(layer)
    x = torch.randn(37, 256, generator=torch.Generator().manual_seed(2)).half()
    out, logits = blk(x.cuda().view(1, 37, -1))
    assert logits.shape == (37, 4)
    rw, sel, _ = blk._route(x.cuda(), 1, True)
    ref_out, ew, ei, ref_logits = O.moe_n_tokens(x, torch.from_numpy(layer["gate"]), 2, w1, w3, w2, "mixtral")
    assert np.allclose(logits.float().cpu().numpy(), ref_logits.float().numpy(), atol=2e-3)
    same = (sel.cpu().sort(dim=1).values == ei.sort(dim=1).values).all(dim=1)
    assert same.float().mean() > 0.9
    got = out.view(37, -1).float().cpu()[same]
    check(got, ref_out.float()[same].numpy())


def test_mixtral_config1_full_size_decode():
    """Mixtral-8x7B-shaped layer, decode batch 1, mixed bits with mean in [1.5, 2.5]."""
    from gemq_b200 import synth
    blk = synth.mixtral_block(seed=0)
    x = torch.randn(1, 1, 4096, generator=torch.Generator().manual_seed(0)).half().cuda()
    out, _ = blk(x)
    _, gw, gi = blk._decode(x.view(1, -1), 0)
    # oracle on the two selected experts only, from the block's own packed tensors
    sel = gi.view(-1).tolist()
    D, Fd, G = 4096, 14336, 128
    acc = np.zeros(D, dtype=np.float64)
    xf = x.view(1, -1).float().cpu().numpy()
    for a, e in enumerate(sel):
        b = blk._nbits_host[e]

        def mat(name, K, N):
            off = int(getattr(blk, f"{name}_wq_strides")[e])
            rows = -(-K // (32 // b))
            wq = getattr(blk, f"{name}_wq").view(-1)[off:off + rows * N].view(rows, N).cpu().numpy()
            zo = int(getattr(blk, f"{name}_zs_strides")[e])
            s = getattr(blk, f"{name}_scales").view(-1)[zo:zo + (K // G) * N].view(K // G, N).cpu().numpy()
            z = getattr(blk, f"{name}_zeros").view(-1)[zo:zo + (K // G) * N].view(K // G, N).cpu().numpy()
            return O.dequantize(wq, s, z, b, G, K).astype(np.float32)

        h1 = xf @ mat("w1", D, Fd)
        h3 = xf @ mat("w3", D, Fd)
        h = (h1 / (1 + np.exp(-h1))) * h3
        acc += float(gw.view(-1)[a]) * (h @ mat("w2", Fd, D))[0]
    check(out.view(1, -1), acc[None, :])
    out2, _ = blk(x)
    assert torch.equal(out, out2)


def test_gemm_tc_vs_oracle():
    """tcgen05 GEMM: single matrix, every bit-width, ragged last row tile."""
    from gemq_b200.kernels import dequant_gemm
    from gemq_b200.kernels._runtime import error_word
    for N in (256, 384):  # 256 columns per CTA, and the 128-column form (N not a multiple of 256)
        for b in (1, 2, 3, 4):
            rng = np.random.default_rng(40 + b + N)
            K, M = 512, 200
            lin = MF.draw_linear(rng, N, K, b)
            x = rng.standard_normal((M, K)).astype(np.float16)
            t = lambda a: torch.from_numpy(np.ascontiguousarray(a)).cuda()
            y = dequant_gemm(t(x), t(lin["wq"]), t(lin["s"]), t(lin["z"]), b, 128)
            assert int(error_word(y.device).item()) == 0
            check(y, O.dequant_gemm(x, lin["wq"], lin["s"], lin["z"], b, 128))


def test_gemm_tc_weights_bit_exact():
    """Identity activations read the de-quantised weights back through the tensor cores:
    they must equal the reference's fp16(fma(q, s, z)) bit for bit, at every bit width
    (3-bit: all five window offsets inside a word occur within 160 reduction elements)."""
    from gemq_b200.kernels import dequant_gemm
    for b in (1, 2, 3, 4):
        rng = np.random.default_rng(70 + b)
        N, K = 384, 640
        lin = MF.draw_linear(rng, N, K, b)
        x = np.eye(K, dtype=np.float16)
        t = lambda a: torch.from_numpy(np.ascontiguousarray(a)).cuda()
        y = dequant_gemm(t(x), t(lin["wq"]), t(lin["s"]), t(lin["z"]), b, 128)
        want = O.dequantize(lin["wq"], lin["s"], lin["z"], b, 128, K)  # [K, N] fp16
        assert np.array_equal(y.cpu().numpy().view(np.uint16), np.ascontiguousarray(want).view(np.uint16)), f"bits={b}"


def test_mixtral_prefill_grouped_gemm():
    layer = MF.make_layer("mixtral", D=256, Fd=512, E=4, A=2, bits=[4, 1, 3, 2], seed=6, gate_std=0.02)
    blk = MF.gpu_block(layer)
    assert blk._prefill_ok()
    w1, w3, w2, _ = MF.oracle_parts(layer)
    T = 300
    x = torch.randn(T, 256, generator=torch.Generator().manual_seed(3)).half()
    out, logits = blk(x.cuda().view(1, T, -1))
    assert blk.prefill_error_code(T) == 0
    _, gw, gi, _ = blk._prefill(x.cuda(), 1, True)
    ref = O.moe_reference_fp32(x, gw.float().cpu(), gi.cpu(), w1, w3, w2)
    check(out.view(T, -1), ref.numpy())
    ref_out, ew, ei, ref_logits = O.moe_n_tokens(x, torch.from_numpy(layer["gate"]), 2, w1, w3, w2, "mixtral")
    same = (gi.cpu().sort(dim=1).values == ei.sort(dim=1).values).all(dim=1)
    assert same.float().mean() > 0.9
    check(out.view(T, -1).float().cpu()[same], ref_out.float()[same].numpy())
    out2, _ = blk(x.cuda().view(1, T, -1))
    assert torch.equal(out, out2)


def test_deepseek_prefill_with_shared_experts_bf16():
    layer = MF.make_layer("deepseek", D=256, Fd=384, E=16, A=6, bits=[1, 2, 3, 4] * 4, seed=8, gate_std=1 / 16.0,
                          n_shared=2)
    blk = MF.gpu_block(layer)
    assert blk._prefill_ok()
    w1, w3, w2, sh = MF.oracle_parts(layer)
    T = 70
    x = torch.randn(T, 256, generator=torch.Generator().manual_seed(4)).to(torch.bfloat16)
    out = blk(x.cuda().view(1, T, -1)).view(T, -1)
    assert out.dtype == torch.bfloat16 and blk.prefill_error_code(T) == 0
    _, gw, gi, _ = blk._prefill(x.cuda(), 2, False)
    ref = O.moe_reference_fp32(x.float(), gw.float().cpu(), gi.cpu(), w1, w3, w2, sh).numpy()
    got = out.float().cpu().numpy()
    # bf16 output and bf16 per-expert contributions (8 mantissa bits); the GEMMs run on fp16 operands
    assert rel_fro(got, ref) < REL_FRO_TOL, rel_fro(got, ref)
    assert max_abs(got, ref) < max(MAX_ABS_TOL, 2.0 ** -7 * float(np.abs(ref).max())), max_abs(got, ref)


def _ep_worker(rank, world, port, results):
    import os
    import torch.distributed as dist
    from gemq_b200 import synth
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    dims = dict(hidden_size=256, intermediate_size=512, num_local_experts=4, num_experts_per_tok=2)
    bits = [1, 2, 3, 4]
    # experts placed by (made-up) routed-row statistics: rank 0 holds expert 0 alone, rank 1 the other three
    ep, _, place = synth.mixtral_expert_parallel(rank, world, seed=5, device=dev, bits=bits, routed_rows=[90, 40, 30, 20],
                                                 **dims)
    assert place == [[0, 0, 1.0], [1, 1, 1.0], [2, 1, 1.0], [3, 1, 1.0]]
    # the same layer with expert 0 held by both ranks (60 % / 40 % of its rows) and expert 2 moved to rank 0
    from gemq_b200.inference.expert_parallel import Placement
    split = Placement([(0, 0, 0.6), (0, 1, 0.4), (1, 1, 1.0), (2, 0, 1.0), (3, 1, 1.0)], 4, world)
    ep2, _, _ = synth.mixtral_expert_parallel(rank, world, seed=5, device=dev, bits=bits, placement=split, **dims)
    full, _, _ = synth.mixtral_expert_parallel(0, 1, seed=5, device=dev, bits=bits, **dims)  # all experts, no exchange
    g = torch.Generator().manual_seed(11 + rank)
    T = 150 + 20 * rank
    x = torch.randn(T, 256, generator=g).half().to(dev)
    sel = torch.stack([torch.randperm(4, generator=g)[:2] for _ in range(T)]).to(dev)
    w = torch.softmax(torch.randn(T, 2, generator=g), -1).half().to(dev)
    y = ep.forward_routed(x, w, sel)
    # single-GPU result with the same routing: every row through its expert, same combine
    from gemq_b200.inference.expert_parallel import combine_in_expert_order
    rows = x.repeat_interleave(2, 0)
    yy = full.local._prefill(rows, 1, True, routing=(w.reshape(-1, 1), sel.reshape(-1, 1)))[0]
    ref = combine_in_expert_order(yy.view(T, 2, -1), sel)
    y2 = ep2.forward_routed(x, w, sel)
    results[rank] = max(float((y.float() - ref.float()).abs().max()), float((y2.float() - ref.float()).abs().max()))
    dist.barrier()
    dist.destroy_process_group()


def test_expert_parallel_two_gpus_matches_single_gpu():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    import torch.multiprocessing as mp
    mgr = mp.Manager()
    results = mgr.dict()
    mp.spawn(_ep_worker, args=(2, 29611, results), nprocs=2, join=True)
    assert max(results.values()) == 0.0, dict(results)
