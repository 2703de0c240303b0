"""Benchmark of the quantised MoE layer: decode batch 1 (config 1, the headline) and prefill (config 3).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--layers L]

Decode.  One step = one MoE layer forward for one token: router, gate/up projections of the two
selected experts, SiLU*mul, down projections and the top-k combine, one kernel launch.
Successive steps walk through L distinct layers (as a decoder does) with different activations,
so the ~100 MB of weights a step reads left the 126 MB L2 long before they are read again.  With
N > 1 (torchrun) every rank runs an independent replica: batch-1 decode reads two experts per
token and has no exchange step.
Prefill (the `prefill` sub-record of the same JSON line).  4096 bf16 tokens, top-2 routing with
Dirichlet(0.5) expert popularity, mixed bits; one GPU: expert-sorted grouped GEMM; N GPUs:
experts sharded over the ranks, tokens exchanged with all-to-all (strong scaling).
Prints ONE JSON line.
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

D, FFN, E, A, G = 4096, 14336, 8, 2, 128
METRIC = "moe_layer_decode_tokens_per_s"
WORKLOAD = "mixtral8x7b_moe_layer_decode_bs1_mixed_1-4bit_g128 (config 1)"
PREFILL_WORKLOAD = "mixtral8x7b_moe_layer_prefill_4096tok_top2_dirichlet0.5_mixed_bits (config 3)"
LAYER_SEED0 = 100
# DRAM bytes (read + write) of one launch of the decode layer kernel over its algorithmic bytes,
# from an ncu capture of three launches (1.038, 1.035, 1.012); applied to the bench's own average bytes per launch.
DECODE_TRAFFIC_RATIO = 1.03
# DRAM bytes of one prefill call at N = 1 (gate/up launch + down launch), from an ncu capture.
PREFILL_TRAFFIC_BYTES = 497.4e6 + 218.5e6 + 464.7e6 + 55.2e6
MIN_TIMED_SECONDS = 0.5


def parse():
    p = argparse.ArgumentParser()
    p.add_argument("--gpus", type=int, default=1)
    p.add_argument("--steps", type=int, default=400)
    p.add_argument("--warmup", type=int, default=40)
    p.add_argument("--impl", default="ours", choices=["ours", "reference"])
    p.add_argument("--layers", type=int, default=8)
    p.add_argument("--no-prefill", action="store_true", help="leave the config-3 sub-record out")
    p.add_argument("--mode", default="bench", choices=["bench", "layer_only", "prefill_only", "cfg2_only", "generate"],
                   help="layer_only / prefill_only / cfg2_only: a short eager loop of one op for profilers; generate: the full "
                        "32-layer decoder (config 4), 512-token prompt, 256 greedy tokens; each prints its own JSON")
    p.add_argument("--batch", type=int, default=1, help="generate mode: sequences decoded together")
    p.add_argument("--gen-layers", type=int, default=32)
    p.add_argument("--prefill-tokens", type=int, default=4096)
    p.add_argument("--shape", default=None, metavar="D,FFN",
                   help="override the layer shape (hidden, ffn); only for quick checks of the JSON contract")
    args = p.parse_args()
    if args.shape:
        global D, FFN
        D, FFN = (int(v) for v in args.shape.split(","))
    return args


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        pk = json.load(open(path))
        return pk["hbm_gbs"], pk["bf16_tflops"], pk.get("bf16_tflops_sustained"), "measured"
    return 6650.0, 1590.0, 1400.0, "fallback"


def host_threads() -> int:
    try:
        return max(1, len(os.sched_getaffinity(0)))
    except AttributeError:
        return max(1, os.cpu_count() or 1)


class ClockSampler:
    """nvidia-smi in the background; samples are collected by a reader thread so that the caller
    can wait for the first one before the timed region starts."""
    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.proc, self.lines = None, []
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "100",
                 "-i", str(index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            return
        self.thread = threading.Thread(target=self._read, daemon=True)
        self.thread.start()

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line)

    def wait_first(self, timeout: float = 5.0):
        t0 = time.time()
        while self.proc is not None and not self.lines and time.time() - t0 < timeout:
            time.sleep(0.05)

    def mark(self) -> int:
        return len(self.lines)

    def stop(self, lo: int = 0, hi=None):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "samples": 0, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        self.thread.join(timeout=2)
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in self.lines[lo:hi]:
            parts = [s.strip() for s in line.split(",")]
            if len(parts) < 6:
                continue
            try:
                sm.append(float(parts[0]))
                mx.append(float(parts[1]))
            except ValueError:
                continue
            for n, v in zip(names, parts[2:6]):
                if v.lower() == "active":
                    reasons.add(n)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "samples": len(sm), "reasons": sorted(reasons)}


# ---- the reference arm / CPU baseline: the oracle's torch path on the host cores --------------------
def cpu_layers(n_layers: int):
    """The decode workload on the host: for each of the first layers of the bench (same seeds, hence
    the same per-expert bit widths as the GPU arm draws), the two experts the CPU router selects,
    as packed CPU tensors.  Codes and scales follow the same distributions as the GPU arm's."""
    import numpy as np
    import torch
    from gemq_b200.synth_bits import draw_expert_bits
    from oracle import gemq_oracle as O
    layers = []
    for li in range(n_layers):
        bits = draw_expert_bits(E, LAYER_SEED0 + li)
        rng = np.random.default_rng(LAYER_SEED0 + li)
        gate = torch.from_numpy((rng.standard_normal((E, D)) * 0.02).astype(np.float16))
        x = torch.from_numpy(rng.standard_normal((1, D)).astype(np.float16))
        wts, sel, _ = O.route_fp16(x, gate, A)

        def mat(n, k, b):
            q = rng.integers(0, 2 ** b, (n, k), dtype=np.uint8)
            s = (np.abs(rng.standard_normal((k // G, n))) * 0.01 + 1e-3).astype(np.float16)
            z = O.kernel_form_offset(s, (rng.random((k // G, n)) * (2 ** b - 1)).astype(np.float16))
            return tuple(torch.from_numpy(a) for a in (O.pack_kernel_form(q, b), s, z))

        experts = []
        for e in sel.view(-1).tolist():
            b = bits[e]
            experts.append((mat(FFN, D, b), mat(FFN, D, b), mat(D, FFN, b), b))
        layers.append(dict(x=x.float(), w=wts.view(-1).float(), experts=experts, bits=[ex[3] for ex in experts]))
    return layers


def cpu_step(layer):
    from oracle import cpu_baseline as CB
    acc = 0
    for (w1, w3, w2, b), wt in zip(layer["experts"], layer["w"]):
        acc = acc + float(wt) * CB.expert_ffn(layer["x"], w1, w3, w2, b, G).float()
    return acc


def cpu_measure(n_layers: int, steps: int, warmup: int, budget_s: float):
    """Time `steps` full layer-tokens on the host (all threads); steps are cut so that the timed
    loop stays within `budget_s`.  Returns (seconds per token, steps timed, warm-ups done, note)."""
    import torch
    threads = host_threads()
    torch.set_num_threads(threads)
    layers = cpu_layers(n_layers)
    t0 = time.perf_counter()
    cpu_step(layers[0])
    first = time.perf_counter() - t0
    warm = max(0, min(warmup, int(0.4 * budget_s / max(first, 1e-3))) - 1)
    for i in range(warm):
        cpu_step(layers[(i + 1) % n_layers])
    k = max(1, min(steps, int(0.6 * budget_s / max(first, 1e-3))))
    t0 = time.perf_counter()
    for i in range(k):
        cpu_step(layers[i % n_layers])
    dt = (time.perf_counter() - t0) / k
    note = (f"full layer-token per step (router on the host, unpack + de-quantise + fp32 matmul of w1, w3, w2 of the "
            f"2 selected experts at their drawn bit widths {[l['bits'] for l in layers]}, every call), "
            f"{n_layers} layers cycled, {k} steps timed after {warm + 1} warm-ups; torch threads={threads}, "
            f"os.cpu_count={os.cpu_count()}")
    return dt, k, warm + 1, note, threads


def decode_config(layers: int, world: int):
    """The workload both arms run; identical for `--impl ours` and `--impl reference`."""
    return {"workload": WORKLOAD if (D, FFN) == (4096, 14336) else f"shape override {D}x{FFN} (not the benchmark)",
            "hidden": D, "ffn": FFN, "experts": E, "top_k": A, "group": G,
            "layers_cycled": layers, "parallelism": f"replicas x{world}",
            "l2": f"inputs larger than L2: {layers} layers x ~100 MB touched per step, cycled"}


def run_reference(args, rank):
    if rank != 0:
        return
    n_layers = min(args.layers, 2)
    dt, k, warm, note, threads = cpu_measure(n_layers, args.steps, args.warmup, budget_s=150.0)
    tok_s = 1.0 / dt
    line = {"impl": "reference", "metric": METRIC, "value": tok_s, "unit": "tokens/s", "n_gpus": args.gpus,
            "steps": k, "warmup": warm, "ms_per_step": dt * 1e3, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": decode_config(args.layers, max(1, args.gpus)),
            "details": {"launch": "host cores only (the reference's torch path; no GPU work)",
                        "layers_cycled_on_host": n_layers},
            "cpu_baseline": {"value": tok_s, "unit": "tokens/s", "cores": threads, "kind": "port", "sample": note},
            "e2e": {"value": tok_s, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line))


# ---- profiler helpers ---------------------------------------------------------------------------------
def profile_loop(args, dev):
    """Eager launches of one op (no graphs), for ncu: warmup + steps iterations."""
    import torch
    from gemq_b200 import synth
    if args.mode == "prefill_only":
        T = args.prefill_tokens
        blk = synth.mixtral_block(seed=0, device=dev)
        x, w, sel, _ = prefill_inputs(T)
        x, w, sel = x.to(dev), w.to(dev), sel.to(dev)
        once = lambda i: blk._prefill(x, 1, True, routing=(w, sel))
        extra = {"tokens": T, "bits": blk._nbits_host}
    elif args.mode == "cfg2_only":
        B = args.batch
        blk = synth.deepseek_block(seed=0, device=dev)
        xs = [torch.randn(B, 1, 2048, device=dev, generator=torch.Generator(device=dev).manual_seed(10 * B + i)).half()
              for i in range(8)]
        once = lambda i: blk(xs[0])  # one activation: the bytes below are those of every call
        _, _, idx = blk._decode(xs[0].view(B, 2048), 2)
        distinct = sorted(set(idx.view(-1).tolist()))
        extra = {"batch": B, "distinct_experts": len(distinct),
                 "algorithmic_bytes": sum(3 * 2048 * 1408 * (blk._nbits_host[e] + 0.25) / 8 for e in distinct)
                 + 3 * 2048 * 2816 * 4.25 / 8 + 2 * 64 * 2048}
    else:
        L = args.layers
        blocks = [synth.mixtral_block(seed=LAYER_SEED0 + i, device=dev) for i in range(L)]
        gen = torch.Generator(device=dev).manual_seed(1234)
        xs = torch.randn(16, 1, 1, D, device=dev, generator=gen).to(torch.float16)
        once = lambda i: blocks[i % L](xs[i % 16])
        extra = {"bits_of_selected_experts": [[blocks[i % L]._nbits_host[e] for e in
                                               blocks[i % L]._decode(xs[i % 16].view(1, D), 0)[2][0].tolist()]
                                              for i in range(min(16, args.steps + args.warmup))]}
    for i in range(args.warmup):
        once(i)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(args.steps):
        once(args.warmup + i)
    e1.record()
    torch.cuda.synchronize()
    print(json.dumps({"mode": args.mode, "steps": args.steps, "avg_us": e0.elapsed_time(e1) * 1e3 / args.steps, **extra}))


def run_generate(args, dev):
    """Config 4: random-initialised Mixtral-8x7B-architecture decoder, bf16 attention, every expert
    quantised with mixed bits averaging 2.0; prompt of 512 random tokens, 256 greedy tokens."""
    import torch
    from gemq_b200.inference import MixtralDecoder, StaticCache, generate
    T, new, B = 512, 256, args.batch
    model = MixtralDecoder(device=dev, seed=1, num_hidden_layers=args.gen_layers)
    prompt = torch.randint(0, model.config.vocab_size, (B, T), generator=torch.Generator().manual_seed(B)).to(dev)
    generate(model, prompt, 8, StaticCache(model.config, T + new))  # warm-up (allocations, lazy module loads)
    seq, stats = generate(model, prompt, new, StaticCache(model.config, T + new))
    hbm_peak, _, _, kind = peaks()
    eb, ab = model.expert_bytes_per_token(), model.attention_bytes_per_token(T + new // 2, B)
    step_s = stats["decode_latency"] / (new - 1)
    print(json.dumps({
        "mode": "generate", "workload": "mixtral8x7b_architecture_random_init_greedy_decode (config 4)",
        "layers": args.gen_layers, "batch": B, "prompt_tokens": T, "new_tokens": new,
        "prefill_tokens_per_s": stats["prefill_throughput"], "decode_tokens_per_s": stats["decode_throughput"],
        "decode_ms_per_step": step_s * 1e3,
        # batch 1: a step streams two experts per layer; larger batches touch most experts (not modelled here)
        "expert_bytes_per_step_bs1": eb, "attention_and_kv_bytes_per_step": ab,
        "hbm_frac_bs1": (eb + ab) / step_s / 1e9 / hbm_peak if B == 1 else None, "peak_kind": kind}))


def run_cfg2(dev):
    """Config 2: DeepSeek-V2-Lite-shaped layer (hidden 2048, intermediate 1408, 64 experts, top-6, two shared
    experts at 4 bits), decode batches of 1 and 16 rows.  Bytes: every distinct selected expert once, the
    shared experts once, the router matrix, at (b + 0.25) / 8 bytes per weight."""
    import torch
    from gemq_b200 import synth
    blk = synth.deepseek_block(seed=0, device=dev)
    hbm_peak, _, _, kind = peaks()
    Dd, Fd, SFd, Ed = 2048, 1408, 2816, 64
    out = {"workload": "deepseek_v2_lite_moe_layer_decode_bs1-16_mixed_bits (config 2)", "peak_kind": kind}
    for B in (1, 16):
        xs = [torch.randn(B, 1, Dd, device=dev, generator=torch.Generator(device=dev).manual_seed(10 * B + i)).half()
              for i in range(8)]
        byts = []
        for x in xs:
            _, _, idx = blk._decode(x.view(B, Dd), 2)
            distinct = set(idx.view(-1).tolist())
            byts.append(sum(3 * Dd * Fd * (blk._nbits_host[e] + 0.25) / 8 for e in distinct)
                        + 3 * Dd * SFd * 4.25 / 8 + 2 * Ed * Dd)
        for i in range(8):
            blk(xs[i % 8])
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        n = 64
        e0.record()
        for i in range(n):
            blk(xs[i % 8])
        e1.record()
        torch.cuda.synchronize()
        s = e0.elapsed_time(e1) * 1e-3 / n
        out[f"bs{B}"] = {"tokens_per_s": B / s, "us_per_step": s * 1e6, "algorithmic_bytes_per_step": sum(byts) / len(byts),
                         "hbm_frac": sum(byts) / len(byts) / s / 1e9 / hbm_peak,
                         "path": "one-launch layer kernel per row" if B <= 4 else "expert-sorted grouped GEMM"}
    return out


def prefill_inputs(T: int):
    import torch
    g = torch.Generator().manual_seed(7)
    torch.manual_seed(7)
    pop = torch.distributions.Dirichlet(torch.full((E,), 0.5)).sample()
    sel = torch.multinomial(pop.expand(T, E), A, replacement=False, generator=g)
    w = torch.softmax(torch.randn(T, A, generator=g), -1).to(torch.bfloat16)
    x = torch.randn(T, D, generator=g).to(torch.bfloat16)
    return x, w, sel, pop


def run_prefill(args, rank, local_rank, world, dev):
    """Config 3 on this process group; returns the sub-record (rank 0) or None."""
    import torch
    import torch.distributed as dist
    from gemq_b200 import synth
    T = args.prefill_tokens
    x_all, w_all, sel_all, _ = prefill_inputs(T)
    lo, hi = rank * T // world, (rank + 1) * T // world
    xh = x_all[lo:hi].contiguous().pin_memory()
    x, w, sel = xh.to(dev), w_all[lo:hi].to(dev), sel_all[lo:hi].to(dev)
    placement = None
    if world > 1:
        layer, bits, placement = synth.mixtral_expert_parallel(rank, world, seed=0, device=dev,
                                                               routed_rows=torch.bincount(sel_all.view(-1), minlength=E))
        step = lambda xin: layer.forward_routed(xin, w, sel)
    else:
        blk = synth.mixtral_block(seed=0, device=dev)
        bits = blk._nbits_host
        step = lambda xin: blk._prefill(xin, 1, True, routing=(w, sel))[0]
    steps = max(3, min(args.steps, 20))
    warm = max(3, min(args.warmup, 5))
    for _ in range(warm):
        step(x)
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        out = step(x)
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1)
    oh = torch.empty(hi - lo, D, dtype=torch.bfloat16).pin_memory()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    for _ in range(steps):
        out = step(xh.to(dev, non_blocking=True))
        oh.copy_(out, non_blocking=True)
        torch.cuda.current_stream().synchronize()
    e2e_s = time.perf_counter() - t0
    if world > 1:
        t = torch.tensor([ms, e2e_s * 1e3], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms, e2e_s = float(t[0]), float(t[1]) * 1e-3
    if rank != 0:
        return None
    _, peak_tf, peak_sus, kind = peaks()
    flops = 2.0 * T * A * 3 * D * FFN
    ach = flops / (ms / steps * 1e-3) / 1e12
    rows = torch.bincount(sel_all.view(-1), minlength=E).tolist()
    if placement is None:
        share = 1.0
    else:
        per_rank = [sum(rows[e] * sh for e, r, sh in placement if r == k) for k in range(world)]
        share = max(per_rank) / float(sum(rows))
    rec = {"metric": "moe_layer_prefill_tokens_per_s", "value": T * steps / (ms * 1e-3), "unit": "tokens/s",
           "steps": steps, "warmup": warm, "ms_per_step": ms / steps, "scaling": "strong", "dtype": "f16",
           "config": {"workload": PREFILL_WORKLOAD, "tokens": T, "bits": bits, "tokens_per_rank": hi - lo,
                      "parallelism": f"expert-parallel x{world}" if world > 1 else "one GPU",
                      "routed_rows_per_expert": rows,
                      # [expert, rank, share of the expert's rows]: an expert above a rank's fair share has replicas
                      "expert_rank_share": [[e, r, round(sh, 4)] for e, r, sh in placement] if placement else None,
                      # share of the routed rows on the busiest rank (1/world = perfectly even): the ceiling of
                      # the speed-up over one GPU is 1 / share
                      "busiest_rank_row_share": share,
                      "l2": "inputs larger than L2: ~0.4 GB of packed weights per step"},
           "e2e": {"value": T * steps / e2e_s, "unit": "tokens/s", "h2d_bytes_per_step": 2 * T * D // world,
                   "d2h_bytes_per_step": 2 * T * D // world},
           "roofline": {"bound": "tensor", "kernel": "grouped_gemm_kernel (gate/up + down; whole prefill call timed)",
                        "achieved": ach / world, "peak": peak_tf, "peak_kind": kind, "unit": "TFLOP/s",
                        "frac": ach / world / peak_tf, "frac_sustained": ach / world / peak_sus if peak_sus else None,
                        "traffic": PREFILL_TRAFFIC_BYTES if world == 1 and T == 4096 else None}}
    return rec


def main():
    args = parse()
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if args.impl == "reference":
        run_reference(args, rank)
        return

    import torch
    import torch.distributed as dist
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: gemq_b200 has no CPU path (use --impl reference for the CPU arm)")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if args.mode == "generate":
        run_generate(args, dev)
        return
    if args.mode != "bench":
        profile_loop(args, dev)
        return
    if world > 1:
        os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
        dist.init_process_group("nccl", device_id=dev)

    from gemq_b200 import synth

    sampler = ClockSampler(local_rank)
    L = args.layers
    blocks = [synth.mixtral_block(seed=LAYER_SEED0 + i, device=dev) for i in range(L)]
    gen = torch.Generator(device=dev).manual_seed(1234)
    n_x = 64
    xs = torch.randn(n_x, 1, 1, D, device=dev, generator=gen).to(torch.float16)
    torch.cuda.synchronize()
    pairs = [(i % L, i % n_x) for i in range(max(L, 16))]
    fused = not os.environ.get("GEMQ_B200_DECODE", "").startswith("s")
    launches_per_step = 1 if fused else 3

    # ---- device-resident throughput: CUDA graphs of consecutive steps ----------------------------
    # A decoder's captured forward chains its MoE layers inside one graph, each kernel's prologue
    # overlapping its predecessor's tail (programmatic dependent launch).  The timed loop replays a
    # graph of len(pairs) consecutive steps (different layers and activations); a remainder of the
    # requested step count runs as one-step graphs.
    graphs = []
    side = torch.cuda.Stream(device=dev)
    with torch.cuda.stream(side):
        for li, xi in pairs:
            blocks[li](xs[xi])
        torch.cuda.synchronize()
        for li, xi in pairs:
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=side):
                o, _ = blocks[li](xs[xi])
            graphs.append((g, o))
        chain = torch.cuda.CUDAGraph()
        with torch.cuda.graph(chain, stream=side):
            for li, xi in pairs:
                blocks[li](xs[xi])
    torch.cuda.synchronize()
    chain_len = len(pairs)

    def run_steps(n):
        for _ in range(n // chain_len):
            chain.replay()
        for i in range(n % chain_len):
            graphs[i][0].replay()

    sampler.wait_first()
    run_steps(args.warmup)
    torch.cuda.synchronize()
    # calibrate the number of passes of the step loop so that the timed region lasts >= MIN_TIMED_SECONDS
    c0, c1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    c0.record()
    run_steps(min(args.steps, 50))
    c1.record()
    torch.cuda.synchronize()
    est = c0.elapsed_time(c1) * 1e-3 / min(args.steps, 50)
    passes = max(1, int(MIN_TIMED_SECONDS / max(est * args.steps, 1e-9)) + 1)
    if world > 1:
        t = torch.tensor([passes], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        passes = int(t.item())
        dist.barrier()
    torch.cuda.synchronize()
    mark0 = sampler.mark()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(passes):
        run_steps(args.steps)
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1)
    if world > 1:
        t = torch.tensor([ms], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    total_steps = passes * args.steps
    tok_s = world * total_steps / (ms * 1e-3)

    # ---- end to end: pinned host input -> device -> layer -> pinned host output, every step -----
    # One CUDA graph per layer holds the host-to-device copy of the staged activation, the layer
    # and the device-to-host copy of its output (the way a decode loop under torch.compile's
    # reduce-overhead mode calls the block); per step the host copies the next activation into the
    # pinned staging buffer, replays the graph, waits for it and reads the output.
    xh = [xs[i].cpu() for i in range(n_x)]
    stage_in = torch.empty(1, 1, D, dtype=torch.float16).pin_memory()
    stage_out = torch.empty(1, 1, D, dtype=torch.float16).pin_memory()
    x_dev = torch.empty(1, 1, D, dtype=torch.float16, device=dev)
    e2e_graphs = []
    with torch.cuda.stream(side):
        stage_in.copy_(xh[0])
        for li in range(L):
            x_dev.copy_(stage_in, non_blocking=True)
            o, _ = blocks[li](x_dev)
            stage_out.copy_(o, non_blocking=True)
        torch.cuda.synchronize()
        for li in range(L):
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=side):
                x_dev.copy_(stage_in, non_blocking=True)
                o, _ = blocks[li](x_dev)
                stage_out.copy_(o, non_blocking=True)
            e2e_graphs.append(g)
    torch.cuda.synchronize()
    sink = 0.0

    # host side of a step through views of the pinned buffers (numpy float16 views share their memory):
    # the copy into the staging buffer and the read of the result cost a fraction of a microsecond
    # instead of several tensor-method calls
    xh_np = [t.view(-1).numpy() for t in xh]
    in_np, out_np = stage_in.view(-1).numpy(), stage_out.view(-1).numpy()
    cur = torch.cuda.current_stream()

    def e2e_steps(n):
        nonlocal sink
        for i in range(n):
            in_np[:] = xh_np[i % n_x]
            e2e_graphs[i % L].replay()
            cur.synchronize()
            sink += float(out_np[0])

    e2e_steps(max(3, args.warmup // 4))
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    e2e_steps(args.steps)
    torch.cuda.synchronize()
    e2e_s = time.perf_counter() - t0
    if world > 1:
        t = torch.tensor([e2e_s], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_s = float(t.item())
    e2e_tok_s = world * args.steps / e2e_s

    # ---- roofline of the dominant kernel: the layer kernel itself (one launch per step) ---------
    routed = []
    for li, xi in pairs:
        _, _, idx = blocks[li]._decode(xs[xi].view(1, D), 0)
        routed.append(idx[0].tolist())
    torch.cuda.synchronize()
    step_bytes = []
    for (li, xi), sel in zip(pairs, routed):
        bits = [blocks[li]._nbits_host[e] for e in sel]
        # per selected expert three matrices at (b + 0.25) / 8 bytes per weight; router matrix; x in, y out
        step_bytes.append(sum(3 * FFN * D * (b + 0.25) / 8 for b in bits) + 2 * E * D + 2 * D + 2 * D)
    n_k = len(pairs)
    with torch.cuda.stream(side):
        kgraph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(kgraph, stream=side):
            for li, xi in pairs:
                blocks[li](xs[xi])
    torch.cuda.synchronize()
    reps = max(3, min(args.steps, 400) // n_k)
    for _ in range(3):
        kgraph.replay()
    torch.cuda.synchronize()
    u0, u1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    u0.record()
    for _ in range(reps):
        kgraph.replay()
    u1.record()
    torch.cuda.synchronize()
    mark1 = sampler.mark()
    k_avg_s = u0.elapsed_time(u1) * 1e-3 / (reps * n_k * launches_per_step)
    alg = sum(step_bytes) / len(step_bytes)
    hbm_peak, _, _, peak_kind = peaks()
    achieved = alg / launches_per_step / k_avg_s / 1e9 if fused else None

    prefill, cfg2 = None, None
    if not args.no_prefill:
        del graphs, chain, e2e_graphs, kgraph
        prefill = run_prefill(args, rank, local_rank, world, dev)
        if rank == 0 and world == 1:
            cfg2 = run_cfg2(dev)
    clocks = sampler.stop(mark0, mark1 + 1)

    if rank == 0:
        line = {
            "metric": METRIC, "value": tok_s, "unit": "tokens/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "passes": passes, "ms_per_step": ms / total_steps, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "f16", "data": "synthetic",
            "config": decode_config(L, world),
            "details": {"launch": f"CUDA graphs of {chain_len} consecutive steps (device-resident arm); CUDA graph of H2D copy + "
                                  "layer + D2H copy per step, host waits for every step (e2e arm)",
                        "approx_bytes_per_step": alg, "timed_seconds": ms * 1e-3},
            "e2e": {"value": e2e_tok_s, "unit": "tokens/s", "h2d_bytes_per_step": 2 * D, "d2h_bytes_per_step": 2 * D},
            "gpu_launches": launches_per_step * total_steps,
            "clocks": clocks,
            "roofline": {"bound": "hbm",
                         "kernel": "moe_decode_kernel (router + gate/up + down + combine, one launch per layer)"
                         if fused else "three launches per layer (router, gate/up GEMV, down GEMV)",
                         "achieved": achieved if fused else alg / (ms / total_steps * 1e-3) / 1e9,
                         "peak": hbm_peak, "peak_kind": peak_kind, "unit": "GB/s",
                         "frac": (achieved if fused else alg / (ms / total_steps * 1e-3) / 1e9) / hbm_peak,
                         "traffic": alg * DECODE_TRAFFIC_RATIO, "algorithmic_bytes_per_launch": alg / launches_per_step,
                         "avg_launch_us": k_avg_s * 1e6,
                         "layer_frac": alg / (ms / total_steps * 1e-3) / 1e9 / hbm_peak},
        }
        if world == 1:
            dt, k, warm, note, threads = cpu_measure(min(L, 2), 20, 2, budget_s=15.0)
            line["cpu_baseline"] = {"value": 1.0 / dt, "unit": "tokens/s", "cores": threads, "kind": "port", "sample": note}
        else:
            line["cpu_baseline"] = None
        if prefill is not None:
            line["prefill"] = prefill
        if cfg2 is not None:
            line["decode_cfg2"] = cfg2
        print(json.dumps(line))
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
