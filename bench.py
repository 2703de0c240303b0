"""Benchmark of the quantised MoE decode layer (Mixtral-8x7B shape, batch 1, mixed bits).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--layers L]

One step = one MoE layer forward for one token: router, fused gate/up GEMV of the two
selected experts, SiLU*mul + down GEMV, top-k combine.  Successive steps walk through L
distinct layers (as a decoder does) with different activations, so the ~100 MB of weights
a step reads were evicted from the 126 MB L2 long before they are read again.  Prints ONE
JSON line.  With N > 1 (torchrun) every rank runs an independent replica: batch-1 decode
reads two experts per token and has no exchange step.
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

D, FFN, E, A, G = 4096, 14336, 8, 2, 128
METRIC = "moe_layer_decode_tokens_per_s"
WORKLOAD = "mixtral8x7b_moe_layer_decode_bs1_mixed_1-4bit_g128 (config 1)"
# dram bytes per launch of the up-projection kernel measured with ncu on this workload; None
# until a capture has been summarised under profiles/.
# ncu (profiles/gemv_stream_kernel_decode_layer.md): dram read + write of three captured launches
# = 1.033 x their algorithmic bytes (reads alone 1.002 x); applied to the bench's own average.
UP_KERNEL_TRAFFIC_RATIO = 1.033


def parse():
    p = argparse.ArgumentParser()
    p.add_argument("--gpus", type=int, default=1)
    p.add_argument("--steps", type=int, default=400)
    p.add_argument("--warmup", type=int, default=40)
    p.add_argument("--impl", default="ours", choices=["ours", "reference"])
    p.add_argument("--layers", type=int, default=8)
    p.add_argument("--cpu-sample-cols", type=int, default=1792)
    p.add_argument("--workload", default="decode", choices=["decode", "prefill"],
                   help="decode: config 1 (default, the headline metric); prefill: config 3, 4096-token grouped GEMM, "
                        "expert-parallel over the ranks when launched with torchrun")
    p.add_argument("--mode", default="bench", choices=["bench", "up_only", "layer_only"],
                   help="up_only / layer_only: a short eager loop of one op for profilers; prints its own timing")
    return p.parse_args()


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        return json.load(open(path))["hbm_gbs"], "measured"
    return 6650.0, "fallback"


class ClockSampler:
    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.proc = None
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "100",
                 "-i", str(index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            pass

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
            out, _ = self.proc.communicate()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in out.strip().splitlines():
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


def cpu_reference_sample(cols: int, threads_note: str):
    """Reference-convention torch path on the host: one token through A experts, on a column
    slice of every matrix; returns seconds per full layer-token (extrapolated) and a note."""
    import torch
    from oracle import cpu_baseline as CB
    from oracle import gemq_oracle as O
    import numpy as np
    rng = np.random.default_rng(0)
    bits = [2, 2]  # mean-2-bit pair of experts
    frac = cols / FFN
    dcols = max(128, int(D * frac) // 128 * 128)

    def mat(n, k, b):
        q = rng.integers(0, 2 ** b, (n, k), dtype=np.uint8)
        s = (np.abs(rng.standard_normal((k // G, n))) * 0.01 + 1e-3).astype(np.float16)
        z = O.kernel_form_offset(s, (rng.random((k // G, n)) * (2 ** b - 1)).astype(np.float16))
        return tuple(torch.from_numpy(a) for a in (O.pack_kernel_form(q, b), s, z))

    experts = [(mat(cols, D, b), mat(cols, D, b), mat(dcols, cols, b), b) for b in bits]
    x = torch.randn(1, D)

    def step():
        acc = 0
        for w1, w3, w2, b in experts:
            acc = acc + CB.expert_ffn(x, w1, w3, w2, b, G).float()
        return acc

    t = CB.time_best(step, repeats=3, warmup=1)
    # work is linear in weights touched: (2*cols*D + dcols*cols) of (3*FFN*D) per expert
    scale = (3.0 * FFN * D) / (2.0 * cols * D + dcols * cols)
    note = (f"A=2 experts at 2 bits, {cols}/{FFN} ffn columns x {D} and {dcols}/{D} x {cols} down columns, "
            f"dequant+matmul every call, time scaled x{scale:.1f} to the full layer; {threads_note}")
    return t * scale, note, step


def run_reference(args, rank):
    import torch
    if rank != 0:
        return
    threads = torch.get_num_threads()
    per_token_s, note, step = cpu_reference_sample(args.cpu_sample_cols, f"torch threads={threads}, os.cpu_count={os.cpu_count()}")
    # K timed steps of the bounded sample (each step = the sample once)
    for _ in range(min(args.warmup, 2)):
        step()
    k = max(1, min(args.steps, 20))
    t0 = time.perf_counter()
    for _ in range(k):
        step()
    dt = (time.perf_counter() - t0) / k
    # use the loop timing (same sample, same scaling as cpu_reference_sample)
    cols = args.cpu_sample_cols
    dcols = max(128, int(D * cols / FFN) // 128 * 128)
    factor = (3.0 * FFN * D) / (2.0 * cols * D + dcols * cols)
    tok_s = 1.0 / (dt * factor)
    line = {"impl": "reference", "metric": METRIC, "value": tok_s, "unit": "tokens/s", "n_gpus": args.gpus,
            "steps": k, "warmup": min(args.warmup, 2), "ms_per_step": dt * factor * 1e3, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": WORKLOAD},
            "cpu_baseline": {"value": tok_s, "unit": "tokens/s", "cores": threads, "kind": "port", "sample": note},
            "e2e": {"value": tok_s, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line))


def profile_loop(args, blocks, xs, pairs, dev):
    """Eager launches of one op (no graphs), for ncu: warmup + steps iterations."""
    import torch
    from gemq_b200.kernels import fused_dequant_up_proj
    routed = [blocks[li]._decode(xs[xi].view(1, D), 0)[2][0].clone() for li, xi in pairs]

    def once(i):
        li, xi = pairs[i % len(pairs)]
        b = blocks[li]
        if args.mode == "up_only":
            fused_dequant_up_proj(xs[xi].view(1, D), routed[i % len(pairs)], b.w1_wq, b.w3_wq, b.w1_scales,
                                  b.w1_zeros, b.w3_scales, b.w3_zeros, b.w1_nbits, b.w1_wq_strides, G)
        else:
            b(xs[xi])

    for i in range(args.warmup):
        once(i)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(args.steps):
        once(i)
    e1.record()
    torch.cuda.synchronize()
    bits = [[blocks[li]._nbits_host[e] for e in r.tolist()] for (li, _), r in zip(pairs, routed)]
    print(json.dumps({"mode": args.mode, "steps": args.steps, "avg_us": e0.elapsed_time(e1) * 1e3 / args.steps,
                      "bits_of_selected_experts": bits[:args.steps + args.warmup]}))


def run_prefill(args, rank, local_rank, world):
    """Config 3: Mixtral-shaped layer, 4096 bf16 tokens, top-2 with Dirichlet(0.5) expert popularity,
    mixed bits.  One GPU: expert-sorted grouped GEMM.  N GPUs: experts sharded, tokens exchanged with
    all-to-all (strong scaling: the 4096 tokens are split over the ranks)."""
    import torch
    import torch.distributed as dist
    from gemq_b200 import synth
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    T, top_k = 4096, A
    g = torch.Generator().manual_seed(7)
    pop = torch.distributions.Dirichlet(torch.full((E,), 0.5)).sample() if False else None
    torch.manual_seed(7)
    pop = torch.distributions.Dirichlet(torch.full((E,), 0.5)).sample()
    sel_all = torch.multinomial(pop.expand(T, E), top_k, replacement=False, generator=g)
    w_all = torch.softmax(torch.randn(T, top_k, generator=g), -1).to(torch.bfloat16)
    x_all = torch.randn(T, D, generator=g).to(torch.bfloat16)
    lo, hi = rank * T // world, (rank + 1) * T // world
    xh = x_all[lo:hi].contiguous().pin_memory()
    x, w, sel = xh.to(dev), w_all[lo:hi].to(dev), sel_all[lo:hi].to(dev)
    if world > 1:
        layer, bits = synth.mixtral_expert_parallel(rank, world, seed=0, device=dev)
        step = lambda xin: layer.forward_routed(xin, w, sel)
    else:
        blk = synth.mixtral_block(seed=0, device=dev)
        bits = blk._nbits_host
        step = lambda xin: blk._prefill(xin, 1, True, routing=(w, sel))[0]
    for _ in range(args.warmup):
        step(x)
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    sampler = ClockSampler(local_rank)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        out = step(x)
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1)
    oh = torch.empty(hi - lo, D, dtype=torch.bfloat16).pin_memory()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        out = step(xh.to(dev, non_blocking=True))
        oh.copy_(out, non_blocking=True)
        torch.cuda.current_stream().synchronize()
    e2e_s = time.perf_counter() - t0
    clocks = sampler.stop()
    if world > 1:
        t = torch.tensor([ms, e2e_s * 1e3], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms, e2e_s = float(t[0]), float(t[1]) * 1e-3
    if rank == 0:
        flops = 2.0 * T * top_k * 3 * D * FFN
        peak_tf = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))["bf16_tflops"] if os.path.exists(
            os.path.join(ROOT, "MEASURED_PEAKS.json")) else 1590.0
        ach = flops / (ms / args.steps * 1e-3) / 1e12
        print(json.dumps({
            "metric": "moe_layer_prefill_tokens_per_s", "value": T * args.steps / (ms * 1e-3), "unit": "tokens/s",
            "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms / args.steps,
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f16", "data": "synthetic",
            "config": {"workload": "mixtral8x7b_moe_layer_prefill_4096tok_top2_dirichlet0.5_mixed_bits (config 3)",
                       "bits": bits, "tokens_per_rank": hi - lo, "parallelism": f"expert-parallel x{world}",
                       # share of the routed rows that lands on the busiest rank (1/world = perfectly even)
                       "busiest_rank_row_share": float(torch.bincount(sel_all.view(-1) // max(1, E // world),
                                                                      minlength=world).max()) / sel_all.numel(),
                       "l2": "inputs larger than L2: ~0.4 GB of packed weights per step"},
            "e2e": {"value": T * args.steps / e2e_s, "unit": "tokens/s", "h2d_bytes_per_step": 2 * T * D // world,
                    "d2h_bytes_per_step": 2 * T * D // world},
            "gpu_launches": 7 * args.steps, "clocks": clocks,
            "roofline": {"bound": "tensor", "kernel": "grouped_gemm_kernel (gate/up + down; whole prefill call timed)",
                         "achieved": ach / world, "peak": peak_tf, "unit": "TFLOP/s", "frac": ach / world / peak_tf,
                         # ncu (profiles/grouped_gemm_kernel_prefill_4096_tokens.md): dram read + write of one
                         # gate/up launch plus one down launch at N=1, bytes per prefill call
                         "traffic": (489.2e6 + 220.7e6 + 465.9e6 + 58.8e6) if world == 1 else None}}))
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def main():
    args = parse()
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if args.impl == "reference":
        run_reference(args, rank)
        return
    if args.workload == "prefill":
        run_prefill(args, rank, local_rank, world)
        return

    import torch
    import torch.distributed as dist
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: gemq_b200 has no CPU path (use --impl reference for the CPU arm)")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)

    from gemq_b200 import synth
    from gemq_b200.kernels import fused_dequant_up_proj

    L = args.layers
    blocks = [synth.mixtral_block(seed=100 + i, device=dev) for i in range(L)]
    gen = torch.Generator(device=dev).manual_seed(1234)
    n_x = 64
    xs = torch.randn(n_x, 1, 1, D, device=dev, generator=gen).to(torch.float16)
    torch.cuda.synchronize()

    pairs = [(i % L, i % n_x) for i in range(max(L, 16))]
    if args.mode != "bench":
        profile_loop(args, blocks, xs, pairs, dev)
        return

    # ---- device-resident throughput: one CUDA graph per (layer, activation) pair --------------
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
    torch.cuda.synchronize()

    def run_steps(n):
        for i in range(n):
            graphs[i % len(graphs)][0].replay()

    run_steps(args.warmup)
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    sampler = ClockSampler(local_rank)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    run_steps(args.steps)
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1)
    if world > 1:
        t = torch.tensor([ms], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    tok_s = world * args.steps / (ms * 1e-3)

    # ---- end to end: pinned host input -> device -> layer -> pinned host output, every step -----
    xh = [xs[i].cpu().pin_memory() for i in range(n_x)]
    oh = torch.empty(1, 1, D, dtype=torch.float16).pin_memory()

    def e2e_steps(n):
        for i in range(n):
            x = xh[i % n_x].to(dev, non_blocking=True)
            o, _ = blocks[i % L](x)
            oh.copy_(o, non_blocking=True)
            torch.cuda.current_stream().synchronize()

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
    clocks = sampler.stop()

    # ---- roofline of the dominant kernel: fused gate/up GEMV (2/3 of the bytes of a step) -----
    routed = []
    for li, xi in pairs:
        _, _, idx = blocks[li]._decode(xs[xi].view(1, D), 0)
        routed.append(idx[0].clone())
    torch.cuda.synchronize()
    up_bytes = []
    for (li, xi), idx in zip(pairs, routed):
        bits = [blocks[li]._nbits_host[e] for e in idx.tolist()]
        up_bytes.append(sum(2 * FFN * D * (b + 0.25) / 8 for b in bits) + 2 * D + 2 * 2 * A * FFN)

    def up_once(i):
        li, xi = pairs[i % len(pairs)]
        b = blocks[li]
        fused_dequant_up_proj(xs[xi].view(1, D), routed[i % len(pairs)], b.w1_wq, b.w3_wq, b.w1_scales, b.w1_zeros,
                              b.w3_scales, b.w3_zeros, b.w1_nbits, b.w1_wq_strides, G)

    # The launches of one graph replay run back to back on the device, so the interval between
    # the two events holds kernel time only (an eager Python call per launch would not).
    n_up = len(pairs)
    with torch.cuda.stream(side):
        for i in range(n_up):
            up_once(i)
        torch.cuda.synchronize()
        up_graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(up_graph, stream=side):
            for i in range(n_up):
                up_once(i)
    torch.cuda.synchronize()
    reps = max(3, min(args.steps, 200) // n_up)
    for _ in range(3):
        up_graph.replay()
    torch.cuda.synchronize()
    u0, u1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    u0.record()
    for _ in range(reps):
        up_graph.replay()
    u1.record()
    torch.cuda.synchronize()
    up_avg_s = u0.elapsed_time(u1) * 1e-3 / (reps * n_up)
    up_alg = sum(up_bytes[i] for i in range(n_up)) / n_up
    peak, peak_kind = peaks()
    achieved = up_alg / up_avg_s / 1e9

    if rank == 0:
        threads = torch.get_num_threads()
        per_token_s, note, _ = cpu_reference_sample(args.cpu_sample_cols,
                                                    f"torch threads={threads}, os.cpu_count={os.cpu_count()}")
        step_bytes = sum(up_bytes) / len(up_bytes) * 1.5
        line = {
            "metric": METRIC, "value": tok_s, "unit": "tokens/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "f16", "data": "synthetic",
            "config": {"workload": WORKLOAD, "hidden": D, "ffn": FFN, "experts": E, "top_k": A, "group": G,
                       "layers_cycled": L, "parallelism": f"replicas x{world}",
                       "l2": f"inputs larger than L2: {L} layers x ~100 MB touched per step, cycled",
                       "launch": "CUDA graph replay per step (device-resident arm); eager public API (e2e arm)",
                       "approx_bytes_per_step": step_bytes},
            "e2e": {"value": e2e_tok_s, "unit": "tokens/s", "h2d_bytes_per_step": 2 * D, "d2h_bytes_per_step": 2 * D},
            "gpu_launches": 3 * args.steps,
            "clocks": clocks,
            "roofline": {"bound": "hbm", "kernel": "gemv_stream_kernel (fused gate/up projection)",
                         "achieved": achieved, "peak": peak, "peak_kind": peak_kind, "unit": "GB/s",
                         "frac": achieved / peak, "traffic": up_alg * UP_KERNEL_TRAFFIC_RATIO,
                         "algorithmic_bytes_per_launch": up_alg, "avg_launch_us": up_avg_s * 1e6,
                         "layer_frac": step_bytes / (ms / args.steps * 1e-3) / 1e9 / peak},
            "cpu_baseline": {"value": 1.0 / per_token_s, "unit": "tokens/s", "cores": threads, "kind": "port",
                             "sample": note},
        }
        print(json.dumps(line))
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
