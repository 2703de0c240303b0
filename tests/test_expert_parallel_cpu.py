"""Host logic of the expert-parallel prefill on CPU ranks (gloo, world size 2): the dispatch
plan, the all-to-all exchange and the ordered combine reproduce the single-process layer."""
import os

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from gemq_b200.inference.expert_parallel import combine_in_expert_order, dispatch_plan, expert_parallel_forward

E, A, D = 8, 2, 16


def toy_expert(x, e_global):
    """Stand-in for an expert FFN in these host-logic tests: a different map per expert."""
    return torch.tanh(x * (0.5 + 0.25 * e_global)) + 0.01 * e_global


def single_process(x, w, sel):
    T = x.shape[0]
    contrib = torch.empty(T, A, D, dtype=x.dtype)
    for t in range(T):
        for a in range(A):
            contrib[t, a] = (toy_expert(x[t].float(), int(sel[t, a])) * float(w[t, a])).to(x.dtype)
    return combine_in_expert_order(contrib, sel)


def make_inputs(seed, T):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(T, D, generator=g).half()
    sel = torch.stack([torch.randperm(E, generator=g)[:A] for _ in range(T)])
    w = torch.softmax(torch.randn(T, A, generator=g), -1).half()
    return x, w, sel


def test_dispatch_plan_groups_by_rank():
    _, _, sel = make_inputs(0, 37)
    order, counts, es = dispatch_plan(sel, E, 4)
    assert counts.sum() == 37 * A and torch.all(es[1:] >= es[:-1])
    dest = es // 2
    assert torch.equal(torch.bincount(dest, minlength=4), counts)
    assert sorted(order.tolist()) == list(range(37 * A))


def _worker(rank, world, port, results):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    per_rank = E // world
    T = 11 + 3 * rank  # ragged token counts per rank
    x, w, sel = make_inputs(100 + rank, T)

    def local_ffn(rows, local_e, wts):
        out = torch.empty_like(rows)
        for i in range(rows.shape[0]):
            e_global = rank * per_rank + int(local_e[i])
            out[i] = (toy_expert(rows[i].float(), e_global) * float(wts[i])).to(rows.dtype)
        return out

    y = expert_parallel_forward(x, w, sel, E, local_ffn)
    ref = single_process(x, w, sel)
    results[rank] = bool(torch.equal(y, ref))
    dist.barrier()
    dist.destroy_process_group()


def test_expert_parallel_matches_single_process_gloo():
    world = 2
    mgr = mp.Manager()
    results = mgr.dict()
    port = 29500 + (os.getpid() % 2000)
    mp.spawn(_worker, args=(world, port, results), nprocs=world, join=True)
    assert dict(results) == {0: True, 1: True}


def test_rank_with_no_tokens_for_some_experts():
    """A rank may receive zero rows: the plan and the combine still hold."""
    x, w, _ = make_inputs(3, 5)
    sel = torch.tensor([[0, 1]] * 5)  # everything goes to rank 0 of 4
    _, counts, _ = dispatch_plan(sel, E, 4)
    assert counts.tolist() == [10, 0, 0, 0]
    contrib = torch.ones(5, A, D).half()
    assert torch.equal(combine_in_expert_order(contrib, sel), torch.full((5, D), 2.0).half())
