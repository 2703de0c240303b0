"""Host logic of the expert-parallel prefill on CPU ranks (gloo, world size 2): the dispatch
plan, the all-to-all exchange and the ordered combine reproduce the single-process layer."""
import os

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from gemq_b200.inference.expert_parallel import (Placement, balanced_placement, combine_in_expert_order, dispatch_plan,
                                                 expert_parallel_forward, local_ids, placed_plan, replicated_placement)

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


def test_balanced_placement_evens_out_rows():
    rows = [4000, 2500, 700, 400, 300, 200, 60, 32]  # skewed popularity, as Dirichlet(0.5) gives
    place = balanced_placement(rows, 2)
    per_rank = [sum(r for r, p in zip(rows, place.tolist()) if p == k) for k in range(2)]
    assert max(per_rank) / sum(rows) < 0.52  # contiguous halves would put 93 % on rank 0
    assert place.tolist() == balanced_placement(rows, 2).tolist()
    loc = local_ids(place)
    for k in range(2):
        mine = [e for e in range(8) if place[e] == k]
        assert [int(loc[e]) for e in mine] == list(range(len(mine)))
    # eight ranks, eight experts: one expert each, the hottest rank holds the hottest expert
    assert sorted(balanced_placement(rows, 8).tolist()) == list(range(8))


def test_dispatch_plan_with_placement_groups_by_rank():
    _, _, sel = make_inputs(1, 29)
    place = torch.tensor([1, 0, 0, 1, 0, 1, 1, 0])
    order, counts, es = dispatch_plan(sel, E, 2, place)
    dest = place[es]
    assert torch.all(dest[1:] >= dest[:-1]) and torch.equal(torch.bincount(dest, minlength=2), counts)
    assert sorted(order.tolist()) == list(range(29 * A))


def test_replicated_placement_splits_the_hot_expert():
    rows = [631, 37, 99, 707, 1509, 1600, 3414, 195]  # one expert draws 42 % of the rows
    for world in (2, 4, 8):
        place = replicated_placement(rows, world)
        load = place.rows_per_rank(rows)
        assert abs(sum(load) - sum(rows)) < 1e-6
        assert max(load) / sum(rows) < 1.1 / world          # without replicas: 0.42 at four ranks
        for e in range(8):
            assert abs(sum(s for e2, _, s in place.instances if e2 == e) - 1.0) < 1e-9
        assert [list(i) for i in place.instances] == [list(i) for i in replicated_placement(rows, world).instances]
    place = replicated_placement(rows, 4)
    assert sorted(r for e, r, _ in place.instances if e == 6) == [0, 1]
    # a sender's rows of the split expert go to the replicas in the placement's proportions, in order
    sel = torch.tensor([[6, 0]] * 10)
    order, counts, loc = placed_plan(sel, place)
    flat = sel.reshape(-1)[order]
    assert counts.tolist() == [6, 4, 0, 10] and flat.tolist() == [6] * 10 + [0] * 10
    assert order[:10].tolist() == [2 * i for i in range(10)]


def _worker(rank, world, port, results, placement=None):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    if isinstance(placement, list) and isinstance(placement[0], tuple):
        place = Placement(placement, E, world)
        mine = place.experts_of[rank]
    else:
        place = torch.tensor(placement) if placement is not None else torch.arange(E) // (E // world)
        mine = [e for e in range(E) if int(place[e]) == rank]
    T = 11 + 3 * rank  # ragged token counts per rank
    x, w, sel = make_inputs(100 + rank, T)

    def local_ffn(rows, local_e, wts):
        out = torch.empty_like(rows)
        for i in range(rows.shape[0]):
            e_global = mine[int(local_e[i])]
            out[i] = (toy_expert(rows[i].float(), e_global) * float(wts[i])).to(rows.dtype)
        return out

    y = expert_parallel_forward(x, w, sel, E, local_ffn, expert_to_rank=None if placement is None else place)
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


def test_expert_parallel_with_uneven_placement_gloo():
    """Rank 0 holds two experts, rank 1 six: ids travel as positions inside the owner's expert list."""
    world = 2
    mgr = mp.Manager()
    results = mgr.dict()
    port = 31500 + (os.getpid() % 2000)
    mp.spawn(_worker, args=(world, port, results, [1, 0, 1, 1, 0, 1, 1, 1]), nprocs=world, join=True)
    assert dict(results) == {0: True, 1: True}


def test_expert_parallel_with_replicated_experts_gloo():
    """Experts 0 and 5 live on both ranks; each sender splits its rows between the replicas."""
    world = 2
    mgr = mp.Manager()
    results = mgr.dict()
    port = 33500 + (os.getpid() % 2000)
    inst = [(0, 0, 0.3), (0, 1, 0.7), (1, 0, 1.0), (2, 1, 1.0), (3, 1, 1.0), (4, 0, 1.0), (5, 1, 0.5), (5, 0, 0.5),
            (6, 0, 1.0), (7, 1, 1.0)]
    mp.spawn(_worker, args=(world, port, results, inst), nprocs=world, join=True)
    assert dict(results) == {0: True, 1: True}


def test_expert_parallel_four_ranks_placement_from_row_counts_gloo():
    """Four ranks, placement computed from the routed-row counts of all ranks' tokens with pieces as
    small as one row: several experts end up on two or more ranks."""
    world = 4
    counts = torch.zeros(E, dtype=torch.int64)
    for r in range(world):
        _, _, sel = make_inputs(100 + r, 11 + 3 * r)
        counts += torch.bincount(sel.reshape(-1), minlength=E)
    # expert 0 made nine times as popular as it is: the counts only steer the placement, any table gives the same result
    place = replicated_placement((counts * torch.tensor([9, 1, 1, 1, 1, 1, 1, 1])).tolist(), world, min_rows=1)
    assert place.max_replicas >= 2
    mgr = mp.Manager()
    results = mgr.dict()
    port = 35500 + (os.getpid() % 2000)
    mp.spawn(_worker, args=(world, port, results, [tuple(i) for i in place.instances]), nprocs=world, join=True)
    assert dict(results) == {0: True, 1: True, 2: True, 3: True}


def test_rank_with_no_tokens_for_some_experts():
    """A rank may receive zero rows: the plan and the combine still hold."""
    x, w, _ = make_inputs(3, 5)
    sel = torch.tensor([[0, 1]] * 5)  # everything goes to rank 0 of 4
    _, counts, _ = dispatch_plan(sel, E, 4)
    assert counts.tolist() == [10, 0, 0, 0]
    contrib = torch.ones(5, A, D).half()
    assert torch.equal(combine_in_expert_order(contrib, sel), torch.full((5, D), 2.0).half())
