"""Expert-parallel prefill: experts sharded over ranks, tokens exchanged with all-to-all.

The reference has no multi-GPU path; this module adds the sharding the quantised MoE layer
admits naturally: experts are independent FFNs, tokens are independent rows.  Every rank holds
the packed weights of its experts (contiguous ranges, or a placement that evens out the routed
rows per rank), all routers are replicated, and rank ``r`` of ``P`` owns ``T/P`` of the tokens.
Per layer:

1. route the local tokens (device side);
2. sort the (token, slot) pairs by destination rank and expert, exchange the per-rank row
   counts, then the rows, each carrying its local expert id and routing weight
   (one ``all_to_all_single`` with variable splits -- the one host read of the step is the counts);
3. run the local experts on the received rows (expert-sorted grouped GEMM);
4. send the weighted outputs back with the reverse ``all_to_all_single``;
5. add each token's contributions in increasing expert id, rounding to the activation dtype
   after every addition (``index_add_`` order of gemq/inference/moe_block.py:191-195).

An expert that alone draws more rows than a rank's fair share can be held by several ranks
(``replicated_placement``); every sender then splits its rows of that expert between the
replicas in fixed proportions.  A row's result does not depend on which replica computes it.

``local_ffn(x_rows, local_expert_ids, weights) -> y_rows`` is the rank's compute; the collective
plumbing is plain ``torch.distributed`` and runs unchanged on NCCL (GPU) and gloo (CPU tests).
"""
from __future__ import annotations

from typing import Callable, Tuple

import torch
import torch.distributed as dist
from torch import Tensor


def contiguous_placement(n_experts: int, world: int) -> Tensor:
    """Expert -> rank with contiguous equal ranges: rank r holds experts [r*E/P, (r+1)*E/P)."""
    assert n_experts % world == 0, "experts must divide evenly over the ranks"
    return torch.arange(n_experts) // (n_experts // world)


def balanced_placement(routed_rows, world: int) -> Tensor:
    """Expert -> rank that evens out the routed rows per rank (the grouped GEMM is tensor bound,
    so a row costs the same at every bit width): experts in decreasing row count, each to the rank
    with the fewest rows so far (ties to the lower rank; deterministic, every rank computes the
    same table from the same statistics).  A rank may hold more experts than another."""
    rows = [int(r) for r in routed_rows]
    load = [0] * world
    held = [0] * world
    place = [0] * len(rows)
    for e in sorted(range(len(rows)), key=lambda i: (-rows[i], i)):
        r = min(range(world), key=lambda k: (load[k], held[k], k))
        place[e] = r
        load[r] += rows[e]
        held[r] += 1
    return torch.tensor(place, dtype=torch.int64)


def local_ids(expert_to_rank: Tensor) -> Tensor:
    """Position of every expert among the experts of its rank (increasing expert id)."""
    loc = torch.zeros_like(expert_to_rank)
    for r in expert_to_rank.unique().tolist():
        mine = torch.nonzero(expert_to_rank == r).view(-1)
        loc[mine] = torch.arange(mine.numel())
    return loc


class Placement:
    """Which ranks hold which experts.  An expert may live on several ranks; replica ``j`` of
    expert ``e`` then takes the rows whose position among a sender's rows of that expert, as a
    fraction, lies in ``[upper[e, j-1], upper[e, j])``.  The weights are a few tens of MB per
    expert, so a copy of the one expert that draws 40 % of the rows costs little memory and lifts
    the ceiling that expert puts on the speed-up.  ``instances`` = [(expert, rank, share), ...]
    with the shares of an expert summing to 1."""

    def __init__(self, instances, n_experts: int, world: int):
        self.instances = [(int(e), int(r), float(s)) for e, r, s in instances]
        self.n_experts, self.world = n_experts, world
        self.experts_of = [sorted({e for e, r, _ in self.instances if r == k}) for k in range(world)]
        per_expert = [[(r, s) for e2, r, s in self.instances if e2 == e] for e in range(n_experts)]
        assert all(per_expert), "every expert needs a rank"
        R = self.max_replicas = max(len(v) for v in per_expert)
        rank = torch.zeros((n_experts, R), dtype=torch.int64)
        local = torch.zeros((n_experts, R), dtype=torch.int64)
        upper = torch.full((n_experts, R), 2.0)
        for e, reps in enumerate(per_expert):
            acc = 0.0
            for j in range(R):
                r, sh = reps[min(j, len(reps) - 1)]
                rank[e, j], local[e, j] = r, self.experts_of[r].index(e)
                if j < len(reps) - 1:
                    acc += sh
                    upper[e, j] = acc
        self.rank, self.local, self.upper = rank, local, upper
        self._dev = {}

    @staticmethod
    def from_expert_to_rank(expert_to_rank: Tensor, world: int) -> "Placement":
        return Placement([(e, int(r), 1.0) for e, r in enumerate(expert_to_rank.tolist())], expert_to_rank.numel(), world)

    def on(self, device):
        key = str(device)
        if key not in self._dev:
            self._dev[key] = (self.rank.to(device), self.local.to(device), self.upper.to(device))
        return self._dev[key]

    def rows_per_rank(self, routed_rows):
        load = [0.0] * self.world
        for e, r, sh in self.instances:
            load[r] += sh * float(routed_rows[e])
        return load


def replicated_placement(routed_rows, world: int, min_rows: int = 256) -> Placement:
    """Placement that evens out the routed rows per rank, splitting an expert over several ranks
    where it alone exceeds a rank's fair share: experts in decreasing row count, each to the rank
    with the fewest rows so far; when the expert does not fit under the fair share there, the rank
    takes what fits and the rest moves on to the next rank (pieces below ``min_rows`` rows -- a
    GEMM tile -- are not split off).  Deterministic: every rank computes the same table."""
    rows = [int(r) for r in routed_rows]
    E, total = len(rows), float(sum(rows))
    target = total / world
    load = [0.0] * world
    held = [0] * world
    inst = []
    for e in sorted(range(E), key=lambda i: (-rows[i], i)):
        left, tried = float(rows[e]), set()
        while True:
            free = [k for k in range(world) if k not in tried]
            r = min(free, key=lambda k: (load[k], held[k], k))
            cap = target - load[r]
            if left <= cap or len(free) == 1 or cap < min_rows or left - cap < min_rows or rows[e] == 0:
                inst.append((e, r, left / rows[e] if rows[e] else 1.0))
                load[r] += left
                held[r] += 1
                break
            inst.append((e, r, cap / rows[e]))
            load[r] += cap
            held[r] += 1
            left -= cap
            tried.add(r)
    return Placement(inst, E, world)


def _as_placement(place, n_experts: int, world: int) -> Placement:
    if isinstance(place, Placement):
        return place
    if place is None:
        place = contiguous_placement(n_experts, world)
    return Placement.from_expert_to_rank(place, world)


def placed_plan(sel: Tensor, place: Placement) -> Tuple[Tensor, Tensor, Tensor]:
    """``sel [T, A]`` expert ids -> (order, send_counts, local_ids_sorted): the flat
    (token * A + slot) pairs sorted by destination rank, then expert id (ties by pair index), the
    pairs per destination, and each sorted pair's expert position on its destination."""
    E = place.n_experts
    rank_d, local_d, upper_d = place.on(sel.device)
    flat = sel.reshape(-1)
    if place.max_replicas == 1:
        dest, loc = rank_d[flat, 0], local_d[flat, 0]
    else:
        onehot = torch.nn.functional.one_hot(flat, E)
        ordinal = (onehot.cumsum(0) * onehot).sum(1) - 1          # position among the rows of the same expert
        count = onehot.sum(0)[flat]
        frac = (ordinal.to(torch.float32) + 0.5) / count.to(torch.float32)
        rep = (frac.unsqueeze(1) >= upper_d[flat]).sum(1, keepdim=True)
        dest, loc = rank_d[flat].gather(1, rep).squeeze(1), local_d[flat].gather(1, rep).squeeze(1)
    _, order = torch.sort(dest * E + flat, stable=True)
    return order, torch.bincount(dest, minlength=place.world), loc[order]


def dispatch_plan(sel: Tensor, n_experts: int, world: int, expert_to_rank: Tensor = None) -> Tuple[Tensor, Tensor, Tensor]:
    """``sel [T, A]`` expert ids -> (order, send_counts, experts_sorted).

    ``order`` lists the flat (token * A + slot) pairs sorted by destination rank, then by expert id
    (ties by pair index, so the plan is deterministic).  ``send_counts [world]`` = pairs per
    destination.  Without ``expert_to_rank`` the placement is contiguous.
    """
    order, send_counts, _ = placed_plan(sel, _as_placement(expert_to_rank, n_experts, world))
    return order, send_counts, sel.reshape(-1)[order]


def combine_in_expert_order(contrib: Tensor, sel: Tensor) -> Tensor:
    """``contrib [T, A, D]`` (already weighted, activation dtype), ``sel [T, A]`` ->
    ``[T, D]``: contributions added in increasing expert id with a rounding per addition."""
    T, A, D = contrib.shape
    by_expert = torch.argsort(sel, dim=1, stable=True)
    ordered = torch.gather(contrib, 1, by_expert.unsqueeze(-1).expand(T, A, D))
    acc = torch.zeros((T, D), dtype=contrib.dtype, device=contrib.device)
    for a in range(A):
        acc = acc + ordered[:, a]
    return acc


_META = 8  # halves appended to a row: local expert id (int32 = 2 halves), routing weight, padding to 16 bytes


def _exchange_counts(send_counts: Tensor, group):
    """All-to-all of the per-destination row counts; returns a function that yields
    (send_list, recv_list) -- the one host read of the step.  On a GPU the read-back is issued
    now and awaited when the function is called, so that work enqueued in between hides it."""
    recv_counts = torch.empty_like(send_counts)
    dist.all_to_all_single(recv_counts, send_counts, group=group)
    both = torch.stack([send_counts, recv_counts])
    if not both.is_cuda:
        return lambda: both.tolist()
    host = torch.empty(both.shape, dtype=both.dtype, pin_memory=True)
    host.copy_(both, non_blocking=True)
    done = torch.cuda.Event()
    done.record()

    def read():
        done.synchronize()
        return host.tolist()
    return read


_plan_scratch: dict = {}


def _dev_key(device) -> int:
    device = torch.device(device)
    return device.index if device.index is not None else torch.cuda.current_device()


def _cuda_tables(place: Placement, device):
    key = ("i32", str(device))
    if key not in place._dev:
        rank, local, upper = place.on(device)
        place._dev[key] = (rank.to(torch.int32).contiguous(), local.to(torch.int32).contiguous(), upper.contiguous())
    return place._dev[key]


def placed_plan_cuda(sel: Tensor, place: Placement):
    """``placed_plan`` in one launch (``gemq_ep_plan``); also returns the inverse permutation."""
    from .. import _capi
    from ..kernels._runtime import stream_ptr
    dev = sel.device
    n = sel.numel()
    rank_t, local_t, upper_t = _cuda_tables(place, dev)
    flat = sel.reshape(-1).contiguous()
    order = torch.empty(n, dtype=torch.int64, device=dev)
    where = torch.empty(n, dtype=torch.int64, device=dev)
    loc = torch.empty(n, dtype=torch.int32, device=dev)
    counts = torch.empty(place.world, dtype=torch.int64, device=dev)
    need = _capi.lib.gemq_ep_plan_scratch_bytes(n)
    scratch = _plan_scratch.get(_dev_key(dev))
    if scratch is None or scratch.numel() < need:
        scratch = _plan_scratch[_dev_key(dev)] = torch.zeros(max(need, 1 << 16), dtype=torch.uint8, device=dev)
    _capi.check("gemq_ep_plan", _capi.lib.gemq_ep_plan(
        flat.data_ptr(), n, place.n_experts, place.world, place.max_replicas, rank_t.data_ptr(), local_t.data_ptr(),
        upper_t.data_ptr(), order.data_ptr(), loc.data_ptr(), where.data_ptr(), counts.data_ptr(), scratch.data_ptr(),
        scratch.numel(), stream_ptr(dev)))
    return order, counts, loc, where


def plan_error_code(device) -> int:
    """Code left by ``gemq_ep_plan`` on ``device`` (0: every expert id was in range); clears it."""
    scratch = _plan_scratch.get(_dev_key(device))
    if scratch is None:
        return 0
    word = scratch[:4].view(torch.int32)
    code = int(word.item())
    word.zero_()
    return code


def expert_parallel_forward(x: Tensor, weights: Tensor, sel: Tensor, n_experts: int,
                            local_ffn: Callable[[Tensor, Tensor, Tensor], Tensor], group=None,
                            expert_to_rank=None) -> Tensor:
    """One expert-parallel MoE layer on this rank's tokens.

    x [T, D], weights [T, A] (activation dtype), sel [T, A] int64 global expert ids;
    ``expert_to_rank``: None (contiguous ranges), an expert -> rank tensor, or a ``Placement``.
    Returns [T, D].  Collective: every rank of ``group`` must call it.  Three collectives: the
    row counts, the rows out (each row carries its local expert id and routing weight in eight
    extra elements, so one all-to-all moves everything), the rows back.  On CUDA tensors the plan,
    the payload, its unpacking and the combine are one kernel each (``csrc/expert_parallel.cu``);
    the tensor-operation forms below them serve CPU tensors (gloo).
    """
    world = dist.get_world_size(group)
    T, D = x.shape
    A = sel.shape[1]
    place = _as_placement(expert_to_rank, n_experts, world)
    cuda = x.is_cuda and T > 0
    if cuda:
        from .. import _capi
        from ..kernels._runtime import stream_ptr
        sp = stream_ptr(x.device)
        order, send_counts, loc_sorted, where = placed_plan_cuda(sel, place)
    else:
        order, send_counts, loc_sorted = placed_plan(sel, place)

    # 1. counts (read back while the payload is being built)
    read_counts = _exchange_counts(send_counts, group)

    # 2. rows with their local expert id and routing weight, one payload
    send = x.new_empty((T * A, D + _META))
    if cuda:
        wflat = weights.reshape(-1).contiguous()
        _capi.check("gemq_ep_pack_rows", _capi.lib.gemq_ep_pack_rows(
            x.contiguous().data_ptr(), order.data_ptr(), loc_sorted.data_ptr(), wflat.data_ptr(), T * A, A, D,
            send.data_ptr(), sp))
    else:
        tok = torch.div(order, A, rounding_mode="floor")
        send[:, :D] = x.index_select(0, tok)
        send[:, D:D + 2] = loc_sorted.to(torch.int32).view(-1, 1).view(x.dtype)
        send[:, D + 2] = weights.reshape(-1).index_select(0, order)
        send[:, D + 3:] = 0
    send_list, recv_list = read_counts()
    n_recv = sum(recv_list)
    recv = x.new_empty((n_recv, D + _META))
    dist.all_to_all_single(recv, send, recv_list, send_list, group=group)
    if cuda and n_recv:
        recv_x = x.new_empty((n_recv, D))
        recv_e = torch.empty(n_recv, dtype=torch.int64, device=x.device)
        recv_w = x.new_empty(n_recv)
        _capi.check("gemq_ep_unpack_rows", _capi.lib.gemq_ep_unpack_rows(
            recv.data_ptr(), n_recv, D, recv_x.data_ptr(), recv_e.data_ptr(), recv_w.data_ptr(), sp))
    else:
        recv_x = recv[:, :D].contiguous()
        recv_e = recv[:, D:D + 2].contiguous().view(torch.int32).view(-1).to(torch.int64)
        recv_w = recv[:, D + 2].contiguous()

    # 3. local experts
    y = local_ffn(recv_x, recv_e, recv_w) if n_recv else recv_x
    assert y.shape == recv_x.shape and y.dtype == x.dtype

    # 4. outputs back to the token owners (same row order as they were sent)
    back = x.new_empty((T * A, D))
    dist.all_to_all_single(back, y.contiguous(), send_list, recv_list, group=group)

    # 5. combine: a token's rows in increasing expert id, a rounding per addition (the first
    #    addition, to zero, is exact)
    if cuda:
        out = x.new_empty((T, D))
        _capi.check("gemq_ep_combine", _capi.lib.gemq_ep_combine(
            back.data_ptr(), where.data_ptr(), sel.contiguous().data_ptr(), T, A, D, int(x.dtype == torch.bfloat16),
            out.data_ptr(), sp))
        return out
    where = torch.empty_like(order)
    where[order] = torch.arange(T * A, device=order.device)
    rows_of = where.view(T, A).gather(1, torch.argsort(sel, dim=1, stable=True))
    acc = back.index_select(0, rows_of[:, 0])
    for a in range(1, A):
        acc = acc + back.index_select(0, rows_of[:, a])
    return acc


class ExpertParallelMixtralMoE:
    """Mixtral-style quantised MoE layer with its experts sharded over the ranks of ``group``.

    ``local_block`` is a ``QuantFusedMixtralMoEBlock`` built from this rank's experts only, with
    ``num_experts_per_tok = 1`` (every received row visits exactly one local expert);
    ``gate_weight [E, D]`` is the full, replicated router.
    """

    def __init__(self, local_block, gate_weight: Tensor, n_experts: int, top_k: int, group=None,
                 expert_to_rank=None):
        self.local = local_block
        self.gate_weight = gate_weight
        self.n_experts, self.top_k, self.group = n_experts, top_k, group
        self.expert_to_rank = expert_to_rank  # None: contiguous ranges; a tensor; or a Placement (replicas allowed)

    def _local_ffn(self, rows: Tensor, local_e: Tensor, wts: Tensor) -> Tensor:
        out, _, _, _ = self.local._prefill(rows, 1, True, routing=(wts.view(-1, 1), local_e.view(-1, 1)))
        return out

    def forward(self, x: Tensor) -> Tensor:
        """x [T_local, D] fp16/bf16 on this rank's GPU -> [T_local, D]."""
        from .moe_block import ROUTE_FP32_SOFTMAX, route_tokens
        w, sel, _ = route_tokens(x, self.gate_weight, self.top_k, ROUTE_FP32_SOFTMAX, True)
        return expert_parallel_forward(x, w, sel, self.n_experts, self._local_ffn, self.group, self.expert_to_rank)

    def forward_routed(self, x: Tensor, w: Tensor, sel: Tensor) -> Tensor:
        return expert_parallel_forward(x, w, sel, self.n_experts, self._local_ffn, self.group, self.expert_to_rank)
