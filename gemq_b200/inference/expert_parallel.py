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


def dispatch_plan(sel: Tensor, n_experts: int, world: int, expert_to_rank: Tensor = None) -> Tuple[Tensor, Tensor, Tensor]:
    """``sel [T, A]`` expert ids -> (order, send_counts, experts_sorted).

    ``order`` lists the flat (token * A + slot) pairs sorted by destination rank, then by expert id
    (ties by pair index, so the plan is deterministic).  ``send_counts [world]`` = pairs per
    destination.  Without ``expert_to_rank`` the placement is contiguous.
    """
    if expert_to_rank is None:
        expert_to_rank = contiguous_placement(n_experts, world)
    e2r = expert_to_rank.to(sel.device)
    flat = sel.reshape(-1)
    dest = e2r[flat]
    _, order = torch.sort(dest * n_experts + flat, stable=True)
    experts_sorted = flat[order]
    send_counts = torch.bincount(dest, minlength=world)
    return order, send_counts, experts_sorted


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


def expert_parallel_forward(x: Tensor, weights: Tensor, sel: Tensor, n_experts: int,
                            local_ffn: Callable[[Tensor, Tensor, Tensor], Tensor], group=None,
                            expert_to_rank: Tensor = None) -> Tensor:
    """One expert-parallel MoE layer on this rank's tokens.

    x [T, D], weights [T, A] (activation dtype), sel [T, A] int64 global expert ids.
    Returns [T, D].  Collective: every rank of ``group`` must call it.  Three collectives: the
    row counts, the rows out (each row carries its local expert id and routing weight in eight
    extra elements, so one all-to-all moves everything), the rows back.
    """
    world = dist.get_world_size(group)
    T, D = x.shape
    A = sel.shape[1]
    if expert_to_rank is None:
        expert_to_rank = contiguous_placement(n_experts, world)
    loc = local_ids(expert_to_rank).to(sel.device)
    order, send_counts, experts_sorted = dispatch_plan(sel, n_experts, world, expert_to_rank)

    # 1. counts
    recv_counts = torch.empty_like(send_counts)
    dist.all_to_all_single(recv_counts, send_counts, group=group)
    both = torch.stack([send_counts, recv_counts]).tolist()  # the one host read of the step
    send_list, recv_list = both
    n_recv = sum(recv_list)

    # 2. rows with their local expert id and routing weight, one payload
    tok = torch.div(order, A, rounding_mode="floor")
    send = x.new_empty((T * A, D + _META))
    send[:, :D] = x.index_select(0, tok)
    send[:, D:D + 2] = loc[experts_sorted].to(torch.int32).view(-1, 1).view(x.dtype)
    send[:, D + 2] = weights.reshape(-1).index_select(0, order)
    recv = x.new_empty((n_recv, D + _META))
    dist.all_to_all_single(recv, send, recv_list, send_list, group=group)
    recv_x = recv[:, :D].contiguous()
    recv_e = recv[:, D:D + 2].contiguous().view(torch.int32).view(-1).to(torch.int64)
    recv_w = recv[:, D + 2].contiguous()

    # 3. local experts
    y = local_ffn(recv_x, recv_e, recv_w) if n_recv else recv_x
    assert y.shape == recv_x.shape and y.dtype == x.dtype

    # 4. outputs back to the token owners (same row order as they were sent)
    back = x.new_empty((T * A, D))
    dist.all_to_all_single(back, y.contiguous(), send_list, recv_list, group=group)

    # 5. combine
    contrib = x.new_empty((T * A, D))
    contrib.index_copy_(0, order, back)
    return combine_in_expert_order(contrib.view(T, A, D), sel)


class ExpertParallelMixtralMoE:
    """Mixtral-style quantised MoE layer with its experts sharded over the ranks of ``group``.

    ``local_block`` is a ``QuantFusedMixtralMoEBlock`` built from this rank's experts only, with
    ``num_experts_per_tok = 1`` (every received row visits exactly one local expert);
    ``gate_weight [E, D]`` is the full, replicated router.
    """

    def __init__(self, local_block, gate_weight: Tensor, n_experts: int, top_k: int, group=None,
                 expert_to_rank: Tensor = None):
        self.local = local_block
        self.gate_weight = gate_weight
        self.n_experts, self.top_k, self.group = n_experts, top_k, group
        self.expert_to_rank = expert_to_rank  # None: contiguous ranges

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
