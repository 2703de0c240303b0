"""Expert-parallel prefill: experts sharded over ranks, tokens exchanged with all-to-all.

The reference has no multi-GPU path; this module adds the sharding the quantised MoE layer
admits naturally: experts are independent FFNs, tokens are independent rows.  Rank ``r`` of
``P`` holds the packed weights of experts ``[r*E/P, (r+1)*E/P)`` (all routers are replicated)
and ``T/P`` of the tokens.  Per layer:

1. route the local tokens (device side);
2. sort the (token, slot) pairs by destination rank and expert, exchange the per-rank row
   counts, then the rows with their local expert id and routing weight
   (``all_to_all_single`` with variable splits -- the one host read of the step is these counts);
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


def dispatch_plan(sel: Tensor, n_experts: int, world: int) -> Tuple[Tensor, Tensor, Tensor]:
    """``sel [T, A]`` expert ids -> (order, send_counts, experts_sorted).

    ``order`` lists the flat (token * A + slot) pairs sorted by expert id (ties by pair index,
    so the plan is deterministic); contiguous expert ranges belong to one rank, hence the pairs
    are also grouped by destination rank.  ``send_counts [world]`` = pairs per destination.
    """
    assert n_experts % world == 0, "experts must divide evenly over the ranks"
    flat = sel.reshape(-1)
    experts_sorted, order = torch.sort(flat, stable=True)
    per_rank = n_experts // world
    send_counts = torch.bincount(torch.div(flat, per_rank, rounding_mode="floor"), minlength=world)
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


def expert_parallel_forward(x: Tensor, weights: Tensor, sel: Tensor, n_experts: int,
                            local_ffn: Callable[[Tensor, Tensor, Tensor], Tensor], group=None) -> Tensor:
    """One expert-parallel MoE layer on this rank's tokens.

    x [T, D], weights [T, A] (activation dtype), sel [T, A] int64 global expert ids.
    Returns [T, D].  Collective: every rank of ``group`` must call it.
    """
    world = dist.get_world_size(group)
    rank = dist.get_rank(group)
    T, D = x.shape
    A = sel.shape[1]
    per_rank = n_experts // world
    order, send_counts, experts_sorted = dispatch_plan(sel, n_experts, world)

    # 1. counts
    recv_counts = torch.empty_like(send_counts)
    dist.all_to_all_single(recv_counts, send_counts, group=group)
    send_list = send_counts.tolist()          # the host read of the step
    recv_list = recv_counts.tolist()
    n_recv = sum(recv_list)

    # 2. rows, local expert ids, routing weights
    tok = torch.div(order, A, rounding_mode="floor")
    send_x = x.index_select(0, tok).contiguous()
    send_e = (experts_sorted % per_rank).contiguous()
    send_w = weights.reshape(-1).index_select(0, order).contiguous()
    recv_x = x.new_empty((n_recv, D))
    recv_e = send_e.new_empty((n_recv,))
    recv_w = send_w.new_empty((n_recv,))
    dist.all_to_all_single(recv_x, send_x, recv_list, send_list, group=group)
    dist.all_to_all_single(recv_e, send_e, recv_list, send_list, group=group)
    dist.all_to_all_single(recv_w, send_w, recv_list, send_list, group=group)

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

    def __init__(self, local_block, gate_weight: Tensor, n_experts: int, top_k: int, group=None):
        self.local = local_block
        self.gate_weight = gate_weight
        self.n_experts, self.top_k, self.group = n_experts, top_k, group

    def _local_ffn(self, rows: Tensor, local_e: Tensor, wts: Tensor) -> Tensor:
        out, _, _, _ = self.local._prefill(rows, 1, True, routing=(wts.view(-1, 1), local_e.view(-1, 1)))
        return out

    def forward(self, x: Tensor) -> Tensor:
        """x [T_local, D] fp16/bf16 on this rank's GPU -> [T_local, D]."""
        from .moe_block import ROUTE_FP32_SOFTMAX, route_tokens
        w, sel, _ = route_tokens(x, self.gate_weight, self.top_k, ROUTE_FP32_SOFTMAX, True)
        return expert_parallel_forward(x, w, sel, self.n_experts, self._local_ffn, self.group)

    def forward_routed(self, x: Tensor, w: Tensor, sel: Tensor) -> Tensor:
        return expert_parallel_forward(x, w, sel, self.n_experts, self._local_ffn, self.group)
