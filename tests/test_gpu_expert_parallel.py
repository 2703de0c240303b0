"""Device side of the expert-parallel token exchange (gemq_ep_plan / pack / unpack / combine)
against the tensor-operation forms the CPU ranks use.  Integer and byte work: bit-exact."""
import pytest
import torch

from gemq_b200.inference.expert_parallel import (Placement, combine_in_expert_order, placed_plan, placed_plan_cuda,
                                                 plan_error_code, replicated_placement)

pytestmark = pytest.mark.gpu


def _routing(seed, T, E, A, skew=False):
    g = torch.Generator().manual_seed(seed)
    if skew:
        p = torch.distributions.Dirichlet(torch.full((E,), 0.5)).sample()
        sel = torch.stack([torch.multinomial(p, A, replacement=False, generator=g) for _ in range(T)])
    else:
        sel = torch.stack([torch.randperm(E, generator=g)[:A] for _ in range(T)])
    return sel.cuda()


@pytest.mark.parametrize("T,E,A,world", [(5, 8, 2, 2), (1024, 8, 2, 4), (2048, 8, 2, 8), (700, 64, 6, 8), (3000, 64, 6, 4)])
def test_plan_matches_tensor_form(T, E, A, world):
    sel = _routing(T, T, E, A, skew=True)
    rows = torch.bincount(sel.view(-1).cpu(), minlength=E).tolist()
    for place in (Placement.from_expert_to_rank(torch.arange(E) // (E // world), world),
                  replicated_placement(rows, world, min_rows=max(1, T // 40))):
        want_order, want_counts, want_loc = placed_plan(sel, place)
        order, counts, loc, where = placed_plan_cuda(sel, place)
        torch.cuda.synchronize()
        assert torch.equal(order, want_order) and torch.equal(counts, want_counts)
        assert torch.equal(loc.to(torch.int64), want_loc)
        assert torch.equal(where[order], torch.arange(T * A, device="cuda"))
        assert plan_error_code("cuda") == 0


def test_plan_reports_ids_out_of_range():
    sel = _routing(3, 40, 8, 2)
    sel[7, 1] = 8
    sel[9, 0] = -1
    place = Placement.from_expert_to_rank(torch.arange(8) // 4, 2)
    order, counts, loc, where = placed_plan_cuda(sel, place)
    torch.cuda.synchronize()
    assert int(counts.sum()) == 80 and sorted(order.tolist()) == list(range(80))  # clamped, never used as an index
    assert plan_error_code("cuda") != 0 and plan_error_code("cuda") == 0


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_pack_unpack_and_combine(dtype):
    from gemq_b200 import _capi
    T, E, A, D = 333, 8, 2, 256
    sel = _routing(11, T, E, A)
    g = torch.Generator().manual_seed(5)
    x = torch.randn(T, D, generator=g).to(dtype).cuda()
    w = torch.softmax(torch.randn(T, A, generator=g), -1).to(dtype).cuda()
    place = replicated_placement(torch.bincount(sel.view(-1).cpu(), minlength=E).tolist(), 4, min_rows=16)
    order, counts, loc, where = placed_plan_cuda(sel, place)
    sp = torch.cuda.current_stream().cuda_stream
    n = T * A
    payload = torch.empty(n, D + 8, dtype=dtype, device="cuda")
    assert _capi.lib.gemq_ep_pack_rows(x.data_ptr(), order.data_ptr(), loc.data_ptr(), w.view(-1).data_ptr(), n, A, D,
                                       payload.data_ptr(), sp) == 0
    tok = torch.div(order, A, rounding_mode="floor")
    assert torch.equal(payload[:, :D], x[tok])
    assert torch.equal(payload[:, D:D + 2].contiguous().view(torch.int32).view(-1), loc)
    assert torch.equal(payload[:, D + 2], w.view(-1)[order])
    rows = torch.empty(n, D, dtype=dtype, device="cuda")
    e = torch.empty(n, dtype=torch.int64, device="cuda")
    ww = torch.empty(n, dtype=dtype, device="cuda")
    assert _capi.lib.gemq_ep_unpack_rows(payload.data_ptr(), n, D, rows.data_ptr(), e.data_ptr(), ww.data_ptr(), sp) == 0
    assert torch.equal(rows, x[tok]) and torch.equal(e, loc.to(torch.int64)) and torch.equal(ww, w.view(-1)[order])
    # combine: rows come back in the order they were sent
    back = (torch.randn(n, D, generator=g) * 3).to(dtype).cuda()
    out = torch.empty(T, D, dtype=dtype, device="cuda")
    assert _capi.lib.gemq_ep_combine(back.data_ptr(), where.data_ptr(), sel.data_ptr(), T, A, D, int(dtype == torch.bfloat16),
                                     out.data_ptr(), sp) == 0
    contrib = torch.empty(n, D, dtype=dtype, device="cuda")
    contrib[order] = back
    assert torch.equal(out, combine_in_expert_order(contrib.view(T, A, D), sel))
