"""CPU, world_size 2 over gloo: the expert-parallel dispatch / combine bookkeeping (split sizes,
arrival order, reverse exchange) with stand-in sort and expert functions."""
import os
import socket

import torch
import torch.distributed as dist
import torch.multiprocessing as mp


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _torch_sort(ids, num_experts):
    flat = ids.reshape(-1).long()
    order = torch.argsort(flat, stable=True)
    inv = torch.empty_like(order)
    inv[order] = torch.arange(order.numel())
    offsets = torch.zeros(num_experts + 1, dtype=torch.int64)
    offsets[1:] = torch.cumsum(torch.bincount(flat, minlength=num_experts), 0)
    return order.to(torch.int32), inv.to(torch.int32), offsets.to(torch.int32)


def _worker(rank, world, port, E, T, H, k, empty_rank):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from fp8_inference_toolkit_b200 import moe_ep

    g = torch.Generator().manual_seed(100 + rank)
    x = torch.randn(T, H, generator=g)
    ids = torch.randint(0, E, (T, k), generator=g, dtype=torch.int32)
    if empty_rank is not None:  # nobody routes to rank `empty_rank`'s experts
        e_loc = E // world
        ids = ids % e_loc + (1 - empty_rank) * e_loc
    w = torch.rand(T, k, generator=g)
    e_loc = E // world

    def expert_fn(rows, ids_local, n_loc):
        assert n_loc == e_loc and rows.shape[0] == ids_local.numel()
        return rows * (1.0 + rank * e_loc + ids_local.float()).unsqueeze(1)

    def combine_fn(y_back, inv, wts, T_, k_):
        return (y_back[inv.long()].view(T_, k_, -1) * wts.unsqueeze(2)).sum(1)

    out = moe_ep.moe_layer_ep(x, ids, w, None, E, sort_fn=_torch_sort, expert_fn=expert_fn, combine_fn=combine_fn)
    ref = (x.unsqueeze(1) * (1.0 + ids.float()).unsqueeze(2) * w.unsqueeze(2)).sum(1)
    assert torch.allclose(out, ref, rtol=1e-5, atol=1e-5), (out - ref).abs().max()
    dist.barrier()
    dist.destroy_process_group()


def _worker_fixed(rank, world, port, E, T, H, k, cap, expect_overflow):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from fp8_inference_toolkit_b200 import moe_ep

    g = torch.Generator().manual_seed(200 + rank)
    x = torch.randn(T, H, generator=g)
    ids = torch.randint(0, E, (T, k), generator=g, dtype=torch.int32)
    ids[0, 0] = -1          # a padded pair: left out of the sort, contributes nothing
    w = torch.rand(T, k, generator=g)
    e_loc = E // world

    def sort_with_left_out(i, n):
        flat = i.reshape(-1).long()
        keep = torch.nonzero((flat >= 0) & (flat < n)).flatten()
        order = keep[torch.argsort(flat[keep], stable=True)]
        sp = torch.full((flat.numel(),), -1, dtype=torch.int32)
        sp[:order.numel()] = order.to(torch.int32)
        inv = torch.full((flat.numel(),), -1, dtype=torch.int32)
        inv[order] = torch.arange(order.numel(), dtype=torch.int32)
        off = torch.zeros(n + 1, dtype=torch.int64)
        off[1:] = torch.cumsum(torch.bincount(flat[keep], minlength=n), 0)
        return sp, inv, off.to(torch.int32)

    def expert_fn(rows_sorted, off_loc):
        out = torch.empty_like(rows_sorted)
        for e in range(e_loc):
            a, b = int(off_loc[e]), int(off_loc[e + 1])
            out[a:b] = rows_sorted[a:b] * (1.0 + rank * e_loc + e)
        return out

    def combine_fn(ret, ret_row, wts, T_, k_):
        rr = ret_row.long().view(T_, k_)
        rows = ret[rr.clamp(min=0)] * (rr >= 0).unsqueeze(2)
        return (rows * wts.unsqueeze(2)).sum(1)

    out, overflow = moe_ep.moe_layer_ep_fixed(x, ids, w, E, cap, sort_with_left_out, expert_fn, combine_fn)
    valid = ((ids >= 0) & (ids < E)).float()
    ref = (x.unsqueeze(1) * (1.0 + ids.float()).unsqueeze(2) * (w * valid).unsqueeze(2)).sum(1)
    assert overflow == expect_overflow
    if not overflow:
        assert torch.allclose(out, ref, rtol=1e-5, atol=1e-5), (out - ref).abs().max()
    else:
        # the caller's duty on overflow: redo the step with exact split sizes -- nothing is lost
        def expert_rows(rows, ids_local, n_loc):
            return rows * (1.0 + rank * e_loc + ids_local.float()).unsqueeze(1)

        def combine_exact(y_back, inv, wts, T_, k_):
            ii = inv.long().view(T_, k_)
            return (y_back[ii.clamp(min=0)] * (ii >= 0).unsqueeze(2) * wts.unsqueeze(2)).sum(1)

        def sort_exact(i, n):
            sp, inv, off = sort_with_left_out(i, n)
            return sp[:int(off[-1])], inv, off

        # the exact path sends only the pairs that were kept
        ids2 = ids.clone()
        out2 = moe_ep.moe_layer_ep(x, ids2.clamp(min=0), w * valid, None, E, sort_fn=_torch_sort, expert_fn=expert_rows,
                                   combine_fn=lambda yb, inv, wts, T_, k_: (yb[inv.long()].view(T_, k_, -1) * wts.unsqueeze(2)).sum(1))
        ref2 = (x.unsqueeze(1) * (1.0 + ids2.clamp(min=0).float()).unsqueeze(2) * (w * valid).unsqueeze(2)).sum(1)
        assert torch.allclose(out2, ref2, rtol=1e-5, atol=1e-5)
    dist.barrier()
    dist.destroy_process_group()


def test_fixed_capacity_protocol_two_ranks():
    from fp8_inference_toolkit_b200 import moe_ep

    E, T, H, k = 8, 37, 16, 3
    cap = moe_ep.ep_capacity(T * k, 2)
    assert cap % 8 == 0 and cap >= T * k // 2
    mp.spawn(_worker_fixed, args=(2, _free_port(), E, T, H, k, cap, False), nprocs=2, join=True)


def test_fixed_capacity_overflow_is_flagged_and_redone():
    mp.spawn(_worker_fixed, args=(2, _free_port(), 8, 37, 16, 3, 8, True), nprocs=2, join=True)


def test_plan_and_unpack_reference_roundtrip():
    """Single process: the headers a rank writes let the receiver place every row; positions are a permutation."""
    from fp8_inference_toolkit_b200 import moe_ep

    world, e_loc, cap = 4, 3, 16
    E = world * e_loc
    g = torch.Generator().manual_seed(0)
    plans = []
    for s in range(world):
        ids = torch.randint(0, E, (40,), generator=g, dtype=torch.int32)
        sp, inv, off = _torch_sort(ids, E)
        plans.append(moe_ep.plan_reference(off, sp, world, cap))
    for d in range(world):
        hdrs = torch.stack([plans[s][0][d] for s in range(world)])
        off_loc, pos_of, R = moe_ep.unpack_reference(hdrs, cap)
        got = pos_of[pos_of >= 0]
        assert sorted(got.tolist()) == list(range(R)) and int(off_loc[-1]) == R
        assert R == sum(int(plans[s][0][d, 0]) for s in range(world))


def _run(empty_rank):
    mp.spawn(_worker, args=(2, _free_port(), 8, 37, 16, 3, empty_rank), nprocs=2, join=True)


def test_ep_dispatch_combine_two_ranks():
    _run(None)


def test_ep_rank_without_rows():
    _run(0)
