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


def _run(empty_rank):
    mp.spawn(_worker, args=(2, _free_port(), 8, 37, 16, 3, empty_rank), nprocs=2, join=True)


def test_ep_dispatch_combine_two_ranks():
    _run(None)


def test_ep_rank_without_rows():
    _run(0)
