"""CPU, world_size 2 over gloo: the dense linears split by output columns as `bench.py --gpus N` splits them.  Every rank
quantises the whole activation itself, multiplies it with its own rows of the quantised weight (here with the CPU
oracle standing in for the kernels) and keeps its output columns; no collective is part of the product path.  The test
gathers the shards and compares them with the unsplit oracle result bit for bit, and checks the end-to-end variant in
which each rank holds M / world activation rows and an all-gather completes them."""
import os
import socket

import numpy as np
import torch
import torch.distributed as dist
import torch.multiprocessing as mp


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, M, K, N):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from oracle import w4a4_oracle as O

    g = torch.Generator().manual_seed(7)                 # the same tensors on every rank
    x = (torch.randn(M, K, generator=g) * 1.5).to(torch.bfloat16)
    w = (torch.randn(N, K, generator=g) * 0.05).to(torch.bfloat16)
    n_loc, m_loc = N // world, M // world

    # weights: each rank quantises and keeps only its rows (output columns)
    wc, ws = O.quant_grouped(w[rank * n_loc:(rank + 1) * n_loc], 128, role="weight")
    # activations, kernel-only arm: replicated input, quantised on every rank
    xc, xs = O.quant_grouped(x, 128)
    shard = O.linear_grouped(xc, wc, xs, ws)             # [M, n_loc] bf16
    assert shard.shape == (M, n_loc)

    # end-to-end arm: every rank starts with M / world rows; an all-gather rebuilds the activations
    mine = x[rank * m_loc:(rank + 1) * m_loc].contiguous()
    full = torch.empty(M, K, dtype=torch.bfloat16)
    dist.all_gather_into_tensor(full.view(torch.int32), mine.view(torch.int32))   # gloo has no bf16: move the bits
    assert torch.equal(full, x)
    xc2, xs2 = O.quant_grouped(full, 128)
    assert np.array_equal(xc2, xc) and np.array_equal(xs2, xs)

    # the shards side by side are the unsplit result
    parts = [torch.empty(M, n_loc // 2, dtype=torch.int32) for _ in range(world)]
    dist.all_gather(parts, shard.contiguous().view(torch.int32))
    got = torch.cat([p.view(torch.bfloat16) for p in parts], dim=1)
    wc_all, ws_all = O.quant_grouped(w, 128, role="weight")
    ref = O.linear_grouped(xc, wc_all, xs, ws_all)
    assert torch.equal(got, ref), (got.float() - ref.float()).abs().max()
    dist.barrier()
    dist.destroy_process_group()


def test_dense_column_split_two_ranks():
    mp.spawn(_worker, args=(2, _free_port(), 8, 256, 64), nprocs=2, join=True)
