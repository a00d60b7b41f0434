"""GPU, 2 ranks over NCCL: the expert-parallel MoE layer equals the single-GPU layer bit for bit
(same rows reach the same experts; tiles never mix experts; the combine order is the same)."""
import os
import socket

import pytest
import torch

pytestmark = pytest.mark.gpu


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _setup_logical_ranks(world, cap=None, T=256, H=512, I=256, E=16, k=4, seed=0):
    from fp8_inference_toolkit_b200 import moe, moe_ep, synthetic

    x, logits = synthetic.moe_inputs(T, H, E, k, seed=seed, device="cuda")
    gu, dn = synthetic.moe_weights(E, H, I, seed=seed + 1, device="cuda")
    ids, w = moe.moe_route(logits, k)
    ids[5, 1] = -1   # a padded pair
    full = moe.MoEWeights.quantize(gu, dn)
    e_loc, t_loc = E // world, T // world
    layers = []
    for r in range(world):
        sl = slice(r * e_loc, (r + 1) * e_loc)
        mine = moe.MoEWeights(full.gate_up_packed[sl].contiguous(), full.gate_up_scale[sl].contiguous(),
                              full.down_packed[sl].contiguous(), full.down_scale[sl].contiguous(), e_loc, H, I)
        layers.append(moe_ep.ExpertParallelMoE(mine, E, t_loc, k, H, world=world, rank=r, cap=cap))
    return x, ids, w, full, layers, t_loc


def _swap(layers, send_name, recv_name, rows_per_block):
    """What the all-to-all does, among ranks played by one process: block d of rank s's send buffer becomes block s of
    rank d's receive buffer."""
    world = len(layers)
    for s, ls in enumerate(layers):
        src = getattr(ls, send_name).view(world, -1)
        for d, ld in enumerate(layers):
            getattr(ld, recv_name).view(world, -1)[s].copy_(src[d])


@pytest.mark.parametrize("world", [1, 2, 4])
def test_fixed_capacity_layer_kernels_one_gpu(world):
    """The expert-parallel layer's kernels with the ranks played one after the other on a single GPU (the exchange is
    a copy): plan and unpack agree with their plain-torch statements, and the combined output of all ranks is the
    single-GPU layer's, bit for bit."""
    from fp8_inference_toolkit_b200 import moe, moe_ep, ops

    x, ids, w, full, layers, t_loc = _setup_logical_ranks(world)
    for r, l in enumerate(layers):
        ts = slice(r * t_loc, (r + 1) * t_loc)
        l._prepare(x[ts].contiguous(), ids[ts].contiguous())
        hdr, slot, ret_row, overflow = moe_ep.plan_reference(l.offsets, l.sorted_pairs, world, l.cap)
        assert not overflow and int(l.overflow.item()) == 0
        assert torch.equal(l.slot.cpu(), slot) and torch.equal(l.ret_row.cpu(), ret_row)
        got_hdr = l.send.view(world, 1 + l.cap, l.row_bytes)[:, 0, :4 * (2 + l.e_loc)].contiguous().view(torch.int32)
        assert torch.equal(got_hdr.cpu(), hdr)
    _swap(layers, "send", "recv", None)
    for l in layers:
        l._unpack()
        hdrs = l.recv.view(world, 1 + l.cap, l.row_bytes)[:, 0, :4 * (2 + l.e_loc)].contiguous().view(torch.int32)
        off_loc, pos_of, R = moe_ep.unpack_reference(hdrs.cpu(), l.cap)
        assert torch.equal(l.off_loc.cpu(), off_loc) and torch.equal(l.pos_of.cpu(), pos_of) and int(l.rows_dev.item()) == R
        l._experts()
        l._pack_return()
    _swap(layers, "ret_send", "ret_recv", None)
    ops.check_status()
    out = torch.cat([moe.moe_combine(l.ret_recv, l.ret_row, w[r * t_loc:(r + 1) * t_loc].contiguous(), t_loc, l.k)
                     for r, l in enumerate(layers)])
    ref = moe.moe_layer(x, ids, w, full)
    assert torch.equal(out, ref)


def test_fixed_capacity_overflow_flag_one_gpu():
    """A capacity that is too small: the flag is raised, every index stays in range (no fault, status clean), and the
    rows that did fit are still placed consistently."""
    from fp8_inference_toolkit_b200 import moe_ep, ops

    x, ids, w, full, layers, t_loc = _setup_logical_ranks(2, cap=64)
    for r, l in enumerate(layers):
        ts = slice(r * t_loc, (r + 1) * t_loc)
        l._prepare(x[ts].contiguous(), ids[ts].contiguous())
        hdr, slot, ret_row, overflow = moe_ep.plan_reference(l.offsets, l.sorted_pairs, 2, l.cap)
        assert overflow and int(l.overflow.item()) == 1
        assert torch.equal(l.slot.cpu(), slot) and torch.equal(l.ret_row.cpu(), ret_row)
    _swap(layers, "send", "recv", None)
    for l in layers:
        l._unpack()
        hdrs = l.recv.view(2, 1 + l.cap, l.row_bytes)[:, 0, :4 * (2 + l.e_loc)].contiguous().view(torch.int32)
        off_loc, pos_of, R = moe_ep.unpack_reference(hdrs.cpu(), l.cap)
        assert torch.equal(l.pos_of.cpu(), pos_of) and int(l.rows_dev.item()) == R
        l._experts()
        l._pack_return()
    ops.check_status()


def _worker(rank, world, port):
    import torch.distributed as dist

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    from fp8_inference_toolkit_b200 import moe, moe_ep, ops, synthetic

    T, H, I, E, k = 512, 512, 256, 16, 4
    x, logits = synthetic.moe_inputs(T, H, E, k, seed=0, device="cuda")
    gu, dn = synthetic.moe_weights(E, H, I, seed=1, device="cuda")
    ids, w = moe.moe_route(logits, k)
    full = moe.MoEWeights.quantize(gu, dn)
    ref = moe.moe_layer(x, ids, w, full)
    e_loc, t_loc = E // world, T // world
    sl = slice(rank * e_loc, (rank + 1) * e_loc)
    mine = moe.MoEWeights(full.gate_up_packed[sl].contiguous(), full.gate_up_scale[sl].contiguous(),
                          full.down_packed[sl].contiguous(), full.down_scale[sl].contiguous(), e_loc, H, I)
    ts = slice(rank * t_loc, (rank + 1) * t_loc)
    for quantized in (False, True):   # bf16 rows, then rows quantised before the exchange: the same result
        out = moe_ep.moe_layer_ep(x[ts].contiguous(), ids[ts].contiguous(), w[ts].contiguous(), mine, E,
                                  quantized_dispatch=quantized)
        ops.check_status()
        assert torch.equal(out, ref[ts]), (quantized, (out.float() - ref[ts].float()).abs().max().item())
    # the fixed-capacity layer (no host synchronisation): the same bits again, twice in a row (buffers are reused)
    for transport in ("nccl", "peer"):
        layer = moe_ep.ExpertParallelMoE(mine, E, t_loc, k, H, transport=transport)
        assert layer.transport == transport
        for _ in range(3):
            out = layer(x[ts].contiguous(), ids[ts].contiguous(), w[ts].contiguous())
            ops.check_status()
            assert torch.equal(out, ref[ts]), transport
        if transport == "peer":
            # the same layer replayed as a CUDA graph (the exchange epoch advances on the device)
            xs, idss, wss = x[ts].contiguous(), ids[ts].contiguous(), w[ts].contiguous()
            graph, gout = layer.capture(xs, idss, wss)
            for _ in range(3):
                gout.zero_()
                graph.replay()
                torch.cuda.synchronize()
                ops.check_status()
                assert torch.equal(gout, ref[ts]), "graph replay"
            out = layer(xs, idss, wss)      # and eager calls still line up with the replays of the other rank
            assert torch.equal(out, ref[ts])
        assert not layer.overflowed()
        layer.close()
    tiny = moe_ep.ExpertParallelMoE(mine, E, t_loc, k, H, cap=64, check_each_call=True, transport="nccl")   # overflows: redone exactly
    assert torch.equal(tiny(x[ts].contiguous(), ids[ts].contiguous(), w[ts].contiguous()), ref[ts])
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_ep_matches_single_gpu():
    import torch.multiprocessing as mp

    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    mp.spawn(_worker, args=(2, _free_port()), nprocs=2, join=True)
