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
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_ep_matches_single_gpu():
    import torch.multiprocessing as mp

    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    mp.spawn(_worker, args=(2, _free_port()), nprocs=2, join=True)
