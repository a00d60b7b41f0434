"""Expert-parallel MoE layer: experts split across ranks, one all-to-all each way.

Rank r owns experts [r*E/n, (r+1)*E/n) and T/n of the tokens.  Per layer:

  1. local sort of the (token, slot) pairs by global expert id (device kernel) -- sorted by expert
     is also sorted by destination rank;
  2. a small all-gather of per-expert counts (the only host synchronisation: split sizes);
  3. dispatch all-to-all of the token rows in sorted order (bf16 rows, or -- on request, CUDA path -- rows
     already quantised to int4 + group scales: 3.8x fewer bytes, same result);
  4. on the owner: rows arrive grouped by source rank, each group sorted by local expert; a second
     device sort merges the groups, `gather+quantise` writes the expert-sorted packed layout,
     the grouped-tile GEMMs run, and the outputs are put back into arrival order;
  5. combine all-to-all (reverse splits) and the weighted sum on the rank that owns the token.

The exchange goes through ``torch.distributed`` (NCCL over NVLink on GPUs).  The bookkeeping is
device-agnostic, so the same code runs among CPU ranks over gloo with stand-in ``sort_fn`` /
``expert_fn`` callables in the tests; the defaults are the CUDA kernels and nothing else.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch
import torch.distributed as dist


@dataclass
class EPPlan:
    """Split sizes and permutations of one dispatch."""
    send_splits: list          # rows sent to each rank
    recv_splits: list          # rows received from each rank
    recv_counts: torch.Tensor  # [world, E_loc] rows from each source for each local expert
    sorted_pairs: torch.Tensor  # local pair order sent out
    inv_pairs: torch.Tensor
    num_pairs: int


def plan_dispatch(expert_ids: torch.Tensor, num_experts: int, sort_fn, group=None) -> EPPlan:
    """Sort local pairs by expert and exchange per-expert counts with every rank."""
    world = dist.get_world_size(group)
    e_loc = num_experts // world
    assert e_loc * world == num_experts, "experts must divide evenly across ranks"
    sorted_pairs, inv_pairs, offsets = sort_fn(expert_ids, num_experts)
    counts = (offsets[1:] - offsets[:-1]).to(torch.int64).contiguous()  # [E], grouped by owner rank
    rank = dist.get_rank(group)
    all_counts = torch.empty(world * num_experts, dtype=torch.int64, device=counts.device)
    dist.all_gather_into_tensor(all_counts, counts, group=group)  # tiny: every rank's per-expert counts
    recv_counts = all_counts.view(world, num_experts)[:, rank * e_loc:(rank + 1) * e_loc].contiguous()
    both = torch.stack([counts.view(world, e_loc).sum(1), recv_counts.sum(1)]).cpu()
    return EPPlan(both[0].tolist(), both[1].tolist(), recv_counts, sorted_pairs, inv_pairs, expert_ids.numel())


def local_expert_ids(plan: EPPlan) -> torch.Tensor:
    """Local expert id of every received row, in arrival order (source-major, expert-minor)."""
    world, e_loc = plan.recv_counts.shape
    ids = torch.arange(e_loc, device=plan.recv_counts.device, dtype=torch.int32).repeat(world)
    return torch.repeat_interleave(ids, plan.recv_counts.reshape(-1), output_size=sum(plan.recv_splits))


def exchange(rows: torch.Tensor, send_splits, recv_splits, group=None) -> torch.Tensor:
    out = rows.new_empty((sum(recv_splits),) + tuple(rows.shape[1:]))
    dist.all_to_all_single(out, rows.contiguous(), output_split_sizes=list(recv_splits),
                           input_split_sizes=list(send_splits), group=group)
    return out


def _moe_layer_ep_quantized(x, expert_ids, expert_w, weights, num_experts, group):
    """CUDA path with the dispatch payload already quantised: 68 bytes per 128 values (64 of codes, one fp32 scale)
    instead of 256 bytes of bf16.  The quantiser works on whole rows, so quantising before the exchange gives the
    codes and scales it would give after it: the layer's result is unchanged bit for bit."""
    from . import moe as _moe

    T, k = expert_ids.shape
    H = x.shape[1]
    G = H // 128
    world = dist.get_world_size(group)
    plan = plan_dispatch(expert_ids, num_experts, _moe.moe_sort_tokens, group)
    P = plan.num_pairs
    ap, asc = _moe.moe_gather_quant(x, plan.sorted_pairs, k)           # [G, P, 64], [G, P] in send order
    payload = torch.cat([ap.permute(1, 0, 2).reshape(P, G * 64),
                         asc.t().contiguous().view(torch.uint8).view(P, G * 4)], dim=1)   # one row per pair
    recv = exchange(payload, plan.send_splits, plan.recv_splits, group)
    R = recv.shape[0]
    if R > 0:
        e_loc = num_experts // world
        sp2, inv2, off2 = _moe.moe_sort_tokens(local_expert_ids(plan), e_loc)
        sel = recv.index_select(0, sp2.long())                           # expert-sorted rows
        ap2 = sel[:, :G * 64].reshape(R, G, 64).permute(1, 0, 2).contiguous()
        asc2 = sel[:, G * 64:].contiguous().view(torch.float32).view(R, G).t().contiguous()
        y = _moe.moe_experts_forward(ap2, asc2, off2, weights)
        ones = torch.ones(R, dtype=torch.float32, device=x.device)
        y_rows = _moe.moe_combine(y, inv2, ones, R, 1)                   # back to arrival order
    else:
        y_rows = x.new_empty((0, H))
    y_back = exchange(y_rows, plan.recv_splits, plan.send_splits, group)
    return _moe.moe_combine(y_back, plan.inv_pairs, expert_w.contiguous(), T, k)


def moe_layer_ep(x: torch.Tensor, expert_ids: torch.Tensor, expert_w: torch.Tensor, weights, num_experts: int,
                 group=None, sort_fn=None, expert_fn=None, combine_fn=None, quantized_dispatch=None) -> torch.Tensor:
    """Expert-parallel MoE layer.  ``x`` bf16 [T_local, H]; ``expert_ids`` int32 [T_local, k] (global ids);
    ``expert_w`` f32 [T_local, k]; ``weights`` = this rank's ``MoEWeights`` (E/n experts).

    ``quantized_dispatch`` (CUDA path only): send quantised rows (1088 bytes per 2048 values) instead of bf16 rows
    (4096 bytes).  Off by default: over NVLink the exchange is a small part of the layer and the re-layout kernels
    cost more than the bytes saved (measured on 2 GPUs: 0.96 ms against 0.79 ms per layer); it is for links an order
    of magnitude slower."""
    if sort_fn is None:
        if quantized_dispatch:
            return _moe_layer_ep_quantized(x, expert_ids, expert_w, weights, num_experts, group)
        from . import moe as _moe  # CUDA kernels; raises if the library is missing

        sort_fn = _moe.moe_sort_tokens

        def expert_fn(rows, ids_local, e_loc):  # noqa: F811
            sp2, inv2, off2 = _moe.moe_sort_tokens(ids_local, e_loc)
            ap, asc = _moe.moe_gather_quant(rows, sp2, 1)
            y = _moe.moe_experts_forward(ap, asc, off2, weights)
            ones = torch.ones(rows.shape[0], dtype=torch.float32, device=rows.device)
            return _moe.moe_combine(y, inv2, ones, rows.shape[0], 1)  # back to arrival order

        def combine_fn(y_back, inv_pairs, w, T, k):  # noqa: F811
            return _moe.moe_combine(y_back, inv_pairs, w.contiguous(), T, k)

    T, k = expert_ids.shape
    world = dist.get_world_size(group)
    plan = plan_dispatch(expert_ids, num_experts, sort_fn, group)
    x_sorted = x.index_select(0, torch.div(plan.sorted_pairs, k, rounding_mode="floor").long())
    rows = exchange(x_sorted, plan.send_splits, plan.recv_splits, group)
    if rows.shape[0] > 0:
        y_rows = expert_fn(rows, local_expert_ids(plan), num_experts // world)
    else:
        y_rows = rows.new_empty((0, x.shape[1]))
    y_back = exchange(y_rows, plan.recv_splits, plan.send_splits, group)
    return combine_fn(y_back, plan.inv_pairs, expert_w, T, k)
