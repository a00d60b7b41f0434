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


# ------------------------------------------------------------------------------------------------------------------
# Fixed-capacity exchange: the same layer without any host synchronisation
# ------------------------------------------------------------------------------------------------------------------
# ``moe_layer_ep`` above needs the split sizes of its all-to-alls on the host, i.e. one device -> host round trip per
# layer, and moves rows with torch indexing kernels.  The protocol below gives every (source, destination) pair a
# block of fixed size instead: one header row (row counts per local expert of the destination) followed by up to
# ``cap`` rows in the source's sorted order.  Blocks of equal size need no split sizes; the receiver derives every
# position from the headers on the device.  A destination that would get more than ``cap`` rows raises an overflow
# word that the caller reads after the layer (like the kernels' status word); the step is then repeated through
# ``moe_layer_ep``, so no token is ever dropped.
#
# ``plan_reference`` / ``unpack_reference`` state the bookkeeping in plain torch (any device); the CUDA kernels
# (``i4tc_moe_ep_plan``, ``i4tc_moe_ep_unpack``) are tested against them, and ``moe_layer_ep_fixed`` runs the whole
# protocol with them among CPU ranks.

def ep_capacity(pairs_per_rank: int, world: int, capacity_factor: float = 1.0) -> int:
    """Rows a rank may send to one destination: the mean, times ``capacity_factor``, plus eight standard deviations of
    a uniform routing and a constant, rounded up to a multiple of 8."""
    mean = pairs_per_rank / world
    cap = mean * capacity_factor + 8.0 * mean ** 0.5 + 32.0
    return int(-(-cap // 8) * 8)


def plan_reference(expert_offsets: torch.Tensor, sorted_pairs: torch.Tensor, world: int, cap: int):
    """Headers, buffer rows and return rows of one dispatch, as ``i4tc_moe_ep_plan`` computes them.

    Returns ``(headers int32 [world, 2 + e_loc], slot int32 [P], ret_row int32 [P], overflow bool)``."""
    off = expert_offsets.to(torch.int64).cpu()
    E = off.numel() - 1
    e_loc = E // world
    P = sorted_pairs.numel()
    hdr = torch.zeros(world, 2 + e_loc, dtype=torch.int32)
    slot = torch.full((P,), -1, dtype=torch.int32)
    ret_row = torch.full((P,), -1, dtype=torch.int32)
    overflow = False
    sp = sorted_pairs.cpu()
    for d in range(world):
        start, end = int(off[d * e_loc]), int(off[(d + 1) * e_loc])
        n = end - start
        overflow |= n > cap
        hdr[d, 0] = min(n, cap)
        hdr[d, 1] = start
        for e in range(e_loc):
            a = min(int(off[d * e_loc + e]) - start, cap)
            b = min(int(off[d * e_loc + e + 1]) - start, cap)
            hdr[d, 2 + e] = b - a
        for j in range(min(n, cap)):
            slot[start + j] = d * (1 + cap) + 1 + j
            ret_row[int(sp[start + j])] = d * cap + j
    return hdr, slot, ret_row, overflow


def unpack_reference(headers: torch.Tensor, cap: int):
    """From the ``world`` received headers ([world, 2 + e_loc], one per source): local expert offsets and the
    expert-sorted position of every received row, as ``i4tc_moe_ep_unpack`` computes them.

    Returns ``(expert_offsets_loc int32 [e_loc + 1], pos_of int32 [world * cap], rows int)``."""
    h = headers.to(torch.int64).cpu()
    world, e_loc = h.shape[0], h.shape[1] - 2
    cnt = h[:, 2:]
    off = torch.zeros(e_loc + 1, dtype=torch.int64)
    off[1:] = torch.cumsum(cnt.sum(0), 0)
    pos_of = torch.full((world * cap,), -1, dtype=torch.int32)
    for s in range(world):
        j = 0
        for e in range(e_loc):
            base = int(off[e]) + int(cnt[:s, e].sum())
            for i in range(int(cnt[s, e])):
                if j < min(int(h[s, 0]), cap):
                    pos_of[s * cap + j] = base + i
                j += 1
    return off.to(torch.int32), pos_of, int(off[-1])


def moe_layer_ep_fixed(x, expert_ids, expert_w, num_experts: int, cap: int, sort_fn, expert_fn, combine_fn, group=None):
    """The fixed-capacity protocol in plain torch (rows travel unquantised): the CPU statement of what
    ``ExpertParallelMoE`` does with kernels.  ``expert_fn(rows_sorted, expert_offsets_loc)`` maps expert-sorted rows to
    outputs.  Returns ``(out, overflow)``; on overflow ``out`` is incomplete and the caller must redo the step."""
    world = dist.get_world_size(group)
    T, k = expert_ids.shape
    H = x.shape[1]
    sorted_pairs, inv_pairs, offsets = sort_fn(expert_ids, num_experts)
    hdr, slot, ret_row, overflow = plan_reference(offsets, sorted_pairs, world, cap)
    e_loc = num_experts // world
    width = max(H, 2 + e_loc)
    send = torch.zeros(world, 1 + cap, width, dtype=torch.float32)
    send[:, 0, :2 + e_loc] = hdr.float()
    ok = slot >= 0
    rows = x.float()[torch.div(sorted_pairs[ok].long(), k, rounding_mode="floor")]
    send.view(-1, width)[slot[ok].long(), :H] = rows
    recv = torch.empty_like(send)
    dist.all_to_all_single(recv.view(-1), send.view(-1), group=group)
    off_loc, pos_of, R = unpack_reference(recv[:, 0, :2 + e_loc].to(torch.int32), cap)
    got = pos_of >= 0
    rows_sorted = torch.zeros(R, H)
    body = recv[:, 1:, :H].reshape(world * cap, H)
    rows_sorted[pos_of[got].long()] = body[got]
    y = expert_fn(rows_sorted, off_loc)
    ret_send = torch.zeros(world * cap, y.shape[1])
    ret_send[got] = y[pos_of[got].long()]
    ret_recv = torch.empty_like(ret_send)
    dist.all_to_all_single(ret_recv.view(-1), ret_send.view(-1), group=group)
    flag = torch.tensor([1.0 if overflow else 0.0])
    dist.all_reduce(flag, op=dist.ReduceOp.MAX, group=group)     # every rank learns of an overflow anywhere
    return combine_fn(ret_recv, ret_row, expert_w, T, k), bool(flag.item() > 0)


class ExpertParallelMoE:
    """Expert-parallel MoE layer on CUDA with fixed-capacity exchange buffers: no device -> host round trip, no torch
    indexing kernels; rows travel quantised (68 bytes per 128 values).  Buffers are allocated once for
    ``tokens_per_rank`` tokens and reused by every call (intermediate results of a call are overwritten by the next).

    ``transport``: ``"nccl"`` exchanges the fixed-size blocks with two ``all_to_all_single`` calls; ``"peer"`` maps
    every rank's receive and return buffers into the others' address space (``torch.distributed._symmetric_memory``)
    and lets the dispatch kernel and the down projection's epilogue store rows straight into the destination's buffer
    over NVLink, ordered by device-side flags with bounded waits -- no collective at all, no capacity padding on the
    wire, the return rows land in the source's own sorted order, and the whole call can be recorded as a CUDA graph
    (``capture``); ``"auto"`` (default) takes ``"peer"`` when symmetric memory can be set up for the group and
    ``"nccl"`` otherwise.

    ``out = layer(x, expert_ids, expert_w)``; afterwards ``layer.overflowed()`` tells whether any rank ran out of
    capacity in a call since the last check (it synchronises and reduces the flag over the ranks), in which case the
    affected outputs are incomplete and the step must be redone through ``moe_layer_ep``.  With ``check_each_call=True``
    the layer does that itself, at the price of one host synchronisation per call."""

    def __init__(self, weights, num_experts: int, tokens_per_rank: int, top_k: int, hidden: int, group=None,
                 capacity_factor: float = 1.0, check_each_call: bool = False, world: int | None = None,
                 rank: int | None = None, cap: int | None = None, transport: str = "auto"):
        from . import moe as _moe
        from ._cabi import lib

        self._moe, self._lib = _moe, lib
        self.group = group
        # `world` / `rank` are only given by tests that play several ranks in one process (and exchange the blocks
        # themselves); normally they come from the process group
        self.world = dist.get_world_size(group) if world is None else world
        self.rank = dist.get_rank(group) if rank is None else rank
        self.weights = weights
        self.E, self.k, self.H, self.T = num_experts, top_k, hidden, tokens_per_rank
        assert num_experts % self.world == 0 and hidden % 128 == 0
        self.e_loc = num_experts // self.world
        self.G = hidden // 128
        self.row_bytes = self.G * 68
        assert self.row_bytes >= 4 * (2 + self.e_loc), "hidden size too small for the header of this many experts"
        self.P = tokens_per_rank * top_k
        self.cap = ep_capacity(self.P, self.world, capacity_factor) if cap is None else cap
        self.check_each_call = check_each_call
        dev = weights.gate_up_packed.device
        self.dev = dev
        W, cap, G, H, I = self.world, self.cap, self.G, hidden, weights.inter
        R = W * cap
        self.r_max = R
        u8, i32, f32, bf16 = torch.uint8, torch.int32, torch.float32, torch.bfloat16
        self.send = torch.zeros(W * (1 + cap) * self.row_bytes, dtype=u8, device=dev)
        self.recv = torch.zeros_like(self.send)
        self.transport = "nccl"
        self.epoch_dev = torch.zeros(1, dtype=torch.int32, device=dev)   # exchanges done so far (peer transport)
        if transport in ("auto", "peer") and world is None and self.world > 1:
            try:
                self._setup_peer()
            except Exception as exc:   # symmetric memory not available for this group: keep the collective transport
                if transport == "peer":
                    raise
                self.peer_error = repr(exc)
        self.slot = torch.empty(self.P, dtype=i32, device=dev)
        self.ret_row = torch.empty(self.P, dtype=i32, device=dev)
        self.overflow = torch.zeros(1, dtype=i32, device=dev)
        self.meta = torch.empty(int(lib.i4tc_moe_ep_meta_ints(W, self.e_loc)), dtype=i32, device=dev)
        self.rows_dev = torch.zeros(1, dtype=i32, device=dev)
        self.pos_of = torch.empty(R, dtype=i32, device=dev)
        self.ap = torch.zeros(G, R, 64, dtype=u8, device=dev)
        self.asc = torch.zeros(G, R, dtype=f32, device=dev)
        self.off_loc = torch.zeros(self.e_loc + 1, dtype=i32, device=dev)
        self.h = torch.zeros(R, 2 * I, dtype=bf16, device=dev)
        self.hp = torch.zeros(I // 128, R, 64, dtype=u8, device=dev)
        self.hs = torch.zeros(I // 128, R, dtype=f32, device=dev)
        self.y = torch.zeros(R, H, dtype=bf16, device=dev)
        self.out_rows = torch.zeros(R, dtype=torch.int64, device=dev)
        self.ret_send = torch.zeros(R, H, dtype=bf16, device=dev)
        self.ret_recv = torch.zeros(R, H, dtype=bf16, device=dev)
        self.tok_packed = torch.empty(G, tokens_per_rank, 64, dtype=u8, device=dev)
        self.tok_scale = torch.empty(G, tokens_per_rank, dtype=f32, device=dev)
        self.sorted_pairs = torch.empty(self.P, dtype=i32, device=dev)
        self.inv_pairs = torch.empty(self.P, dtype=i32, device=dev)
        self.offsets = torch.empty(num_experts + 1, dtype=i32, device=dev)
        self.sort_scratch = torch.empty(max(int(lib.i4tc_moe_sort_scratch_bytes(self.P, num_experts)), 4), dtype=u8, device=dev)

    def _setup_peer(self):
        """One symmetric allocation per rank: [receive blocks | return rows in this rank's sorted order | flags]."""
        import os

        os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")   # plain peer mappings only
        import torch.distributed._symmetric_memory as symm_mem

        def up(n):
            return (n + 255) // 256 * 256

        W = self.world
        recv_bytes = up(W * (1 + self.cap) * self.row_bytes)
        ret_bytes = up(self.P * self.H * 2)
        total = recv_bytes + ret_bytes + 256
        buf = symm_mem.empty(total, dtype=torch.uint8, device=self.dev)
        buf.zero_()
        hdl = symm_mem.rendezvous(buf, dist.group.WORLD if self.group is None else self.group)
        ptrs = [int(p) for p in hdl.buffer_ptrs]
        i64 = torch.int64
        self._symm, self._hdl = buf, hdl
        self.recv = buf[:W * (1 + self.cap) * self.row_bytes]
        self.ret_local = buf[recv_bytes:recv_bytes + self.P * self.H * 2].view(torch.bfloat16).view(self.P, self.H)
        flags = buf[recv_bytes + ret_bytes:recv_bytes + ret_bytes + 256].view(torch.int32)
        self.flags_dispatch, self.flags_return = flags[:W], flags[32:32 + W]
        assert W <= 32
        self.recv_bases = torch.tensor(ptrs, dtype=i64, device=self.dev)
        self.ret_bases = torch.tensor([p + recv_bytes for p in ptrs], dtype=i64, device=self.dev)
        fbase = recv_bytes + ret_bytes
        self.flag_addrs_dispatch = torch.tensor([p + fbase + 4 * self.rank for p in ptrs], dtype=i64, device=self.dev)
        self.flag_addrs_return = torch.tensor([p + fbase + 128 + 4 * self.rank for p in ptrs], dtype=i64, device=self.dev)
        torch.cuda.synchronize(self.dev)
        dist.barrier(group=self.group)    # every rank's flags are zero before anyone signals
        self.transport = "peer"
        self.send = None

    # -- stages -------------------------------------------------------------------------------------------------
    def _prepare(self, x, expert_ids):
        from ._cabi import check
        lib, d, st = self._lib, self.dev.index, torch.cuda.current_stream(self.dev).cuda_stream
        ids = expert_ids.contiguous().view(-1)
        assert ids.numel() == self.P and x.shape == (self.T, self.H) and x.dtype == torch.bfloat16 and x.is_contiguous()
        peer = self.transport == "peer"
        bases = self.recv_bases.data_ptr() if peer else None
        send = None if peer else self.send.data_ptr()
        check(lib.i4tc_moe_sort(ids.data_ptr(), self.P, self.E, self.sorted_pairs.data_ptr(), self.inv_pairs.data_ptr(),
                                self.offsets.data_ptr(), self.sort_scratch.data_ptr(), self.sort_scratch.numel(), d, st),
              "moe_sort")
        check(lib.i4tc_moe_ep_plan(self.offsets.data_ptr(), self.sorted_pairs.data_ptr(), self.P, self.E, self.world,
                                   self.cap, self.row_bytes, send, self.slot.data_ptr(), self.ret_row.data_ptr(),
                                   self.overflow.data_ptr(), bases, self.rank, d, st), "moe_ep_plan")
        # every token is quantised once; its 68 bytes per group are then copied to the block row of each of its pairs
        check(lib.i4tc_quant_grouped(x.data_ptr(), 0, self.T, self.H, x.stride(0), 128, self.tok_packed.data_ptr(),
                                     self.tok_scale.data_ptr(), 0, d, st), "quant_grouped")
        check(lib.i4tc_moe_gather_packed(self.tok_packed.data_ptr(), self.tok_scale.data_ptr(), self.T, self.G,
                                         self.sorted_pairs.data_ptr(), self.P, self.k, send, None, self.slot.data_ptr(),
                                         self.row_bytes, bases, self.cap, self.rank, d, st), "moe_gather_packed")

    def _signal(self, addrs, bump: bool):
        from ._cabi import check
        check(self._lib.i4tc_peer_signal_counter(addrs.data_ptr(), self.world, self.epoch_dev.data_ptr(), int(bump),
                                                 self.dev.index, torch.cuda.current_stream(self.dev).cuda_stream),
              "peer_signal_counter")

    def _wait(self, flags):
        from ._cabi import check
        check(self._lib.i4tc_peer_wait_counter(flags.data_ptr(), self.world, self.epoch_dev.data_ptr(), self.dev.index,
                                               torch.cuda.current_stream(self.dev).cuda_stream), "peer_wait_counter")

    def _unpack(self):
        from ._cabi import check
        lib, d, st = self._lib, self.dev.index, torch.cuda.current_stream(self.dev).cuda_stream
        check(lib.i4tc_moe_ep_unpack(self.recv.data_ptr(), self.world, self.e_loc, self.cap, self.row_bytes, self.G,
                                     self.ap.data_ptr(), self.asc.data_ptr(), self.off_loc.data_ptr(),
                                     self.pos_of.data_ptr(), self.meta.data_ptr(), self.rows_dev.data_ptr(), d, st),
              "moe_ep_unpack")

    def _experts(self):
        from ._cabi import check
        lib, d, st = self._lib, self.dev.index, torch.cuda.current_stream(self.dev).cuda_stream
        w, m = self.weights, self._moe
        m.moe_w4a4_grouped_gemm(self.ap, self.asc, w.gate_up_packed, w.gate_up_scale, self.off_loc, self.h, 2 * w.inter,
                                self.G, self.e_loc)
        check(lib.i4tc_moe_silu_mul_quant_rows(self.h.data_ptr(), self.r_max, self.rows_dev.data_ptr(), w.inter,
                                               self.hp.data_ptr(), self.hs.data_ptr(), d, st), "moe_silu_mul_quant_rows")
        if self.transport == "peer":
            # the down projection writes every row straight into the return buffer of the rank it came from
            check(lib.i4tc_moe_ep_return_rows(self.pos_of.data_ptr(), self.r_max, self.H, self.ret_bases.data_ptr(),
                                              self.meta.data_ptr(), self.world, self.e_loc, self.cap,
                                              self.out_rows.data_ptr(), d, st), "moe_ep_return_rows")
            m.moe_w4a4_grouped_gemm_rows(self.hp, self.hs, w.down_packed, w.down_scale, self.off_loc, self.out_rows,
                                         self.H, w.inter // 128, self.e_loc)
        else:
            m.moe_w4a4_grouped_gemm(self.hp, self.hs, w.down_packed, w.down_scale, self.off_loc, self.y, self.H,
                                    w.inter // 128, self.e_loc)

    def _pack_return(self):
        from ._cabi import check
        lib, d, st = self._lib, self.dev.index, torch.cuda.current_stream(self.dev).cuda_stream
        if self.transport == "peer":
            return   # the down projection already stored the rows where they belong
        else:
            check(lib.i4tc_moe_ep_pack_return(self.y.data_ptr(), self.pos_of.data_ptr(), self.r_max, self.H,
                                              self.ret_send.data_ptr(), None, None, 0, 0, 0, d, st), "moe_ep_pack_return")

    def _stages(self, x, expert_ids, expert_w):
        if self.transport == "peer":
            yield "sort_plan_quantise_store", lambda: (self._prepare(x, expert_ids), self._signal(self.flag_addrs_dispatch, True))
            yield "wait_rows", lambda: self._wait(self.flags_dispatch)
            yield "unpack", self._unpack
            yield "experts", self._experts
            yield "return_signal", lambda: self._signal(self.flag_addrs_return, False)
            yield "wait_returns", lambda: self._wait(self.flags_return)
            yield "combine", lambda: self._moe.moe_combine(self.ret_local, self.inv_pairs, expert_w.contiguous(), self.T, self.k)
            return
        yield "sort_plan_quantise", lambda: self._prepare(x, expert_ids)
        yield "dispatch_all_to_all", lambda: dist.all_to_all_single(self.recv, self.send, group=self.group)
        yield "unpack", self._unpack
        yield "experts", self._experts
        yield "pack_return", self._pack_return
        yield "combine_all_to_all", lambda: dist.all_to_all_single(self.ret_recv.view(-1), self.ret_send.view(-1), group=self.group)
        yield "combine", lambda: self._moe.moe_combine(self.ret_recv, self.ret_row, expert_w.contiguous(), self.T, self.k)

    def __call__(self, x: torch.Tensor, expert_ids: torch.Tensor, expert_w: torch.Tensor) -> torch.Tensor:
        out = None
        for _, fn in self._stages(x, expert_ids, expert_w):
            out = fn()
        if self.check_each_call and self.overflowed():
            out = moe_layer_ep(x, expert_ids, expert_w, self.weights, self.E, group=self.group)
        return out

    def capture(self, x: torch.Tensor, expert_ids: torch.Tensor, expert_w: torch.Tensor):
        """One call of the layer on these (static) tensors as a CUDA graph: ``graph, out = layer.capture(...)``, then
        ``graph.replay()`` redoes the layer on whatever the tensors hold and leaves the result in ``out``.  Peer
        transport only (every launch of the layer is then one of this library's kernels and the exchange epoch lives
        on the device).  Collective: every rank captures, and later replays, the same number of times."""
        assert self.transport == "peer", "graph capture needs the peer transport"
        side = torch.cuda.Stream(self.dev)
        side.wait_stream(torch.cuda.current_stream(self.dev))
        with torch.cuda.stream(side):
            for _ in range(2):   # first-use allocations (workspaces, device info) happen outside the capture
                self(x, expert_ids, expert_w)
        side.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=side):
            out = self(x, expert_ids, expert_w)
        return graph, out

    def overflowed(self) -> bool:
        """True if any rank exceeded its capacity in a call since the last check (collective: every rank must call it)."""
        flag = self.overflow.clone()
        dist.all_reduce(flag, op=dist.ReduceOp.MAX, group=self.group)
        hit = bool(flag.item() != 0)
        self.overflow.zero_()
        return hit

    def stage_times_us(self, x, expert_ids, expert_w, reps: int = 10) -> dict:
        """Mean device time of each stage (CUDA events; a stage's wait for the slowest rank is part of its exchange)."""
        acc = {}
        for it in range(reps + 2):
            evs, names = [torch.cuda.Event(enable_timing=True)], []
            evs[0].record()
            for name, fn in self._stages(x, expert_ids, expert_w):
                fn()
                e = torch.cuda.Event(enable_timing=True)
                e.record()
                evs.append(e)
                names.append(name)
            torch.cuda.synchronize()
            if it >= 2:
                for i, n in enumerate(names):
                    acc[n] = acc.get(n, 0.0) + evs[i].elapsed_time(evs[i + 1]) * 1e3 / reps
        return {n: round(v, 1) for n, v in acc.items()}

    def close(self) -> None:
        if self.transport == "peer":
            torch.cuda.synchronize(self.dev)
            dist.barrier(group=self.group)   # nobody still writes into a buffer that is about to go
        for n in ("send", "recv", "ap", "asc", "h", "hp", "hs", "y", "ret_send", "ret_recv", "ret_local", "_symm", "_hdl"):
            setattr(self, n, None)
