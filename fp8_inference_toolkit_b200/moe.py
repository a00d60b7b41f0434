"""MoE grouped W4A4 ops (no counterpart in the reference, whose "grouped" always means K groups).

A layer is: route -> device-side sort of (token, slot) pairs by expert -> gather + grouped-quantise
into expert-sorted layout -> grouped-tile GEMM (gate+up) -> SwiGLU + re-quantise -> grouped-tile
GEMM (down) -> weighted combine.  With expert parallelism the sorted pairs are exchanged with one
all-to-all each way (``torch.distributed``; NCCL on GPUs, gloo in CPU tests of the host logic).
"""
from __future__ import annotations

from dataclasses import dataclass

import torch

from . import _cabi
from ._cabi import check, lib
from .ops import _dev, _require, _stream, static_int4_weight_quant_grouped


def moe_route(logits: torch.Tensor, top_k: int = 8):
    """softmax over experts, top-k, weights renormalised to sum to one.  Returns (ids i32 [T,k], w f32 [T,k])."""
    p = torch.softmax(logits.float(), dim=-1)
    w, idx = torch.topk(p, top_k, dim=-1)
    w = w / w.sum(dim=-1, keepdim=True)
    return idx.to(torch.int32).contiguous(), w.to(torch.float32).contiguous()


def moe_sort_tokens(expert_ids: torch.Tensor, num_experts: int):
    """Stable sort of the flattened (token, slot) pairs by expert id, entirely on the device.

    Returns ``(sorted_pairs i32 [P], inv_pairs i32 [P], expert_offsets i32 [E+1])`` where
    ``sorted_pairs[i]`` is the pair index (token*top_k + slot) at sorted position ``i`` and
    ``inv_pairs`` is its inverse."""
    _require(expert_ids.is_cuda and expert_ids.dtype == torch.int32, "expert_ids must be an int32 CUDA tensor")
    ids = expert_ids.contiguous().view(-1)
    P = ids.numel()
    dev = ids.device
    sorted_pairs = torch.empty(P, dtype=torch.int32, device=dev)
    inv_pairs = torch.empty(P, dtype=torch.int32, device=dev)
    offsets = torch.empty(num_experts + 1, dtype=torch.int32, device=dev)
    nbytes = lib.i4tc_moe_sort_scratch_bytes(P, num_experts)
    scratch = torch.empty(max(nbytes, 4), dtype=torch.uint8, device=dev)
    check(lib.i4tc_moe_sort(ids.data_ptr(), P, num_experts, sorted_pairs.data_ptr(), inv_pairs.data_ptr(),
                            offsets.data_ptr(), scratch.data_ptr(), scratch.numel(), _dev(ids), _stream(ids)),
          "moe_sort_tokens")
    return sorted_pairs, inv_pairs, offsets


def moe_gather_quant(x: torch.Tensor, sorted_pairs: torch.Tensor, top_k: int):
    """Rows ``x[sorted_pairs // top_k]`` grouped-quantised (gs=128) into [G,P,64] / [G,P].  A pair index that
    names no row of ``x`` (the -1 entries the sort leaves for ids outside [0, E)) gives a row of zero codes."""
    _require(x.is_cuda and x.dim() == 2 and x.is_contiguous(), "x must be a contiguous 2D CUDA tensor")
    _require(x.dtype == torch.bfloat16, "x must be bfloat16")
    K = x.shape[1]
    _require(K % 128 == 0, "hidden size must be a multiple of 128")
    P = sorted_pairs.numel()
    G = K // 128
    packed = torch.empty((G, P, 64), dtype=torch.uint8, device=x.device)
    scale = torch.empty((G, P), dtype=torch.float32, device=x.device)
    check(lib.i4tc_moe_gather_quant(x.data_ptr(), _cabi.BF16, x.shape[0], K, x.stride(0), sorted_pairs.data_ptr(), P, top_k,
                                    packed.data_ptr(), scale.data_ptr(), _dev(x), _stream(x)), "moe_gather_quant")
    return packed, scale


def moe_quant_gather(x: torch.Tensor, sorted_pairs: torch.Tensor, top_k: int):
    """The result of ``moe_gather_quant`` by quantising every token once and copying its packed row to each of its
    (token, slot) pairs: the quantiser works on whole rows, so the codes and scales are the same, with ``top_k`` times
    less arithmetic.  Rows of pairs the sort left out (index -1) are left unwritten: no later stage reads them."""
    from .ops import dynamic_int4_quant_grouped

    _require(x.is_cuda and x.dim() == 2 and x.is_contiguous() and x.dtype == torch.bfloat16,
             "x must be a contiguous 2D bfloat16 CUDA tensor")
    T, K = x.shape
    _require(K % 128 == 0, "hidden size must be a multiple of 128")
    G = K // 128
    tp, ts = dynamic_int4_quant_grouped(x, 128)
    P = sorted_pairs.numel()
    packed = torch.empty((G, P, 64), dtype=torch.uint8, device=x.device)
    scale = torch.empty((G, P), dtype=torch.float32, device=x.device)
    check(lib.i4tc_moe_gather_packed(tp.data_ptr(), ts.data_ptr(), T, G, sorted_pairs.data_ptr(), P, top_k,
                                     packed.data_ptr(), scale.data_ptr(), None, 0, None, 0, 0, _dev(x), _stream(x)),
          "moe_quant_gather")
    return packed, scale


def moe_w4a4_grouped_gemm(a_packed, scale_a, b_packed, scale_b, expert_offsets, out, N: int, num_groups: int,
                          num_experts: int) -> None:
    """out[r,:] = linear_grouped(a[:, r, :], W_e) for rows r of expert e (bf16 [P,N], caller-allocated).

    ``a_packed`` [G,P,64], ``scale_a`` [G,P]; ``b_packed`` [E,G,N,64], ``scale_b`` [E,G,N];
    ``expert_offsets`` int32 [E+1] on the device."""
    P = out.shape[0]
    _require(out.dtype == torch.bfloat16 and out.is_contiguous() and out.shape[1] == N, "out must be bf16 [P,N]")
    _require(a_packed.dtype == torch.uint8 and a_packed.is_contiguous() and a_packed.numel() == num_groups * P * 64,
             "a_packed must be [G,P,64] uint8")
    _require(b_packed.dtype == torch.uint8 and b_packed.is_contiguous()
             and b_packed.numel() == num_experts * num_groups * N * 64, "b_packed must be [E,G,N,64] uint8")
    _require(scale_a.dtype == torch.float32 and scale_a.numel() == num_groups * P, "scale_a must be f32 [G,P]")
    _require(scale_b.dtype == torch.float32 and scale_b.numel() == num_experts * num_groups * N,
             "scale_b must be f32 [E,G,N]")
    _require(expert_offsets.dtype == torch.int32 and expert_offsets.numel() == num_experts + 1,
             "expert_offsets must be int32 [E+1]")
    check(lib.i4tc_moe_grouped_gemm(a_packed.data_ptr(), scale_a.data_ptr(), b_packed.data_ptr(),
                                    scale_b.data_ptr(), expert_offsets.data_ptr(), out.data_ptr(), P, N,
                                    num_groups, num_experts, _dev(out), _stream(out)), "moe_w4a4_grouped_gemm")


def moe_w4a4_grouped_gemm_rows(a_packed, scale_a, b_packed, scale_b, expert_offsets, out_rows, N: int, num_groups: int,
                               num_experts: int) -> None:
    """The grouped GEMM with output row r written to address ``out_rows[r]`` (int64 [P] on the device, 16-byte aligned
    addresses of N bf16 values each; they may lie in another GPU's memory)."""
    P = out_rows.numel()
    _require(out_rows.dtype == torch.int64 and out_rows.is_cuda and out_rows.is_contiguous(), "out_rows must be int64 [P]")
    _require(N % 8 == 0, "N must be a multiple of 8")
    _require(a_packed.dtype == torch.uint8 and a_packed.is_contiguous() and a_packed.numel() == num_groups * P * 64,
             "a_packed must be [G,P,64] uint8")
    _require(b_packed.dtype == torch.uint8 and b_packed.is_contiguous()
             and b_packed.numel() == num_experts * num_groups * N * 64, "b_packed must be [E,G,N,64] uint8")
    _require(scale_a.dtype == torch.float32 and scale_a.numel() == num_groups * P, "scale_a must be f32 [G,P]")
    _require(scale_b.dtype == torch.float32 and scale_b.numel() == num_experts * num_groups * N,
             "scale_b must be f32 [E,G,N]")
    _require(expert_offsets.dtype == torch.int32 and expert_offsets.numel() == num_experts + 1,
             "expert_offsets must be int32 [E+1]")
    check(lib.i4tc_moe_grouped_gemm_rows(a_packed.data_ptr(), scale_a.data_ptr(), b_packed.data_ptr(),
                                         scale_b.data_ptr(), expert_offsets.data_ptr(), out_rows.data_ptr(), P, N,
                                         num_groups, num_experts, _dev(out_rows), _stream(out_rows)),
          "moe_w4a4_grouped_gemm_rows")


def moe_silu_mul_quant(h: torch.Tensor):
    """bf16 [P,2I] laid out [gate | up] -> SwiGLU -> grouped-quantised [I/128,P,64] / [I/128,P]."""
    _require(h.is_cuda and h.dtype == torch.bfloat16 and h.is_contiguous(), "h must be contiguous bf16 CUDA")
    P, two_i = h.shape
    I = two_i // 2
    _require(I % 128 == 0, "intermediate size must be a multiple of 128")
    packed = torch.empty((I // 128, P, 64), dtype=torch.uint8, device=h.device)
    scale = torch.empty((I // 128, P), dtype=torch.float32, device=h.device)
    check(lib.i4tc_moe_silu_mul_quant(h.data_ptr(), P, I, packed.data_ptr(), scale.data_ptr(), _dev(h), _stream(h)),
          "moe_silu_mul_quant")
    return packed, scale


def moe_combine(y: torch.Tensor, inv_pairs: torch.Tensor, weights: torch.Tensor, T: int, top_k: int):
    """out[t] = bf16(sum_j w[t,j] * y[inv_pairs[t*k+j]]) -> bf16 [T,H]."""
    H = y.shape[1]
    out = torch.empty((T, H), dtype=torch.bfloat16, device=y.device)
    check(lib.i4tc_moe_combine(y.data_ptr(), inv_pairs.data_ptr(), weights.data_ptr(), T, top_k, H,
                               out.data_ptr(), _dev(y), _stream(y)), "moe_combine")
    return out


@dataclass
class MoEWeights:
    """Per-expert grouped-quantised weights, stacked: gate_up [E,G1,2I,64] / [E,G1,2I], down [E,G2,H,64] / [E,G2,H]."""
    gate_up_packed: torch.Tensor
    gate_up_scale: torch.Tensor
    down_packed: torch.Tensor
    down_scale: torch.Tensor
    num_experts: int
    hidden: int
    inter: int

    @staticmethod
    def quantize(w_gate_up: torch.Tensor, w_down: torch.Tensor) -> "MoEWeights":
        """``w_gate_up`` bf16 [E,2I,H], ``w_down`` bf16 [E,H,I] -> group-128 int4 (weight role)."""
        E, two_i, H = w_gate_up.shape
        gp, gs, dp, ds = [], [], [], []
        for e in range(E):
            p, s = static_int4_weight_quant_grouped(w_gate_up[e], 128)
            gp.append(p); gs.append(s)
            p, s = static_int4_weight_quant_grouped(w_down[e], 128)
            dp.append(p); ds.append(s)
        return MoEWeights(torch.stack(gp), torch.stack(gs), torch.stack(dp), torch.stack(ds), E, H, two_i // 2)


def moe_experts_forward(x_rows_packed, x_rows_scale, expert_offsets, w: MoEWeights) -> torch.Tensor:
    """Expert MLPs over expert-sorted, already quantised rows: gate+up -> SwiGLU+quant -> down.  bf16 [P,H]."""
    P = x_rows_scale.shape[1]
    dev = x_rows_scale.device
    h = torch.empty((P, 2 * w.inter), dtype=torch.bfloat16, device=dev)
    moe_w4a4_grouped_gemm(x_rows_packed, x_rows_scale, w.gate_up_packed, w.gate_up_scale, expert_offsets, h,
                          2 * w.inter, w.hidden // 128, w.num_experts)
    ap, asc = moe_silu_mul_quant(h)
    y = torch.empty((P, w.hidden), dtype=torch.bfloat16, device=dev)
    moe_w4a4_grouped_gemm(ap, asc, w.down_packed, w.down_scale, expert_offsets, y, w.hidden, w.inter // 128,
                          w.num_experts)
    return y


def moe_layer(x: torch.Tensor, expert_ids: torch.Tensor, expert_w: torch.Tensor, w: MoEWeights) -> torch.Tensor:
    """Single-GPU MoE layer.  ``x`` bf16 [T,H]; ``expert_ids`` i32 [T,k]; ``expert_w`` f32 [T,k] -> bf16 [T,H]."""
    T, top_k = expert_ids.shape
    sorted_pairs, inv_pairs, offsets = moe_sort_tokens(expert_ids, w.num_experts)
    ap, asc = moe_quant_gather(x, sorted_pairs, top_k)
    y = moe_experts_forward(ap, asc, offsets, w)
    return moe_combine(y, inv_pairs, expert_w.contiguous(), T, top_k)
