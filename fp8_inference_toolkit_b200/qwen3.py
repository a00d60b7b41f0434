"""Qwen3-8B-shaped prefill with every linear replaced by the W4A4 group-128 linear
(BASELINE configs[4]: 36 layers, hidden 4096, 32 query / 8 KV heads, head_dim 128, SwiGLU 12288,
RMSNorm, RoPE; attention stays in bf16 through torch SDPA).  Random-initialised weights: this is a
throughput harness for the caller side of the op boundary, not a checkpoint loader.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch
import torch.nn.functional as F
from torch import nn

from . import moe as _moe
from . import ops
from .linear import W4A4Linear, apply_quantized


@dataclass
class Qwen3Config:
    hidden: int = 4096
    layers: int = 36
    q_heads: int = 32
    kv_heads: int = 8
    head_dim: int = 128
    inter: int = 12288
    vocab: int = 151936
    rope_theta: float = 1.0e6
    eps: float = 1e-6


class RMSNorm(nn.Module):
    def __init__(self, dim: int, eps: float, device=None):
        super().__init__()
        self.weight = nn.Parameter(torch.ones(dim, dtype=torch.bfloat16, device=device), requires_grad=False)
        self.eps = eps

    def forward(self, x):
        xf = x.float()
        return (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + self.eps)).to(x.dtype) * self.weight


def rope_tables(seq: int, head_dim: int, theta: float, device):
    inv = 1.0 / (theta ** (torch.arange(0, head_dim, 2, device=device, dtype=torch.float32) / head_dim))
    ang = torch.outer(torch.arange(seq, device=device, dtype=torch.float32), inv)
    return ang.cos().to(torch.bfloat16), ang.sin().to(torch.bfloat16)


def apply_rope(x, cos, sin):
    # x [B, H, S, D]; rotate-half convention
    d = x.shape[-1] // 2
    x1, x2 = x[..., :d], x[..., d:]
    c, s = cos[None, None], sin[None, None]
    return torch.cat([x1 * c - x2 * s, x2 * c + x1 * s], dim=-1)


class Block(nn.Module):
    def __init__(self, cfg: Qwen3Config, device, per_channel: bool, gen: torch.Generator, fused: bool = True):
        super().__init__()
        self.cfg = cfg
        qkv_out = (cfg.q_heads + 2 * cfg.kv_heads) * cfg.head_dim
        self.qkv = self._lin(cfg.hidden, qkv_out, device, per_channel, gen)
        self.o = self._lin(cfg.q_heads * cfg.head_dim, cfg.hidden, device, per_channel, gen)
        self.gate_up = self._lin(cfg.hidden, 2 * cfg.inter, device, per_channel, gen)
        self.down = self._lin(cfg.inter, cfg.hidden, device, per_channel, gen)
        self.ln1 = RMSNorm(cfg.hidden, cfg.eps, device)
        self.ln2 = RMSNorm(cfg.hidden, cfg.eps, device)
        self.q_norm = RMSNorm(cfg.head_dim, cfg.eps, device)
        self.k_norm = RMSNorm(cfg.head_dim, cfg.eps, device)
        # fold the quantisers into RMSNorm / SwiGLU (per-group scales only; the per-channel ops keep the plain path)
        self.fused = fused and not per_channel

    @staticmethod
    def _lin(k, n, device, per_channel, gen):
        lin = W4A4Linear(k, n, per_channel=per_channel, device=device)
        # fill in slabs so that an 8-billion-parameter model never needs an fp32 copy of a whole matrix
        for r0 in range(0, n, 4096):
            r1 = min(n, r0 + 4096)
            lin.weight.data[r0:r1] = (torch.randn(r1 - r0, k, device=device, generator=gen) * 0.02).to(torch.bfloat16)
        return lin.quantize_()  # the bf16 weight is released here

    def forward(self, x, cos, sin):
        cfg = self.cfg
        B, S, _ = x.shape
        if self.fused:
            return self._forward_fused(x, cos, sin)
        qkv = self.qkv(self.ln1(x))
        q, k, v = qkv.split([cfg.q_heads * cfg.head_dim, cfg.kv_heads * cfg.head_dim, cfg.kv_heads * cfg.head_dim], -1)
        q = self.q_norm(q.view(B, S, cfg.q_heads, cfg.head_dim)).transpose(1, 2)
        k = self.k_norm(k.view(B, S, cfg.kv_heads, cfg.head_dim)).transpose(1, 2)
        v = v.view(B, S, cfg.kv_heads, cfg.head_dim).transpose(1, 2)
        q, k = apply_rope(q, cos, sin), apply_rope(k, cos, sin)
        a = F.scaled_dot_product_attention(q, k, v, is_causal=True, enable_gqa=True)
        x = x + self.o(a.transpose(1, 2).reshape(B, S, -1))
        gu = self.gate_up(self.ln2(x))
        g, u = gu.split(cfg.inter, -1)
        return x + self.down(F.silu(g) * u)


    def _attention(self, qkv, B, S, cos, sin):
        cfg = self.cfg
        q, k, v = qkv.split([cfg.q_heads * cfg.head_dim, cfg.kv_heads * cfg.head_dim, cfg.kv_heads * cfg.head_dim], -1)
        q = self.q_norm(q.view(B, S, cfg.q_heads, cfg.head_dim)).transpose(1, 2)
        k = self.k_norm(k.view(B, S, cfg.kv_heads, cfg.head_dim)).transpose(1, 2)
        v = v.view(B, S, cfg.kv_heads, cfg.head_dim).transpose(1, 2)
        q, k = apply_rope(q, cos, sin), apply_rope(k, cos, sin)
        a = F.scaled_dot_product_attention(q, k, v, is_causal=True, enable_gqa=True)
        return a.transpose(1, 2).reshape(B, S, -1)

    def _forward_fused(self, x, cos, sin):
        """Per-group mode with the quantisers folded into the ops in front of them: RMSNorm + quantise in one
        kernel before qkv and gate+up, SwiGLU + quantise in one kernel before down."""
        B, S, H = x.shape
        M = B * S
        xp, xs = ops.rmsnorm_int4_quant_grouped(x.view(M, H), self.ln1.weight, self.ln1.eps)
        qkv = apply_quantized(self.qkv, xp, xs, M).view(B, S, -1)
        x = x + self.o(self._attention(qkv, B, S, cos, sin))
        xp, xs = ops.rmsnorm_int4_quant_grouped(x.view(M, H), self.ln2.weight, self.ln2.eps)
        gu = apply_quantized(self.gate_up, xp, xs, M)
        ap, asc = _moe.moe_silu_mul_quant(gu)
        return x + apply_quantized(self.down, ap, asc, M).view(B, S, H)


class Qwen3Prefill(nn.Module):
    def __init__(self, cfg: Qwen3Config = Qwen3Config(), device="cuda", per_channel: bool = False, seed: int = 1,
                 fused: bool = True):
        super().__init__()
        self.cfg = cfg
        gen = torch.Generator(device=device).manual_seed(seed)
        self.embed = nn.Embedding(cfg.vocab, cfg.hidden, device=device, dtype=torch.bfloat16)
        self.blocks = nn.ModuleList(Block(cfg, device, per_channel, gen, fused) for _ in range(cfg.layers))
        self.norm = RMSNorm(cfg.hidden, cfg.eps, device)

    @torch.no_grad()
    def forward(self, ids: torch.Tensor) -> torch.Tensor:
        """Token ids [B, S] -> final hidden states [B, S, hidden] (prefill; no LM head, no KV cache)."""
        x = self.embed(ids)
        cos, sin = rope_tables(ids.shape[1], self.cfg.head_dim, self.cfg.rope_theta, ids.device)
        for blk in self.blocks:
            x = blk(x, cos, sin)
        return self.norm(x)
