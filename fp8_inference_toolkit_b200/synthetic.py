"""Seeded synthetic inputs with the shapes and value distributions of the benchmark configurations
(they stand in for real Qwen3 activations and weights, which are not available offline)."""
from __future__ import annotations

import math

import torch

#: Qwen3-8B linear shapes (K, N): QKV, O, gate+up, down
QWEN3_8B_SHAPES = {"qkv": (4096, 6144), "o": (4096, 4096), "gate_up": (4096, 24576), "down": (12288, 4096)}


def activations(M: int, K: int, seed: int = 0, outlier_frac: float | None = None, device="cpu") -> torch.Tensor:
    """bf16 [M,K] ~ N(0,1) with a few outlier channels scaled x20.

    ``outlier_frac=None`` uses 8 channels per 4096 (config 0/1); the quantise benchmark uses 1 %."""
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(M, K, generator=g, dtype=torch.float32)
    n_out = max(1, round(K * 8 / 4096)) if outlier_frac is None else max(1, math.ceil(outlier_frac * K))
    idx = torch.randperm(K, generator=g)[:n_out]
    x[:, idx] *= 20.0
    return x.to(torch.bfloat16).to(device)


def weights(N: int, K: int, seed: int = 1, device="cpu") -> torch.Tensor:
    """bf16 [N,K] ~ N(0, 0.02)."""
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(N, K, generator=g, dtype=torch.float32) * 0.02).to(torch.bfloat16).to(device)


def random_packed(shape, seed: int, device="cpu") -> torch.Tensor:
    """Uniformly random packed int4 bytes (every code in [-8, 7] equally likely)."""
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, 256, shape, generator=g, dtype=torch.uint8).to(device)


def moe_inputs(T: int, H: int, E: int, top_k: int, seed: int = 0, device="cpu"):
    """x bf16 [T,H] ~ N(0,1), router logits f32 [T,E] ~ N(0,1)."""
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(T, H, generator=g, dtype=torch.float32).to(torch.bfloat16)
    logits = torch.randn(T, E, generator=g, dtype=torch.float32)
    return x.to(device), logits.to(device)


def moe_weights(E: int, H: int, I: int, seed: int = 1, device="cpu"):
    """gate+up bf16 [E,2I,H] and down bf16 [E,H,I], both ~ N(0, 0.02)."""
    g = torch.Generator().manual_seed(seed)
    gu = (torch.randn(E, 2 * I, H, generator=g, dtype=torch.float32) * 0.02).to(torch.bfloat16)
    dn = (torch.randn(E, H, I, generator=g, dtype=torch.float32) * 0.02).to(torch.bfloat16)
    return gu.to(device), dn.to(device)
