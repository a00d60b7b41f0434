"""The caller side of the op boundary: the two-phase protocol of the reference's vLLM linear
method (``create_weights`` / ``process_weights_after_loading`` / ``apply``; described in
``docs/native_int4_tc_implementation_report.md:515-562``), as plain classes plus an ``nn.Module``.

Mode selection follows the plugin's environment flag ``INT4TC_PER_CHANNEL``
(``int4_native_tc/benchmark_all.py:46-59``): set to ``1`` for per-token / per-channel scales,
otherwise per-group-128 scales (the reference's "Enhanced-PG" symmetric configuration).
"""
from __future__ import annotations

import os

import torch
from torch import nn

from . import ops

GROUP_SIZE = 128


def per_channel_from_env() -> bool:
    return os.environ.get("INT4TC_PER_CHANNEL", "0") == "1"


class W4A4Int4TCLinearMethod:
    """``process_weights_after_loading`` quantises the bf16 weight once; ``apply`` quantises the
    activations and runs the W4A4 GEMM on every forward."""

    def __init__(self, per_channel: bool | None = None):
        self.per_channel = per_channel_from_env() if per_channel is None else per_channel

    def create_weights(self, layer: nn.Module, input_size: int, output_size: int, params_dtype=torch.bfloat16,
                       device=None) -> None:
        layer.weight = nn.Parameter(torch.empty(output_size, input_size, dtype=params_dtype, device=device),
                                    requires_grad=False)
        layer.input_size_per_partition = input_size
        layer.output_size_per_partition = output_size

    def process_weights_after_loading(self, layer: nn.Module) -> None:
        w = layer.weight.data
        if self.per_channel:
            packed, scale = ops.static_int4_weight_quant(w)  # [N,K/2], [N]
        else:
            packed, scale = ops.static_int4_weight_quant_grouped(w, GROUP_SIZE)  # [G,N,64], [G,N]
        layer.weight = None
        layer.weight_int4 = nn.Parameter(packed, requires_grad=False)
        layer.weight_scale = nn.Parameter(scale, requires_grad=False)

    def apply(self, layer: nn.Module, x: torch.Tensor, bias: torch.Tensor | None = None) -> torch.Tensor:
        K = layer.input_size_per_partition
        N = layer.output_size_per_partition
        x2d = x.reshape(-1, K)
        M = x2d.shape[0]
        out = torch.empty((M, N), dtype=torch.bfloat16, device=x.device)
        if self.per_channel:
            xp, xs = ops.dynamic_int4_quant(x2d)
            ops.cutlass_int4_scaled_mm(xp, layer.weight_int4, xs, layer.weight_scale, out, M, N, K)
        else:
            xp, xs = ops.dynamic_int4_quant_grouped(x2d, GROUP_SIZE)
            ops.cutlass_int4_fused_grouped_gemm(xp, layer.weight_int4, xs, layer.weight_scale, out, M, N,
                                                GROUP_SIZE, K // GROUP_SIZE)
        if out.dtype != x.dtype:
            out = out.to(x.dtype)
        if bias is not None:
            out = out + bias
        return out.reshape(*x.shape[:-1], N)


def apply_quantized(layer: nn.Module, x_packed: torch.Tensor, x_scale: torch.Tensor, M: int,
                    bias: torch.Tensor | None = None) -> torch.Tensor:
    """The per-group linear on activations that are already quantised ([G,M,64] codes, [G,M] scales) -- for
    callers that fuse the quantiser into the preceding op (RMSNorm, SwiGLU).  bf16 [M, N]."""
    K = layer.input_size_per_partition
    N = layer.output_size_per_partition
    out = torch.empty((M, N), dtype=torch.bfloat16, device=x_scale.device)
    ops.cutlass_int4_fused_grouped_gemm(x_packed, layer.weight_int4, x_scale, layer.weight_scale, out, M, N,
                                        GROUP_SIZE, K // GROUP_SIZE)
    return out if bias is None else out + bias


class W4A4Linear(nn.Module):
    """Drop-in for ``nn.Linear`` whose weight is quantised to int4 at load time.

    ``state_dict`` holds ``weight_int4`` (packed) and ``weight_scale`` once quantised, so a
    quantised layer round-trips through ``torch.save`` / ``load_state_dict`` without
    re-quantising."""

    def __init__(self, in_features: int, out_features: int, bias: bool = False, per_channel: bool | None = None,
                 device=None, dtype=torch.bfloat16):
        super().__init__()
        self.in_features, self.out_features = in_features, out_features
        self.method = W4A4Int4TCLinearMethod(per_channel)
        self.method.create_weights(self, in_features, out_features, dtype, device)
        self.bias = nn.Parameter(torch.zeros(out_features, dtype=dtype, device=device), requires_grad=False) if bias else None
        self.quantized = False

    @classmethod
    def from_linear(cls, lin: nn.Linear, per_channel: bool | None = None) -> "W4A4Linear":
        m = cls(lin.in_features, lin.out_features, lin.bias is not None, per_channel, lin.weight.device, lin.weight.dtype)
        m.weight.data.copy_(lin.weight.data)
        if lin.bias is not None:
            m.bias.data.copy_(lin.bias.data)
        m.quantize_()
        return m

    def quantize_(self) -> "W4A4Linear":
        if not self.quantized:
            self.method.process_weights_after_loading(self)
            self.quantized = True
        return self

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        if not self.quantized:
            self.quantize_()
        return self.method.apply(self, x, self.bias)

    def _load_from_state_dict(self, state_dict, prefix, *args, **kwargs):
        if prefix + "weight_int4" in state_dict and not self.quantized:
            self.weight = None
            self.weight_int4 = nn.Parameter(torch.empty_like(state_dict[prefix + "weight_int4"], device=self._dev()),
                                            requires_grad=False)
            self.weight_scale = nn.Parameter(torch.empty_like(state_dict[prefix + "weight_scale"], device=self._dev()),
                                             requires_grad=False)
            self.quantized = True
        return super()._load_from_state_dict(state_dict, prefix, *args, **kwargs)

    def _dev(self):
        for p in self.parameters():
            return p.device
        return None
