"""The caller side of the op boundary: the two-phase protocol of the reference's vLLM linear
method (``create_weights`` / ``process_weights_after_loading`` / ``apply``; described in
``docs/native_int4_tc_implementation_report.md:515-562``), as plain classes plus an ``nn.Module``.

Mode selection follows the plugin's environment flags (``int4_native_tc/benchmark_all.py:46-59``,
``int4_native_tc/INT4_QUANTIZATION_REPORT.md:796-802``):

* ``INT4TC_PER_CHANNEL=1``: per-token / per-channel scales; otherwise per-group-128 scales (the
  reference's "Enhanced-PG" configuration), refined by
* ``INT4TC_ASYMMETRIC=1``: asymmetric activation codes, zero-point term inside the fused GEMM
  (one quantiser + one GEMM per layer, as ``int4_native_tc/profile_layer.py:83-119``);
* ``INT4TC_CLIP_RATIO=r`` (0 < r <= 1, default 1): outlier clipping of the activation range;
* ``INT4TC_CALIBRATION_STATS=file`` (+ ``INT4TC_SQ_ALPHA``, default 0.5): SmoothQuant factors from the
  collector's statistics file, baked into the weight at load time and divided out of the activations.
"""
from __future__ import annotations

import os

import torch
from torch import nn

from . import ops

GROUP_SIZE = 128


def per_channel_from_env() -> bool:
    return os.environ.get("INT4TC_PER_CHANNEL", "0") == "1"


_STATS_CACHE: dict = {}


def _load_stats(path: str) -> dict:
    if path not in _STATS_CACHE:
        from .calibration import ActivationStatsCollector

        _STATS_CACHE[path] = ActivationStatsCollector.load(path)
    return _STATS_CACHE[path]


class W4A4Int4TCLinearMethod:
    """``process_weights_after_loading`` quantises the bf16 weight once; ``apply`` quantises the
    activations and runs the W4A4 GEMM on every forward.

    Every argument defaults to the plugin's environment flag of the same meaning (module docstring).
    ``calibration_stats`` is a statistics file path or the dict it holds; ``layer_name`` picks this layer's entry."""

    def __init__(self, per_channel: bool | None = None, asymmetric: bool | None = None,
                 clip_ratio: float | None = None, calibration_stats=None, sq_alpha: float | None = None,
                 layer_name: str | None = None):
        env = os.environ
        self.per_channel = per_channel_from_env() if per_channel is None else per_channel
        self.asymmetric = (env.get("INT4TC_ASYMMETRIC", "0") == "1") if asymmetric is None else asymmetric
        self.clip_ratio = float(env.get("INT4TC_CLIP_RATIO", "1.0")) if clip_ratio is None else float(clip_ratio)
        if not (0.0 < self.clip_ratio <= 1.0):
            raise ValueError("clip ratio must be in (0, 1]")
        self.sq_alpha = float(env.get("INT4TC_SQ_ALPHA", "0.5")) if sq_alpha is None else float(sq_alpha)
        if calibration_stats is None:
            calibration_stats = env.get("INT4TC_CALIBRATION_STATS") or None
        self.calibration_stats = calibration_stats
        self.layer_name = layer_name
        if self.per_channel and (self.asymmetric or self.clip_ratio < 1.0 or calibration_stats is not None):
            raise ValueError("asymmetric codes, clipping and SmoothQuant belong to the per-group configuration")

    def _input_absmax(self, K: int):
        st = self.calibration_stats
        if st is None:
            return None
        if isinstance(st, str):
            st = _load_stats(st)
        entry = st.get(self.layer_name) if self.layer_name is not None else None
        if entry is None:
            return None   # a layer the calibration run never saw keeps its weight as it is
        a = entry["input_absmax"] if isinstance(entry, dict) else entry.input_absmax
        if a.numel() != K:
            raise ValueError(f"calibration entry of {self.layer_name!r} has {a.numel()} channels, the layer {K}")
        return a

    def create_weights(self, layer: nn.Module, input_size: int, output_size: int, params_dtype=torch.bfloat16,
                       device=None) -> None:
        layer.weight = nn.Parameter(torch.empty(output_size, input_size, dtype=params_dtype, device=device),
                                    requires_grad=False)
        layer.input_size_per_partition = input_size
        layer.output_size_per_partition = output_size

    def process_weights_after_loading(self, layer: nn.Module) -> None:
        w = layer.weight.data
        layer.smooth_scale = None
        layer.w_col_sum = None
        if self.per_channel:
            packed, scale = ops.static_int4_weight_quant(w)  # [N,K/2], [N]
        else:
            a = self._input_absmax(w.shape[1])
            if a is not None:
                from .calibration import apply_smoothing_to_weight, compute_smoothing_factors

                sm = compute_smoothing_factors(w, a.to(w.device), self.sq_alpha).to(w.dtype)
                w = apply_smoothing_to_weight(w, sm)
                layer.smooth_scale = nn.Parameter(sm.contiguous(), requires_grad=False)
            packed, scale = ops.static_int4_weight_quant_grouped(w.contiguous(), GROUP_SIZE)  # [G,N,64], [G,N]
            if self.asymmetric:
                layer.w_col_sum = nn.Parameter(ops.int4_weight_group_sums(packed), requires_grad=False)
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
        elif self.asymmetric:
            sm = getattr(layer, "smooth_scale", None)
            xp, xs, azp = ops.dynamic_int4_quant_asymmetric_clipped_grouped(
                x2d, GROUP_SIZE, self.clip_ratio, None if sm is None else sm.to(x2d.dtype))
            ops.cutlass_int4_fused_grouped_gemm_azp(xp, layer.weight_int4, xs, layer.weight_scale, out, azp,
                                                    layer.w_col_sum, M, N, GROUP_SIZE, K // GROUP_SIZE)
        else:
            sm = getattr(layer, "smooth_scale", None)
            if sm is not None:
                x2d = x2d / sm.to(x2d.dtype)
            if self.clip_ratio < 1.0:
                xp, xs = ops.dynamic_int4_quant_clipped_grouped(x2d, GROUP_SIZE, self.clip_ratio)
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
                 device=None, dtype=torch.bfloat16, **method_kwargs):
        super().__init__()
        self.in_features, self.out_features = in_features, out_features
        self.method = W4A4Int4TCLinearMethod(per_channel, **method_kwargs)
        self.smooth_scale = None
        self.w_col_sum = None
        self.method.create_weights(self, in_features, out_features, dtype, device)
        self.bias = nn.Parameter(torch.zeros(out_features, dtype=dtype, device=device), requires_grad=False) if bias else None
        self.quantized = False

    @classmethod
    def from_linear(cls, lin: nn.Linear, per_channel: bool | None = None, **method_kwargs) -> "W4A4Linear":
        m = cls(lin.in_features, lin.out_features, lin.bias is not None, per_channel, lin.weight.device,
                lin.weight.dtype, **method_kwargs)
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
            dev = self._dev()   # read before the bf16 weight goes: it may be this module's only parameter
            self.weight = None
            for name in ("weight_int4", "weight_scale", "smooth_scale", "w_col_sum"):
                if prefix + name in state_dict:
                    setattr(self, name, nn.Parameter(torch.empty_like(state_dict[prefix + name], device=dev),
                                                     requires_grad=False))
            self.quantized = True
        return super()._load_from_state_dict(state_dict, prefix, *args, **kwargs)

    def _dev(self):
        for p in self.parameters():
            return p.device
        return None
