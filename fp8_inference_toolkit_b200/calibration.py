"""Calibration hooks: running per-input-channel absmax of every ``nn.Linear`` and the SmoothQuant
factor arithmetic.  Same public names, arguments and file format as the reference's
``int4_native_tc/calibration/collector.py:17-102`` and ``calibration/smoothquant.py:19-64``; pure
PyTorch (these run once, offline, on any device)."""
from __future__ import annotations

from dataclasses import dataclass

import torch
from torch import nn

_FLOOR = 1e-5


@dataclass
class LayerStats:
    """Statistics of one linear layer: ``input_absmax`` [K], ``weight_absmax`` [K], rows seen so far."""

    input_absmax: torch.Tensor
    weight_absmax: torch.Tensor
    num_samples: int


class ActivationStatsCollector:
    """Registers a forward-pre-hook on every ``nn.Linear`` of ``model`` and keeps, per layer, the
    element-wise maximum over all calls of ``|x|`` reduced over tokens."""

    def __init__(self, model: nn.Module) -> None:
        self.stats: dict[str, LayerStats] = {}
        self._hooks = []
        self._register_hooks(model)

    def _register_hooks(self, model: nn.Module) -> None:
        for name, mod in model.named_modules():
            if isinstance(mod, nn.Linear):
                self._hooks.append(mod.register_forward_pre_hook(self._make_hook(name)))

    def _make_hook(self, name: str):
        def hook(module, args):
            self._collect(name, module, args)

        return hook

    def _collect(self, name: str, module: nn.Module, input) -> None:
        x = input[0].detach()
        x = x.reshape(-1, x.shape[-1])
        cur = x.abs().amax(dim=0).float()
        st = self.stats.get(name)
        if st is None:
            w = getattr(module, "weight", None)
            w_absmax = w.detach().abs().amax(dim=0).float() if w is not None else torch.zeros_like(cur)
            self.stats[name] = LayerStats(cur, w_absmax, x.shape[0])
        else:
            st.input_absmax = torch.maximum(st.input_absmax, cur)
            st.num_samples += x.shape[0]

    def remove_hooks(self) -> None:
        for h in self._hooks:
            h.remove()
        self._hooks.clear()

    def save(self, path: str) -> None:
        """``torch.save`` of ``{layer: {"input_absmax", "weight_absmax", "num_samples"}}`` (CPU tensors)."""
        torch.save({k: {"input_absmax": v.input_absmax.cpu(), "weight_absmax": v.weight_absmax.cpu(),
                        "num_samples": v.num_samples} for k, v in self.stats.items()}, path)

    @staticmethod
    def load(path: str) -> dict:
        return torch.load(path, weights_only=False)


def compute_smoothing_factors(weight: torch.Tensor, input_absmax: torch.Tensor, alpha: float = 0.5) -> torch.Tensor:
    """``s_j = a_j**alpha / w_j**(1-alpha)`` with ``a`` the calibrated activation absmax and ``w`` the
    per-input-channel weight absmax, both floored at 1e-5, as is the result."""
    w = weight.detach().float().abs().amax(dim=0).clamp(min=_FLOOR)
    a = input_absmax.float().clamp(min=_FLOOR)
    return (a.pow(alpha) / w.pow(1.0 - alpha)).clamp(min=_FLOOR)


def apply_smoothing_to_weight(weight: torch.Tensor, smooth_scale: torch.Tensor) -> torch.Tensor:
    """``W * diag(s)``: column ``j`` of ``W`` [N,K] times ``s_j``; activations are divided by ``s`` at run time."""
    return weight * smooth_scale.to(weight.dtype).unsqueeze(0)
