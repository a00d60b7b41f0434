"""CPU: calibration hooks (collector shapes / accumulation / save-load, SmoothQuant algebra), in the
spirit of the reference's ``test_enhanced_quantization.py:113-242``."""
import torch
from torch import nn

from int4_native_tc.calibration import (ActivationStatsCollector, LayerStats, apply_smoothing_to_weight,
                                        compute_smoothing_factors)


class Tiny(nn.Module):
    def __init__(self):
        super().__init__()
        self.a = nn.Linear(16, 32, bias=False)
        self.b = nn.Linear(32, 8)

    def forward(self, x):
        return self.b(torch.relu(self.a(x)))


def test_collector_shapes_accumulate_and_remove(tmp_path):
    torch.manual_seed(0)
    m = Tiny()
    c = ActivationStatsCollector(m)
    x1 = torch.randn(4, 5, 16)
    x2 = torch.randn(3, 16) * 3
    m(x1)
    m(x2)
    assert set(c.stats) == {"a", "b"}
    st = c.stats["a"]
    assert isinstance(st, LayerStats) and st.input_absmax.shape == (16,) and st.weight_absmax.shape == (16,)
    assert st.num_samples == 23
    want = torch.maximum(x1.reshape(-1, 16).abs().amax(0), x2.abs().amax(0))
    assert torch.equal(st.input_absmax, want)
    assert torch.equal(st.weight_absmax, m.a.weight.abs().amax(0))
    p = tmp_path / "stats.pt"
    c.save(str(p))
    d = ActivationStatsCollector.load(str(p))
    assert torch.equal(d["b"]["input_absmax"], c.stats["b"].input_absmax) and d["a"]["num_samples"] == 23
    c.remove_hooks()
    m(torch.randn(2, 16) * 100)
    assert c.stats["a"].num_samples == 23


def test_smoothquant_invariance_and_range():
    torch.manual_seed(1)
    X = torch.randn(64, 48)
    X[:, 3] *= 30
    W = torch.randn(20, 48) * 0.05
    s = compute_smoothing_factors(W, X.abs().amax(0), 0.5)
    assert s.shape == (48,) and (s > 0).all()
    Ws = apply_smoothing_to_weight(W, s)
    assert torch.allclose((X / s) @ Ws.T, X @ W.T, atol=1e-4)
    assert (X / s).abs().max() < X.abs().max()  # the outlier channel is tamed
    # alpha = 0 leaves activations to the weights' scale only; zero inputs hit the floors, not NaN
    s0 = compute_smoothing_factors(torch.zeros(4, 8), torch.zeros(8), 0.5)
    assert torch.isfinite(s0).all() and (s0 >= 1e-5).all()
    assert apply_smoothing_to_weight(W.to(torch.bfloat16), s).dtype == torch.bfloat16
