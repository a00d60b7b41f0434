"""GPU: the caller side of the boundary -- W4A4Linear (two-phase protocol, state_dict round trip) and the
Qwen3-shaped prefill harness on a tiny configuration."""
import numpy as np
import pytest
import torch

from oracle import w4a4_oracle as O

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("per_channel", [False, True])
def test_linear_module_matches_oracle(per_channel):
    from fp8_inference_toolkit_b200 import synthetic
    from fp8_inference_toolkit_b200.linear import W4A4Linear

    K, N, M = 512, 384, 40
    w = synthetic.weights(N, K, 3)
    x = synthetic.activations(M, K, 4)
    lin = torch.nn.Linear(K, N, bias=True, dtype=torch.bfloat16)
    lin.weight.data.copy_(w)
    lin.bias.data.copy_(torch.randn(N, generator=torch.Generator().manual_seed(5)) * 0.1)
    q = W4A4Linear.from_linear(lin.cuda(), per_channel=per_channel)
    assert q.weight is None and q.weight_int4.dtype == torch.uint8
    y = q(x.cuda().view(2, 20, K))
    assert y.shape == (2, 20, N) and y.dtype == torch.bfloat16
    if per_channel:
        xc, xs = O.quant_rowwise(x, "activation")
        wc, ws = O.quant_rowwise(w, "weight")
        ref = O.linear_per_channel(xc, wc, xs, ws)
    else:
        xc, xs = O.quant_grouped(x, 128, "activation")
        wc, ws = O.quant_grouped(w, 128, "weight")
        ref = O.linear_grouped(xc, wc, xs, ws)
    # the bias can cancel the product almost completely, so the error is bounded relative to the two addends
    # (1e-2 of the north star applied to the GEMM output, plus the helper's floor), not to their sum
    g, bias = ref.float(), lin.bias.data.float().cpu()
    full = (g + bias).to(torch.bfloat16).float()
    bound = 1e-2 * (g.abs() + bias.abs()) + 1e-3 * g.abs().max()
    err = (y.view(M, N).float().cpu() - full).abs()
    assert (err <= bound).all(), f"W4A4Linear: worst error / bound = {(err / bound).max():.3f}"
    # state_dict round trip keeps the packed weight; no re-quantisation, identical output
    sd = {k: v.cpu() for k, v in q.state_dict().items()}
    assert set(sd) == {"weight_int4", "weight_scale", "bias"}
    q2 = W4A4Linear(K, N, bias=True, per_channel=per_channel, device="cuda")
    q2.load_state_dict(sd)
    assert q2.quantized and torch.equal(q2(x.cuda()), q(x.cuda()))


@pytest.mark.parametrize("flags", [
    {"INT4TC_ASYMMETRIC": "1"},
    {"INT4TC_CLIP_RATIO": "0.95"},
    {"INT4TC_ASYMMETRIC": "1", "INT4TC_CLIP_RATIO": "0.95"},
    {"INT4TC_CALIBRATION_STATS": "file"},
    {"INT4TC_ASYMMETRIC": "1", "INT4TC_CLIP_RATIO": "0.95", "INT4TC_CALIBRATION_STATS": "file", "INT4TC_SQ_ALPHA": "0.6"},
])
def test_linear_module_enhanced_flags_match_oracle(monkeypatch, tmp_path, flags):
    """The plugin's environment flags (asymmetric codes, clipping, SmoothQuant from a statistics file) reach the
    kernels through W4A4Linear, one quantiser + one GEMM per forward, and each combination equals the oracle's
    composition bit for bit (M > 128: the unsplit tensor-core path)."""
    from fp8_inference_toolkit_b200 import synthetic
    from fp8_inference_toolkit_b200.calibration import ActivationStatsCollector, apply_smoothing_to_weight, compute_smoothing_factors
    from fp8_inference_toolkit_b200.linear import W4A4Linear

    K, N, M = 512, 384, 160
    w = synthetic.weights(N, K, 3)
    x = (synthetic.activations(M, K, 4).float() + 0.75).to(torch.bfloat16)    # shifted: the asymmetric case
    lin = torch.nn.Linear(K, N, bias=False, dtype=torch.bfloat16)
    lin.weight.data.copy_(w)
    stats_file = None
    if "INT4TC_CALIBRATION_STATS" in flags:
        holder = torch.nn.Sequential()
        holder.add_module("proj", lin)
        col = ActivationStatsCollector(holder)
        holder(x)
        col.remove_hooks()
        stats_file = str(tmp_path / "calib.pt")
        col.save(stats_file)
    for k, v in flags.items():
        monkeypatch.setenv(k, stats_file if v == "file" else v)
    q = W4A4Linear.from_linear(lin.cuda(), layer_name="proj")
    y = q(x.cuda())
    asym = flags.get("INT4TC_ASYMMETRIC") == "1"
    clip = float(flags.get("INT4TC_CLIP_RATIO", "1.0"))
    wq, sm = w, None
    if stats_file is not None:
        a = x.abs().amax(dim=0).float()
        sm = compute_smoothing_factors(w, a, float(flags.get("INT4TC_SQ_ALPHA", "0.5"))).to(torch.bfloat16)
        wq = apply_smoothing_to_weight(w, sm)
        assert torch.equal(q.smooth_scale.cpu(), sm)
    wc, ws = O.quant_grouped(wq, 128, "weight")
    assert np.array_equal(q.weight_int4.cpu().numpy(), O.pack_int4(wc))
    if asym:
        xc, xs, adj = O.quant_asymmetric_grouped(x, 128, clip, sm)
        wcs = O.weight_group_sums(wc)
        assert np.array_equal(q.w_col_sum.cpu().numpy(), wcs)
        ref = O.to_bf16(O.linear_grouped_azp_f32(xc, wc, xs, ws, adj, wcs))
    else:
        xin = x if sm is None else (x / sm)
        xc, xs = O.quant_clipped_grouped(xin, 128, clip) if clip < 1.0 else O.quant_grouped(xin, 128, "activation")
        ref = O.linear_grouped(xc, wc, xs, ws)
    assert torch.equal(y.cpu(), ref)
    sd = {k: v.cpu() for k, v in q.state_dict().items()}     # CPU tensors, as after torch.load
    q2 = W4A4Linear(K, N, layer_name="proj", device="cuda")
    q2.load_state_dict(sd)
    assert q2.weight_int4.is_cuda and torch.equal(q2(x.cuda()), y)


def test_env_flag_selects_mode(monkeypatch):
    from fp8_inference_toolkit_b200.linear import W4A4Int4TCLinearMethod

    monkeypatch.setenv("INT4TC_PER_CHANNEL", "1")
    assert W4A4Int4TCLinearMethod().per_channel
    monkeypatch.setenv("INT4TC_PER_CHANNEL", "0")
    assert not W4A4Int4TCLinearMethod().per_channel


def test_tiny_qwen3_prefill_runs():
    from fp8_inference_toolkit_b200 import ops
    from fp8_inference_toolkit_b200.qwen3 import Qwen3Config, Qwen3Prefill

    cfg = Qwen3Config(hidden=256, layers=2, q_heads=4, kv_heads=2, head_dim=64, inter=512, vocab=1000)
    m = Qwen3Prefill(cfg, "cuda")
    ids = torch.randint(0, cfg.vocab, (3, 40), device="cuda")
    y = m(ids)
    ops.check_status()
    assert y.shape == (3, 40, 256) and torch.isfinite(y.float()).all()
    assert torch.equal(y, m(ids))  # deterministic
    # causality: changing a later token leaves earlier positions untouched
    ids2 = ids.clone()
    ids2[:, -1] = (ids2[:, -1] + 1) % cfg.vocab
    assert torch.equal(m(ids2)[:, :-1], y[:, :-1])
    # the fused quantisers (RMSNorm + quantise, SwiGLU + quantise) follow the plain path closely
    m_plain = Qwen3Prefill(cfg, "cuda", fused=False)
    m_plain.embed.load_state_dict(m.embed.state_dict())   # the linears are seeded, the embedding table is not
    y_plain = m_plain(ids)
    cos = torch.nn.functional.cosine_similarity(y.float().flatten(), y_plain.float().flatten(), dim=0).item()
    assert cos > 0.995, cos
