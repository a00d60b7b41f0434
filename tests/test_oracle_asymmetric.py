"""CPU: the oracle's asymmetric / clipped quantisers and zero-point linear against independent restatements
(torch fp32 for the quantiser, float64 for the linear), and the new C-ABI entry points' argument checks."""
import numpy as np
import torch

from oracle import w4a4_oracle as O


def _acts(M, K, seed, shift=0.6):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(M, K, generator=g) * 1.5 + shift
    x[:, ::97] *= 6.0
    if M > 2:
        x[1] = 0.0
        x[2] = 3.25
    return x.to(torch.bfloat16)


def _torch_asymmetric(x, gs, clip, smooth):
    """The reference's torch formulation of asymmetric quantisation (test_enhanced_quantization.py:262-268:
    scale = range / qmax, azp = round(-min / scale), q = round(x / scale + azp).clamp(0, qmax)), applied per
    (row, group) with qmax = 15, the kernel's scale floor, clipping and smoothing (int4_quant.cu:1353-1419)."""
    v = x.float()
    if smooth is not None:
        v = v / smooth.float()[None, :]
    M, K = v.shape
    v = v.reshape(M, K // gs, gs).permute(1, 0, 2)
    t = v.abs().amax(dim=2, keepdim=True) * torch.tensor(clip, dtype=torch.float32)
    c = torch.minimum(torch.maximum(v, -t), t)
    mn, mx = c.amin(dim=2, keepdim=True), c.amax(dim=2, keepdim=True)
    scale = ((mx - mn) / 15.0).clamp(min=float(O.K_MIN_SCALE))
    azp = torch.round(-mn / scale).clamp(0, 15)
    q = torch.round(c / scale + azp).clamp(0, 15)
    return (q - 8).to(torch.int8).numpy(), scale[..., 0].numpy(), (8.0 - azp)[..., 0].numpy()


def test_asymmetric_matches_torch_restatement():
    for (M, K, gs, clip, use_smooth) in [(7, 512, 128, 1.0, False), (19, 2048, 128, 0.9, False),
                                         (9, 1024, 256, 0.8, True), (5, 256, 64, 1.0, True)]:
        x = _acts(M, K, seed=M + K)
        sm = None
        if use_smooth:
            sm = (torch.rand(K, generator=torch.Generator().manual_seed(3)) * 1.5 + 0.25).to(torch.bfloat16)
        codes, s, adj = O.quant_asymmetric_grouped(x, gs, clip, sm)
        tc, ts, ta = _torch_asymmetric(x, gs, clip, sm)
        np.testing.assert_array_equal(codes, tc)
        np.testing.assert_array_equal(s, ts)
        np.testing.assert_array_equal(adj, ta)


def test_asymmetric_properties():
    x = _acts(33, 1024, seed=2)
    codes, s, adj = O.quant_asymmetric_grouped(x, 128)
    assert codes.min() >= -8 and codes.max() <= 7
    assert adj.min() >= -7 and adj.max() <= 8 and np.all(adj == np.rint(adj))
    xg = O._grouped_view(x, 128)
    deq = (codes.astype(np.float32) + adj[:, :, None]) * s[:, :, None]
    live = (xg.max(axis=2) - xg.min(axis=2)) / 15.0 >= O.K_MIN_SCALE      # groups whose scale is not the floor
    err = np.abs(deq - xg).max(axis=2)
    # zero-point rounding can push the extreme values half a step past the grid: error <= one step there
    assert np.all(err[live] <= s[live] * 1.0001)
    assert np.median(err[live] / s[live]) <= 0.51
    # the all-zero row dequantises to exactly zero
    assert np.all(deq[:, 1, :] == 0.0)


def test_clipped_properties():
    x = _acts(17, 1024, seed=5)
    c1, s1 = O.quant_clipped_grouped(x, 128, 1.0)
    c0, s0 = O.quant_grouped(x, 128)
    np.testing.assert_array_equal(c1, c0)
    np.testing.assert_array_equal(s1, s0)
    c9, s9 = O.quant_clipped_grouped(x, 128, 0.9)
    assert np.all(s9 <= s1) and c9.min() >= -8 and c9.max() <= 7
    # the outliers saturate, everything inside the clipped range is within half a step
    xg = O._grouped_view(x, 128)
    inside = np.abs(xg) <= (np.abs(xg).max(axis=2) * np.float32(0.9))[:, :, None]
    live = (s9 > O.K_MIN_SCALE)[:, :, None] & inside
    err = np.abs(c9.astype(np.float32) * s9[:, :, None] - xg)
    assert np.all(err[live] <= (np.broadcast_to(s9[:, :, None], err.shape)[live]) * 0.5001)


def test_zero_point_linear_algebra():
    rng = np.random.RandomState(0)
    G, M, N = 4, 9, 13
    a = rng.randint(-8, 8, size=(G, M, 128)).astype(np.int8)
    b = rng.randint(-8, 8, size=(G, N, 128)).astype(np.int8)
    sa = rng.uniform(0.01, 0.1, size=(G, M)).astype(np.float32)
    sb = rng.uniform(0.01, 0.1, size=(G, N)).astype(np.float32)
    adj = rng.randint(-7, 9, size=(G, M)).astype(np.float32)
    wcs = O.weight_group_sums(b)
    np.testing.assert_array_equal(wcs, b.astype(np.int64).sum(axis=2).astype(np.float32))
    f = O.linear_grouped_azp_f32(a, b, sa, sb, adj, wcs)
    # (codes + azp_adj) are the zero-point-corrected activations: the linear of those, in float64
    a64 = a.astype(np.float64) + adj.astype(np.float64)[:, :, None]
    ref = np.zeros((M, N))
    for g in range(G):
        ref += (a64[g] @ b[g].astype(np.float64).T) * sa[g].astype(np.float64)[:, None] * sb[g].astype(np.float64)[None, :]
    np.testing.assert_allclose(f, ref, rtol=1e-5, atol=1e-5 * np.abs(ref).max())
    # azp_adj = 0 is the symmetric linear, bit for bit
    np.testing.assert_array_equal(O.linear_grouped_azp_f32(a, b, sa, sb, np.zeros_like(adj), wcs),
                                  O.linear_grouped_f32(a, b, sa, sb))


def test_new_entry_points_reject_bad_arguments(lib_built):
    from fp8_inference_toolkit_b200 import _cabi

    lib = _cabi.lib
    # rejected before any CUDA call
    assert lib.i4tc_quant_asymmetric_grouped(None, 0, 4, 256, 256, 32, 1.0, None, None, None, None, 0, None) == -3
    assert "group_size" in _cabi.last_error()
    assert lib.i4tc_quant_asymmetric_grouped(None, 0, 4, 256, 256, 128, 1.5, None, None, None, None, 0, None) == -1
    assert "clip_ratio" in _cabi.last_error()
    assert lib.i4tc_quant_clipped_grouped(None, 0, 4, 200, 200, 128, 1.0, None, None, 0, None) == -1
    assert "divisible" in _cabi.last_error()
    assert lib.i4tc_gemm_grouped_azp(None, None, None, None, None, None, None, 4, 4, 64, 2, 0, None) == -3
    assert lib.i4tc_weight_group_sums(None, 4, 12, None, 0, None) == -1
    assert lib.i4tc_weight_group_sums(None, 0, 128, None, 0, None) == 0
