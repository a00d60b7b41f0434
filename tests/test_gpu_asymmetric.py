"""GPU parity of the clipped / asymmetric / smoothed activation quantisers and of the zero-point GEMM against the
CPU oracle, through the reference-named ops (the reference's cases: test_enhanced_quantization.py:252-285,
profile_layer.py:96-119)."""
import numpy as np
import pytest
import torch

from oracle import w4a4_oracle as O
from tests.helpers import assert_close_bf16, dev_f32, dev_packed, rand_codes

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def tc():
    import int4_native_tc

    return int4_native_tc


def _acts(M, K, seed, dtype=torch.bfloat16, shift=0.6):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(M, K, generator=g) * 1.5 + shift
    x[:, ::97] *= 6.0          # a few outliers per row, the case clipping is for
    if M > 2:
        x[1] = 0.0             # an all-zero row
        x[2] = 3.25            # a constant row (zero range)
    return x.to(dtype)


def _codes_of(packed: torch.Tensor) -> np.ndarray:
    return O.unpack_int4(packed.cpu().numpy())


@pytest.mark.parametrize("M,K,gs", [(1, 128, 128), (7, 512, 128), (33, 4096, 128), (5, 256, 64), (9, 1024, 256)])
@pytest.mark.parametrize("clip", [1.0, 0.85])
def test_clipped_grouped_bit_exact(tc, M, K, gs, clip):
    x = _acts(M, K, seed=M * 131 + K)
    packed, scale = tc.dynamic_int4_quant_clipped_grouped(x.cuda(), gs, clip)
    codes, s = O.quant_clipped_grouped(x, gs, clip)
    assert packed.shape == (K // gs, M, gs // 2) and scale.shape == (K // gs, M)
    np.testing.assert_array_equal(scale.cpu().numpy(), s)
    np.testing.assert_array_equal(_codes_of(packed), codes)


def test_clip_one_matches_plain_grouped(tc):
    x = _acts(17, 1024, seed=5).cuda()
    p0, s0 = tc.dynamic_int4_quant_grouped(x, 128)
    p1, s1 = tc.dynamic_int4_quant_clipped_grouped(x, 128, 1.0)
    assert torch.equal(p0, p1) and torch.equal(s0, s1)


@pytest.mark.parametrize("M,K,gs", [(1, 128, 128), (7, 512, 128), (33, 4096, 128), (5, 256, 64), (9, 1024, 256)])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_asymmetric_grouped_bit_exact(tc, M, K, gs, dtype):
    x = _acts(M, K, seed=M * 17 + K, dtype=dtype)
    packed, scale, adj = tc.dynamic_int4_quant_asymmetric_grouped(x.cuda(), gs)
    codes, s, a = O.quant_asymmetric_grouped(x, gs)
    np.testing.assert_array_equal(scale.cpu().numpy(), s)
    np.testing.assert_array_equal(adj.cpu().numpy(), a)
    np.testing.assert_array_equal(_codes_of(packed), codes)


@pytest.mark.parametrize("clip,smooth", [(0.9, False), (1.0, True), (0.8, True)])
def test_asymmetric_clipped_smoothed_bit_exact(tc, clip, smooth):
    M, K = 19, 2048
    x = _acts(M, K, seed=77)
    sm = None
    if smooth:
        g = torch.Generator().manual_seed(3)
        sm = (torch.rand(K, generator=g) * 1.5 + 0.25).to(torch.bfloat16)
    packed, scale, adj = tc.dynamic_int4_quant_asymmetric_clipped_grouped(x.cuda(), 128, clip,
                                                                          sm.cuda() if smooth else None)
    codes, s, a = O.quant_asymmetric_grouped(x, 128, clip, sm)
    np.testing.assert_array_equal(scale.cpu().numpy(), s)
    np.testing.assert_array_equal(adj.cpu().numpy(), a)
    np.testing.assert_array_equal(_codes_of(packed), codes)


def test_asymmetric_strided_rows(tc):
    big = _acts(12, 1024 + 64, seed=9).cuda()
    x = big[:, :1024]                       # row stride 1088 elements
    packed, scale, adj = tc.dynamic_int4_quant_asymmetric_grouped(x, 128)
    codes, s, a = O.quant_asymmetric_grouped(x.cpu(), 128)
    np.testing.assert_array_equal(_codes_of(packed), codes)
    np.testing.assert_array_equal(scale.cpu().numpy(), s)


def _adversarial(M, K, seed, dtype):
    """Rows that stress the rounding decisions: lattice values (exact ties), a large offset with a tiny range, huge and
    tiny magnitudes, one-sided rows."""
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(M, K, generator=g)
    x[0] = torch.randint(-30, 31, (K,), generator=g).float() * 0.25          # quarter lattice: ties everywhere
    x[1] = 100.0 + torch.randint(0, 4, (K,), generator=g).float() * 0.5      # offset >> range
    x[2] = torch.randint(0, 16, (K,), generator=g).float()                   # already codes 0..15
    x[3] = torch.rand(K, generator=g) * 1e-6                                 # below the scale floor
    x[4] = torch.randn(K, generator=g) * 1e4                                 # large
    x[5] = -torch.rand(K, generator=g) * 7.0                                 # one-sided negative
    x[6] = torch.randint(-7, 8, (K,), generator=g).float() * 0.5 + 0.5       # half-integers
    x[7, ::2] = 0.0
    return x.to(dtype)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("gs,clip", [(128, 1.0), (128, 0.7), (64, 0.1), (256, 0.95)])
def test_quantisers_adversarial_both_kernels(tc, dtype, gs, clip):
    """The 128-bit kernel (aligned rows) and the general one (rows that start 8 bytes off) give the oracle's codes on
    rows built to sit on rounding boundaries."""
    M, K = 24, 2048
    x = _adversarial(M, K, seed=gs + int(clip * 100), dtype=dtype)
    codes, s, a = O.quant_asymmetric_grouped(x, gs, clip)
    ccodes, cs = O.quant_clipped_grouped(x, gs, clip)
    wide = torch.zeros(M, K + 8, dtype=dtype, device="cuda")
    wide[:, 4:K + 4] = x.cuda()
    for xin in (x.cuda(), wide[:, 4:K + 4]):
        packed, scale, adj = tc.dynamic_int4_quant_asymmetric_clipped_grouped(xin, gs, clip, None)
        np.testing.assert_array_equal(scale.cpu().numpy(), s)
        np.testing.assert_array_equal(adj.cpu().numpy(), a)
        np.testing.assert_array_equal(_codes_of(packed), codes)
        packed, scale = tc.dynamic_int4_quant_clipped_grouped(xin, gs, clip)
        np.testing.assert_array_equal(scale.cpu().numpy(), cs)
        np.testing.assert_array_equal(_codes_of(packed), ccodes)


def test_asymmetric_argument_checks(tc):
    x = torch.zeros(4, 256, dtype=torch.bfloat16, device="cuda")
    with pytest.raises(RuntimeError, match="clip_ratio"):
        tc.dynamic_int4_quant_asymmetric_clipped_grouped(x, 128, 1.5)
    with pytest.raises(RuntimeError, match="divisible"):
        tc.dynamic_int4_quant_clipped_grouped(x, 96, 1.0)
    with pytest.raises(RuntimeError, match="group_size"):
        tc.dynamic_int4_quant_asymmetric_grouped(x, 32)


def test_weight_group_sums_exact(tc):
    rng = np.random.RandomState(4)
    codes = rand_codes(rng, (3, 50, 128))
    out = tc.int4_weight_group_sums(dev_packed(codes))
    np.testing.assert_array_equal(out.cpu().numpy(), O.weight_group_sums(codes))


@pytest.mark.parametrize("M,N,G", [(1, 256, 2), (5, 130, 3), (48, 384, 4), (100, 512, 8), (300, 200, 3),
                                   (520, 768, 4), (1024, 1024, 8), (1536, 2048, 16)])
def test_grouped_gemm_azp_matches_oracle(tc, M, N, G):
    rng = np.random.RandomState(M * 7 + N + G)
    a = rand_codes(rng, (G, M, 128))
    b = rand_codes(rng, (G, N, 128))
    sa = rng.uniform(0.01, 0.1, size=(G, M)).astype(np.float32)
    sb = rng.uniform(0.01, 0.1, size=(G, N)).astype(np.float32)
    adj = rng.randint(-7, 9, size=(G, M)).astype(np.float32)
    wcs = O.weight_group_sums(b)
    ref = O.to_bf16(O.linear_grouped_azp_f32(a, b, sa, sb, adj, wcs))
    out = torch.empty(M, N, dtype=torch.bfloat16, device="cuda")
    tc.cutlass_int4_fused_grouped_gemm_azp(dev_packed(a), dev_packed(b), dev_f32(sa), dev_f32(sb), out,
                                           dev_f32(adj), dev_f32(wcs), M, N, 128, G)
    torch.cuda.synchronize()
    assert_close_bf16(out, ref, f"azp {M}x{N}x{G}")
    o = out.float().cpu().numpy()
    r = ref.float().numpy()
    if M > 128:
        # the zero-point term enters each group's integer sum before the scales, as in the reference's epilogue:
        # the oracle's operations in the oracle's order, hence the same bits
        assert np.array_equal(o, r)
    else:
        # small M: K ranges summed afterwards (another order of fp32 additions): at most one bf16 step apart
        assert (o != r).mean() < 0.02
        np.testing.assert_allclose(o, r, rtol=2.0 ** -7, atol=1e-3 * np.abs(r).max())


def test_azp_zero_adjust_equals_symmetric(tc):
    """azp_adj = 0 makes the zero-point term vanish: same bits as the symmetric fused linear."""
    rng = np.random.RandomState(11)
    M, N, G = 200, 384, 4
    a, b = rand_codes(rng, (G, M, 128)), rand_codes(rng, (G, N, 128))
    sa = dev_f32(rng.uniform(0.01, 0.1, size=(G, M)))
    sb = dev_f32(rng.uniform(0.01, 0.1, size=(G, N)))
    ap, bp = dev_packed(a), dev_packed(b)
    o0 = torch.empty(M, N, dtype=torch.bfloat16, device="cuda")
    o1 = torch.empty_like(o0)
    tc.cutlass_int4_fused_grouped_gemm(ap, bp, sa, sb, o0, M, N, 128, G)
    tc.cutlass_int4_fused_grouped_gemm_azp(ap, bp, sa, sb, o1, torch.zeros(G, M, device="cuda"),
                                           tc.int4_weight_group_sums(bp), M, N, 128, G)
    assert torch.equal(o0, o1)


def test_asymmetric_linear_end_to_end(tc):
    """Quantise -> zero-point GEMM reproduces x @ W^T better than the symmetric path on shifted activations
    (the reason the reference has the path: test_enhanced_quantization.py:287-316)."""
    M, K, N = 256, 1024, 512
    g = torch.Generator().manual_seed(21)
    x = (torch.rand(M, K, generator=g) * 4.0 + 0.5).to(torch.bfloat16).cuda()   # all positive
    w = (torch.randn(N, K, generator=g) * 0.05).to(torch.bfloat16).cuda()
    bp, sb = tc.static_int4_weight_quant_grouped(w, 128)
    wdq = torch.from_numpy(O.unpack_int4(bp.cpu().numpy())).float() * sb.cpu()[:, :, None]      # [G,N,128]
    exact = x.float().cpu() @ wdq.permute(1, 0, 2).reshape(N, K).T
    G = K // 128
    ap, sa, adj = tc.dynamic_int4_quant_asymmetric_grouped(x, 128)
    out = torch.empty(M, N, dtype=torch.bfloat16, device="cuda")
    tc.cutlass_int4_fused_grouped_gemm_azp(ap, bp, sa, sb, out, adj, tc.int4_weight_group_sums(bp), M, N, 128, G)
    sp, ss = tc.dynamic_int4_quant_grouped(x, 128)
    out_s = torch.empty_like(out)
    tc.cutlass_int4_fused_grouped_gemm(sp, bp, ss, sb, out_s, M, N, 128, G)
    e_asym = (out.float().cpu() - exact).norm() / exact.norm()
    e_sym = (out_s.float().cpu() - exact).norm() / exact.norm()
    assert e_asym < 0.9 * e_sym, (float(e_asym), float(e_sym))
