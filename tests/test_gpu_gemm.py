"""GPU parity: the tcgen05 W4A4 GEMM against the CPU oracle.  int32 accumulators are compared bit
for bit; bf16 outputs within 1e-2 relative and cosine >= 0.9999 (per-channel outputs are in fact
compared bit for bit as well, since the epilogue uses the oracle's multiplication order)."""
import os

import numpy as np
import pytest
import torch

from oracle import w4a4_oracle as O
from tests.helpers import assert_close_bf16, dev_f32, dev_packed, rand_codes

pytestmark = pytest.mark.gpu

TUNINGS = [(0, -1), (64, 1), (128, 1), (64, 0), (128, 0), (256, 0)]


@pytest.fixture(scope="module")
def tc():
    import int4_native_tc

    return int4_native_tc


@pytest.fixture()
def ops():
    from fp8_inference_toolkit_b200 import ops as _ops

    yield _ops
    _ops.set_tuning(0, -1)
    _ops.check_status()


@pytest.mark.parametrize("tile_n,swap", TUNINGS)
def test_kat_small(tc, ops, golden_dir, tile_n, swap):
    z = np.load(os.path.join(golden_dir, "kat_gemm_4x128x8.npz"))
    ops.set_tuning(tile_n, swap)
    out = tc.cutlass_int4_gemm(torch.from_numpy(z["a_packed"]).cuda(), torch.from_numpy(z["b_packed"]).cuda(), 4, 8, 128)
    ops.check_status()
    assert out.dtype == torch.int32 and out.shape == (4, 8)
    assert np.array_equal(out.cpu().numpy(), z["c"])


@pytest.mark.parametrize("tile_n,swap", TUNINGS)
def test_kat_llm_size(tc, ops, golden_dir, tile_n, swap):
    z = np.load(os.path.join(golden_dir, "kat_gemm_16x2560x2560.npz"))
    rng = np.random.RandomState(int(z["seed"]))
    a = rng.randint(-8, 8, size=(16, 2560)).astype(np.int8)
    b = rng.randint(-8, 8, size=(2560, 2560)).astype(np.int8)
    ops.set_tuning(tile_n, swap)
    out = tc.cutlass_int4_gemm(dev_packed(a), dev_packed(b), 16, 2560, 2560)
    ops.check_status()
    assert np.array_equal(out.cpu().numpy(), z["c"])


@pytest.mark.parametrize("M,N,K", [(1, 8, 64), (17, 100, 192), (128, 256, 128), (129, 1000, 2560),
                                   (300, 257, 320), (1, 4096, 4096), (513, 72, 12288), (40, 24, 65536)])
def test_int32_ragged_exact(tc, ops, M, N, K):
    rng = np.random.RandomState(M * 7 + N * 3 + K)
    a, b = rand_codes(rng, (M, K)), rand_codes(rng, (N, K))
    ref = O.int_gemm(a, b) if K * 64 < (1 << 24) else (a.astype(np.int64) @ b.astype(np.int64).T).astype(np.int32)
    for tile_n, swap in [(0, -1), (128, 0), (64, 1)]:
        ops.set_tuning(tile_n, swap)
        out = tc.cutlass_int4_gemm(dev_packed(a), dev_packed(b), M, N, K)
        ops.check_status()
        assert np.array_equal(out.cpu().numpy(), ref), (tile_n, swap)


def test_extreme_codes_exact(tc, ops):
    """All codes -8: every product is +64, the largest accumulator the path can see."""
    M, N, K = 130, 260, 12288
    a = np.full((M, K), -8, np.int8)
    b = np.full((N, K), -8, np.int8)
    out = tc.cutlass_int4_gemm(dev_packed(a), dev_packed(b), M, N, K)
    assert (out == 64 * K).all()
    b[:] = 7
    out = tc.cutlass_int4_gemm(dev_packed(a), dev_packed(b), M, N, K)
    assert (out == -56 * K).all()


def test_scaled_kat(tc, ops, golden_dir):
    z = np.load(os.path.join(golden_dir, "kat_scaled_8x256x16.npz"))
    out = torch.empty(8, 16, dtype=torch.bfloat16, device="cuda")
    tc.cutlass_int4_scaled_mm(dev_packed(z["a"]), dev_packed(z["b"]), dev_f32(z["scale_a"]), dev_f32(z["scale_b"]),
                              out, 8, 16, 256)
    ops.check_status()
    o = out.float().cpu().numpy()
    rel = np.abs(o - z["ref"]) / (np.abs(z["ref"]) + 1e-10)
    assert rel.max() < 1e-2  # the reference's own assertion
    assert torch.equal(out.cpu(), O.linear_per_channel(z["a"], z["b"], z["scale_a"], z["scale_b"]))


@pytest.mark.parametrize("M,N,K", [(16, 4096, 4096), (200, 520, 2560), (1024, 512, 1024)])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_scaled_bit_exact(tc, ops, M, N, K, dtype):
    rng = np.random.RandomState(M + N + K)
    a, b = rand_codes(rng, (M, K)), rand_codes(rng, (N, K))
    sa = (rng.rand(M).astype(np.float32) + 0.01) * 0.1
    sb = (rng.rand(N).astype(np.float32) + 0.01) * 0.01
    f = O.dequant_per_channel(O.int_gemm(a, b), sa, sb)
    ref = torch.from_numpy(f).to(dtype)
    for tile_n, swap in [(0, -1), (128, 0), (256, 0), (128, 1)]:
        ops.set_tuning(tile_n, swap)
        out = torch.empty(M, N, dtype=dtype, device="cuda")
        tc.cutlass_int4_scaled_mm(dev_packed(a), dev_packed(b), dev_f32(sa), dev_f32(sb), out, M, N, K)
        ops.check_status()
        assert torch.equal(out.cpu(), ref), (tile_n, swap)


@pytest.mark.parametrize("M,N,K", [(512, 512, 256), (600, 1000, 1024), (1024, 264, 4096), (257, 256, 128), (520, 300, 192)])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_cta_pairs_scaled_bit_exact(tc, ops, M, N, K, dtype):
    """Per-channel GEMM on SM pairs (256 x 256 tiles, forced on): bit-identical to the oracle, ragged M and N
    included (a pair's second thread block may own no valid row at all)."""
    rng = np.random.RandomState(M + N + K + 1)
    a, b = rand_codes(rng, (M, K)), rand_codes(rng, (N, K))
    sa = (rng.rand(M).astype(np.float32) + 0.01) * 0.1
    sb = (rng.rand(N).astype(np.float32) + 0.01) * 0.01
    ref = torch.from_numpy(O.dequant_per_channel(O.int_gemm(a, b), sa, sb)).to(dtype)
    try:
        ops.set_cta_pairs(1)
        ops.set_tuning(256, 0)
        out = torch.full((M, N), float("nan"), dtype=dtype, device="cuda")
        tc.cutlass_int4_scaled_mm(dev_packed(a), dev_packed(b), dev_f32(sa), dev_f32(sb), out, M, N, K)
        ops.check_status()
        assert torch.equal(out.cpu(), ref)
    finally:
        ops.set_cta_pairs(-1)
        ops.set_tuning(0, -1)


@pytest.mark.parametrize("M,N,G", [(512, 256, 3), (700, 520, 8), (1024, 1024, 32)])
def test_cta_pairs_grouped(tc, ops, M, N, G):
    """Per-group GEMM on SM pairs (forced on) against the oracle, and bit-identical to the single-block path."""
    rng = np.random.RandomState(M + N + G + 2)
    a, b = rand_codes(rng, (G, M, 128)), rand_codes(rng, (G, N, 128))
    sa = (rng.rand(G, M).astype(np.float32) + 0.01) * 0.1
    sb = (rng.rand(G, N).astype(np.float32) + 0.01) * 0.01
    ref = O.linear_grouped(a, b, sa, sb)
    ap, bp = dev_packed(a), dev_packed(b)
    outs = {}
    try:
        ops.set_tuning(256, 0)
        for mode in (0, 1):
            ops.set_cta_pairs(mode)
            out = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device="cuda")
            tc.cutlass_int4_fused_grouped_gemm(ap, bp, dev_f32(sa), dev_f32(sb), out, M, N, 128, G)
            ops.check_status()
            assert_close_bf16(out, ref, f"pairs={mode} {M}x{N}x{G}")
            outs[mode] = out.cpu()
    finally:
        ops.set_cta_pairs(-1)
        ops.set_tuning(0, -1)
    assert torch.equal(outs[0], outs[1])


@pytest.mark.parametrize("M", [1, 2, 3, 5, 8, 13, 16])
@pytest.mark.parametrize("N,G", [(100, 3), (4096, 32), (257, 96)])
def test_small_m_weight_streaming(tc, ops, M, N, G):
    """A handful of tokens take a weight-streaming kernel (automatic choice: CUDA cores for one or two tokens, the
    register-fed tensor-core kernel from three on): per-channel results are bit-identical to the oracle, per-group
    results within the tolerance, and both agree with the tile kernel."""
    rng = np.random.RandomState(M * 7 + N + G)
    K = G * 128
    a, b = rand_codes(rng, (G, M, 128)), rand_codes(rng, (G, N, 128))
    sa = (rng.rand(G, M).astype(np.float32) + 0.01) * 0.1
    sb = (rng.rand(G, N).astype(np.float32) + 0.01) * 0.01
    ref_g = O.linear_grouped(a, b, sa, sb)
    ar, br = a.transpose(1, 0, 2).reshape(M, K), b.transpose(1, 0, 2).reshape(N, K)
    ref_c = torch.from_numpy(O.dequant_per_channel(O.int_gemm(ar, br), sa[0], sb[0]))
    ap, bp, arp, brp = dev_packed(a), dev_packed(b), dev_packed(ar), dev_packed(br)
    outs = []
    try:
        for tile_n, swap in [(0, -1), (64, 1)]:   # automatic (weight streaming), then the tensor-core kernel
            ops.set_tuning(tile_n, swap)
            og = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device="cuda")
            tc.cutlass_int4_fused_grouped_gemm(ap, bp, dev_f32(sa), dev_f32(sb), og, M, N, 128, G)
            ops.check_status()
            assert_close_bf16(og, ref_g, f"grouped M={M} N={N} G={G} tuning={tile_n}")
            for dtype in (torch.bfloat16, torch.float16):
                oc = torch.full((M, N), float("nan"), dtype=dtype, device="cuda")
                tc.cutlass_int4_scaled_mm(arp, brp, dev_f32(sa[0]), dev_f32(sb[0]), oc, M, N, K)
                ops.check_status()
                assert torch.equal(oc.cpu(), ref_c.to(dtype)), (M, N, G, tile_n, dtype)
            outs.append(og.float().cpu())
    finally:
        ops.set_tuning(0, -1)
    # two summation orders of the same fp32 terms: a couple of bf16 ulps at most
    assert (outs[0] - outs[1]).abs().max() <= 2e-2 * outs[1].abs().max() + 1e-6


@pytest.mark.parametrize("M", [1, 4, 8, 9, 16, 17, 24, 31, 32])
@pytest.mark.parametrize("N,G", [(16, 1), (48, 3), (4096, 32), (512, 96), (6144, 7)])
def test_small_m_register_fed_kernel(tc, ops, M, N, G):
    """The register-fed tensor-core kernel (forced for 1..32 tokens): per-channel results bit-identical to the oracle in
    both output types, per-group results within the tolerance and a couple of bf16 steps from the tile kernel's."""
    rng = np.random.RandomState(M * 11 + N + G)
    K = G * 128
    a, b = rand_codes(rng, (G, M, 128)), rand_codes(rng, (G, N, 128))
    if M > 2:
        a[:, 1, :] = -8      # extreme codes on a whole token: the largest group sums
        b[:, 3, :] = -8
    sa = (rng.rand(G, M).astype(np.float32) + 0.01) * 0.1
    sb = (rng.rand(G, N).astype(np.float32) + 0.01) * 0.01
    ref_g = O.linear_grouped(a, b, sa, sb)
    ar, br = a.transpose(1, 0, 2).reshape(M, K), b.transpose(1, 0, 2).reshape(N, K)
    ref_c = torch.from_numpy(O.dequant_per_channel(O.int_gemm(ar, br), sa[0], sb[0]))
    ap, bp, arp, brp = dev_packed(a), dev_packed(b), dev_packed(ar), dev_packed(br)
    outs = {}
    try:
        for path in (2, 3):
            ops.set_small_m_path(path)
            og = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device="cuda")
            tc.cutlass_int4_fused_grouped_gemm(ap, bp, dev_f32(sa), dev_f32(sb), og, M, N, 128, G)
            ops.check_status()
            assert_close_bf16(og, ref_g, f"grouped M={M} N={N} G={G} path={path}")
            outs[path] = og.float().cpu()
            for dtype in (torch.bfloat16, torch.float16):
                oc = torch.full((M, N), float("nan"), dtype=dtype, device="cuda")
                tc.cutlass_int4_scaled_mm(arp, brp, dev_f32(sa[0]), dev_f32(sb[0]), oc, M, N, K)
                ops.check_status()
                assert torch.equal(oc.cpu(), ref_c.to(dtype)), (M, N, G, path, dtype)
    finally:
        ops.set_small_m_path(0)
    assert (outs[2] - outs[3]).abs().max() <= 2e-2 * outs[3].abs().max() + 1e-6


def test_small_m_kernel_with_scales_that_are_only_4_byte_aligned(tc, ops):
    """The register-fed kernel brings the weight scales in with 16-byte bulk copies when it can; scales that start on
    an odd float fall back to plain loads, with the same result."""
    rng = np.random.RandomState(3)
    M, N, G = 12, 256, 8
    a, b = rand_codes(rng, (G, M, 128)), rand_codes(rng, (G, N, 128))
    sa = (rng.rand(G, M).astype(np.float32) + 0.01) * 0.1
    sb = (rng.rand(G, N).astype(np.float32) + 0.01) * 0.01
    ref = O.linear_grouped(a, b, sa, sb)
    buf = torch.zeros(G * N + 1, dtype=torch.float32, device="cuda")
    sb_odd = buf[1:].view(G, N)
    sb_odd.copy_(torch.from_numpy(sb))
    assert sb_odd.data_ptr() % 16 == 4
    outs = []
    for scale_b in (dev_f32(sb), sb_odd):
        out = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device="cuda")
        tc.cutlass_int4_fused_grouped_gemm(dev_packed(a), dev_packed(b), dev_f32(sa), scale_b, out, M, N, 128, G)
        ops.check_status()
        assert_close_bf16(out, ref, "odd scale alignment")
        outs.append(out)
    assert torch.equal(outs[0], outs[1])
    with pytest.raises(RuntimeError):
        ops.set_small_m_path(7)


def test_config0_end_to_end(tc, ops):
    """x [16,4096] with outlier channels, W [4096,4096]: quantise on the GPU, per-channel linear,
    compare codes, scales and bf16 output with the oracle bit for bit."""
    from fp8_inference_toolkit_b200 import synthetic

    x = synthetic.activations(16, 4096, seed=0)
    w = synthetic.weights(4096, 4096, seed=1)
    xp, xs = tc.dynamic_int4_quant(x.cuda())
    wp, ws = tc.static_int4_weight_quant(w.cuda())
    xc, xso = O.quant_rowwise(x, "activation")
    wc, wso = O.quant_rowwise(w, "weight")
    assert np.array_equal(xp.cpu().numpy(), O.pack_int4(xc)) and np.array_equal(xs.cpu().numpy(), xso)
    assert np.array_equal(wp.cpu().numpy(), O.pack_int4(wc)) and np.array_equal(ws.cpu().numpy(), wso)
    out = torch.empty(16, 4096, dtype=torch.bfloat16, device="cuda")
    tc.cutlass_int4_scaled_mm(xp, wp, xs, ws, out, 16, 4096, 4096)
    ops.check_status()
    ref = O.linear_per_channel(xc, wc, xso, wso)
    assert torch.equal(out.cpu(), ref)
    full = x.float() @ w.float().T
    cos = torch.nn.functional.cosine_similarity(out.float().cpu().flatten(), full.flatten(), dim=0)
    assert cos > 0.5  # sanity only: per-token int4 with x20 outlier channels is a coarse quantiser


@pytest.mark.parametrize("M,N,G", [(1, 8, 1), (10, 96, 3), (64, 128, 2), (100, 3584, 20), (257, 300, 5),
                                   (700, 512, 20), (32, 2560, 76)])
def test_grouped_partials_and_output(tc, ops, M, N, G):
    rng = np.random.RandomState(M + 3 * N + G)
    a, b = rand_codes(rng, (G, M, 128)), rand_codes(rng, (G, N, 128))
    sa = (rng.rand(G, M).astype(np.float32) + 0.01) * 0.1
    sb = (rng.rand(G, N).astype(np.float32) + 0.01) * 0.01
    part = O.grouped_int_partials(a, b)
    ref = O.linear_grouped(a, b, sa, sb)
    ap, bp = dev_packed(a), dev_packed(b)
    for tile_n, swap in TUNINGS:
        ops.set_tuning(tile_n, swap)
        got = ops.int4_grouped_partials(ap, bp, M, N, G)
        ops.check_status()
        assert np.array_equal(got.cpu().numpy(), part), (tile_n, swap)
        out = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device="cuda")
        tc.cutlass_int4_fused_grouped_gemm(ap, bp, dev_f32(sa), dev_f32(sb), out, M, N, 128, G)
        ops.check_status()
        assert_close_bf16(out, ref, f"grouped {M}x{N}x{G} tile {tile_n} swap {swap}")
        if M > 128:
            # one fused multiply-add per group in ascending order, exactly the oracle's operations: the same bits
            assert torch.equal(out.cpu(), ref), (tile_n, swap)
        else:
            # small M: the K groups are cut into ranges whose fp32 sums are added afterwards (another order)
            assert (out.cpu() == ref).float().mean() > 0.98


@pytest.mark.parametrize("M,N,G", [(1, 256, 8), (16, 4096, 32), (100, 640, 7), (128, 384, 96)])
def test_split_k_small_m(tc, ops, M, N, G):
    """Small-M per-group path with the K groups cut into 1..8 ranges: every split count agrees with the
    oracle, and a forced single range equals the automatic choice within the same tolerance."""
    rng = np.random.RandomState(M + N + G)
    a, b = rand_codes(rng, (G, M, 128)), rand_codes(rng, (G, N, 128))
    sa = (rng.rand(G, M).astype(np.float32) + 0.01) * 0.1
    sb = (rng.rand(G, N).astype(np.float32) + 0.01) * 0.01
    ref = O.linear_grouped(a, b, sa, sb)
    ap, bp = dev_packed(a), dev_packed(b)
    try:
        for splits in (0, 1, 2, 3, 8):
            ops.set_split_k(splits)
            out = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device="cuda")
            tc.cutlass_int4_fused_grouped_gemm(ap, bp, dev_f32(sa), dev_f32(sb), out, M, N, 128, G)
            ops.check_status()
            assert_close_bf16(out, ref, f"split-K {splits} {M}x{N}x{G}")
    finally:
        ops.set_split_k(0)


@pytest.mark.parametrize("M,N,K", [(16, 512, 4096), (9, 257, 12288), (100, 640, 1024)])
def test_split_k_per_channel_exact(tc, ops, M, N, K):
    """Small-M per-channel path with K cut into ranges: the ranges carry exact integer sums, so every split count
    gives the oracle's result bit for bit."""
    rng = np.random.RandomState(M + N + K)
    a, b = rand_codes(rng, (M, K)), rand_codes(rng, (N, K))
    sa = (rng.rand(M).astype(np.float32) + 0.01) * 0.1
    sb = (rng.rand(N).astype(np.float32) + 0.01) * 0.01
    ref = torch.from_numpy(O.dequant_per_channel(O.int_gemm(a, b), sa, sb))
    ap, bp = dev_packed(a), dev_packed(b)
    try:
        ops.set_tuning(64, 1)   # tensor-core kernel, weights on the row side
        for splits in (1, 2, 5, 8):
            ops.set_split_k(splits)
            for dtype in (torch.bfloat16, torch.float16):
                out = torch.full((M, N), float("nan"), dtype=dtype, device="cuda")
                tc.cutlass_int4_scaled_mm(ap, bp, dev_f32(sa), dev_f32(sb), out, M, N, K)
                ops.check_status()
                assert torch.equal(out.cpu(), ref.to(dtype)), (splits, dtype)
    finally:
        ops.set_split_k(0)
        ops.set_tuning(0, -1)


def test_grouped_aliases_and_checks(tc, ops):
    rng = np.random.RandomState(9)
    M, N, G = 10, 64, 2
    a, b = rand_codes(rng, (G, M, 128)), rand_codes(rng, (G, N, 128))
    sa, sb = np.ones((G, M), np.float32), np.ones((G, N), np.float32)
    outs = []
    for name in ["cutlass_int4_fused_grouped_gemm", "cutlass_int4_fused_grouped_gemm_v5",
                 "cutlass_int4_fused_grouped_gemm_v7", "cutlass_int4_fused_grouped_gemm_v8",
                 "cutlass_int4_fused_grouped_gemm_v9", "cutlass_int4_scaled_mm_grouped"]:
        out = torch.empty(M, N, dtype=torch.bfloat16, device="cuda")
        getattr(tc, name)(dev_packed(a), dev_packed(b), dev_f32(sa), dev_f32(sb), out, M, N, 128, G)
        outs.append(out)
    for o in outs[1:]:
        assert torch.equal(o, outs[0])
    out16 = torch.empty(M, N, dtype=torch.float16, device="cuda")
    with pytest.raises(RuntimeError, match="BF16"):
        tc.cutlass_int4_fused_grouped_gemm(dev_packed(a), dev_packed(b), dev_f32(sa), dev_f32(sb), out16, M, N, 128, G)
    with pytest.raises(RuntimeError, match="group_size=128"):
        tc.cutlass_int4_fused_grouped_gemm(dev_packed(a), dev_packed(b), dev_f32(sa), dev_f32(sb), outs[0], M, N, 64, G)
    with pytest.raises(RuntimeError, match="multiple of 64"):
        tc.cutlass_int4_gemm(dev_packed(a[0]), dev_packed(b[0]), M, N, 100)


@pytest.mark.parametrize("M", [1, 16, 128, 1024])
@pytest.mark.parametrize("shape", ["qkv", "o", "gate_up", "down"])
def test_config1_quantised_linear(tc, ops, M, shape):
    """Qwen3-8B shapes, group-128: GPU quantise + fused GEMM against the oracle end to end."""
    from fp8_inference_toolkit_b200 import synthetic

    K, N = synthetic.QWEN3_8B_SHAPES[shape]
    x = synthetic.activations(M, K, seed=0)
    w = synthetic.weights(N, K, seed=1)
    xp, xs = tc.dynamic_int4_quant_grouped(x.cuda(), 128)
    wp, ws = tc.static_int4_weight_quant_grouped(w.cuda(), 128)
    out = torch.empty(M, N, dtype=torch.bfloat16, device="cuda")
    tc.cutlass_int4_fused_grouped_gemm(xp, wp, xs, ws, out, M, N, 128, K // 128)
    ops.check_status()
    xc, xso = O.quant_grouped(x, 128, "activation")
    wc, wso = O.quant_grouped(w, 128, "weight")
    assert np.array_equal(xp.cpu().numpy(), O.pack_int4(xc))
    assert np.array_equal(wp.cpu().numpy(), O.pack_int4(wc))
    # every row up to 128 tokens; 48 sampled rows at M = 1024 (the oracle's exact fused multiply-add is slow)
    rows = np.arange(M) if M <= 128 else np.sort(np.random.RandomState(M).choice(M, 48, replace=False))
    ref = O.linear_grouped(xc[:, rows], wc, xso[:, rows], wso)
    got = out[torch.from_numpy(rows).cuda()]
    assert_close_bf16(got, ref, f"{shape} M={M}")
    if M > 128:
        assert torch.equal(got.cpu(), ref)   # unsplit tensor-core path: the oracle's operations in the oracle's order


@pytest.mark.parametrize("shape", ["qkv", "o", "gate_up", "down"])
@pytest.mark.parametrize("epi_warps", [8, 16])
def test_config1_largest_sampled_rows(tc, ops, shape, epi_warps):
    """M=8192, all four Qwen3-8B linears: 32 sampled rows against the oracle, plus linearity in the
    activation scales (doubling scale_a doubles the output exactly in bf16); both epilogue widths."""
    from fp8_inference_toolkit_b200 import synthetic

    M, (K, N) = 8192, synthetic.QWEN3_8B_SHAPES[shape]
    ops.set_epilogue_warps(epi_warps)
    G = K // 128
    x = synthetic.activations(M, K, seed=0, device="cuda")
    w = synthetic.weights(N, K, seed=1, device="cuda")
    xp, xs = tc.dynamic_int4_quant_grouped(x, 128)
    wp, ws = tc.static_int4_weight_quant_grouped(w, 128)
    out = torch.empty(M, N, dtype=torch.bfloat16, device="cuda")
    tc.cutlass_int4_fused_grouped_gemm(xp, wp, xs, ws, out, M, N, 128, G)
    ops.check_status()
    rows = np.random.RandomState(1).choice(M, 32, replace=False)
    ridx = torch.from_numpy(rows).cuda()
    xc = O.unpack_int4(xp[:, ridx].cpu().numpy())
    wc = O.unpack_int4(wp.cpu().numpy())
    ref = O.linear_grouped(xc, wc, xs[:, ridx].cpu().numpy(), ws.cpu().numpy())
    assert_close_bf16(out[ridx], ref, f"{shape} M=8192 sampled rows")
    assert torch.equal(out[ridx].cpu(), ref)
    out2 = torch.empty_like(out)
    tc.cutlass_int4_fused_grouped_gemm(xp, wp, (xs * 2).contiguous(), ws, out2, M, N, 128, G)
    ops.set_epilogue_warps(0)
    assert torch.equal(out2.float(), out.float() * 2)


@pytest.mark.parametrize("K,N", [(2560, 9728), (2560, 3584), (9728, 2560)])
@pytest.mark.parametrize("M", [1, 10, 32, 64, 100, 700])
def test_reference_kernel_test_shapes(tc, ops, M, K, N):
    """The shapes of the reference's own kernel-vs-kernel checks (int4_native_tc/test_v5_correctness.py:12-52,
    116-138: Qwen3-4B projections at M in {1, 10, 32, 64, 100, 700}), here against the CPU oracle: quantised
    codes bit for bit, per-group integer partial sums bit for bit, bf16 output within 1e-2 / cosine 0.9999."""
    from fp8_inference_toolkit_b200 import synthetic

    G = K // 128
    x = synthetic.activations(M, K, seed=M)
    w = synthetic.weights(N, K, seed=K + N)
    xp, xs = tc.dynamic_int4_quant_grouped(x.cuda(), 128)
    wp, ws = tc.static_int4_weight_quant_grouped(w.cuda(), 128)
    out = torch.empty(M, N, dtype=torch.bfloat16, device="cuda")
    tc.cutlass_int4_fused_grouped_gemm(xp, wp, xs, ws, out, M, N, 128, G)
    ops.check_status()
    xc, xso = O.quant_grouped(x, 128, "activation")
    wc, wso = O.quant_grouped(w, 128, "weight")
    assert np.array_equal(xp.cpu().numpy(), O.pack_int4(xc))
    assert np.array_equal(wp.cpu().numpy(), O.pack_int4(wc))
    assert_close_bf16(out, O.linear_grouped(xc, wc, xso, wso), f"K={K} N={N} M={M}")
    if M <= 32:
        part = ops.int4_grouped_partials(xp, wp, M, N, G)
        assert np.array_equal(part.cpu().numpy(), O.grouped_int_partials(xc, wc))


def test_split_k_workspace_is_per_stream_and_never_moves(tc, ops):
    """The split-K workspace belongs to one (device, stream); growing it keeps the buffer handed out before (a CUDA
    graph replayed after the growth still computes the right thing), and a second stream gets its own."""
    rng = np.random.RandomState(3)
    M, N, G = 64, 512, 16
    a, b = rand_codes(rng, (G, M, 128)), rand_codes(rng, (G, N, 128))
    sa = dev_f32((rng.rand(G, M) + 0.01) * 0.1)
    sb = dev_f32((rng.rand(G, N) + 0.01) * 0.01)
    ap, bp = dev_packed(a), dev_packed(b)
    ops.set_split_k(4)
    side = torch.cuda.Stream()
    out = torch.empty(M, N, dtype=torch.bfloat16, device="cuda")
    with torch.cuda.stream(side):
        assert ops.workspace_bytes() == 0
        ops.reserve_workspace(1 << 20)
        first = ops.workspace_bytes()
        assert first >= (16 << 20)
        tc.cutlass_int4_fused_grouped_gemm(ap, bp, sa, sb, out, M, N, 128, G)   # warm-up outside capture
        side.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=side):
            tc.cutlass_int4_fused_grouped_gemm(ap, bp, sa, sb, out, M, N, 128, G)
        ops.reserve_workspace(first * 3)            # grows: a new buffer beside the one the graph holds
        assert ops.workspace_bytes() >= first * 3
        big = torch.full((int(first) // 4,), 7.0, device="cuda")   # would reuse freed memory if the old buffer had been freed
        out.zero_()
        g.replay()
        side.synchronize()
        del big
    ops.set_split_k(0)
    ops.check_status()
    ref = O.linear_grouped(a, b, sa.cpu().numpy(), sb.cpu().numpy())
    assert_close_bf16(out, ref, "graph replay after workspace growth")
    other = torch.cuda.Stream()
    with torch.cuda.stream(other):
        assert ops.workspace_bytes() == 0               # another stream: its own (not yet needed) workspace


@pytest.mark.parametrize("M,N,G", [(700, 1000, 5), (1024, 1536, 8), (513, 192, 3)])
def test_192_wide_tiles_on_sm_pairs(tc, ops, M, N, G):
    """192-column tiles (256 x 192 on a pair of SMs, twelve epilogue warps): per-group, zero-point and per-channel
    outputs equal the oracle bit for bit, ragged edges included."""
    rng = np.random.RandomState(M + N + G)
    a, b = rand_codes(rng, (G, M, 128)), rand_codes(rng, (G, N, 128))
    sa = (rng.rand(G, M).astype(np.float32) + 0.01) * 0.1
    sb = (rng.rand(G, N).astype(np.float32) + 0.01) * 0.01
    adj = rng.randint(-7, 9, size=(G, M)).astype(np.float32)
    ap, bp = dev_packed(a), dev_packed(b)
    ops.set_tuning(192, 0)
    out = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device="cuda")
    tc.cutlass_int4_fused_grouped_gemm(ap, bp, dev_f32(sa), dev_f32(sb), out, M, N, 128, G)
    ops.check_status()
    assert torch.equal(out.cpu(), O.linear_grouped(a, b, sa, sb))
    wcs = O.weight_group_sums(b)
    out.fill_(float("nan"))
    tc.cutlass_int4_fused_grouped_gemm_azp(ap, bp, dev_f32(sa), dev_f32(sb), out, dev_f32(adj), dev_f32(wcs), M, N, 128, G)
    ops.check_status()
    assert torch.equal(out.cpu(), O.to_bf16(O.linear_grouped_azp_f32(a, b, sa, sb, adj, wcs)))
    K = G * 128
    ar = a.transpose(1, 0, 2).reshape(M, K)
    br = b.transpose(1, 0, 2).reshape(N, K)
    out.fill_(float("nan"))
    tc.cutlass_int4_scaled_mm(dev_packed(ar), dev_packed(br), dev_f32(sa[0]), dev_f32(sb[0]), out, M, N, K)
    ops.check_status()
    assert torch.equal(out.cpu(), O.linear_per_channel(ar, br, sa[0], sb[0]))
