"""GPU parity: fused quantise+pack and unpack against the CPU oracle, bit for bit, through the
reference-named ops (which call the C ABI)."""
import os

import numpy as np
import pytest
import torch

from oracle import w4a4_oracle as O

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def tc():
    import int4_native_tc

    return int4_native_tc


def _x(M, K, seed, dtype=torch.bfloat16, zero_rows=()):
    from fp8_inference_toolkit_b200 import synthetic

    x = synthetic.activations(M, K, seed).to(dtype)
    for r in zero_rows:
        x[r] = 0
    return x


@pytest.mark.parametrize("M,K", [(16, 4096), (5, 2560), (3, 64), (1, 2), (7, 10), (2, 12288), (3, 20000),
                                 (9, 8192), (4, 16384), (33, 2048)])
@pytest.mark.parametrize("role", ["activation", "weight"])
def test_rowwise_bit_exact(tc, M, K, role):
    x = _x(M, K, seed=M * 131 + K, zero_rows=(0,) if M > 2 else ())
    fn = tc.dynamic_int4_quant if role == "activation" else tc.static_int4_weight_quant
    packed, scale = fn(x.cuda())
    codes, s = O.quant_rowwise(x, role)
    assert packed.shape == (M, K // 2) and packed.dtype == torch.uint8
    assert scale.shape == (M,) and scale.dtype == torch.float32
    assert np.array_equal(packed.cpu().numpy(), O.pack_int4(codes))
    assert np.array_equal(scale.cpu().numpy(), s)


@pytest.mark.parametrize("dtype", [torch.float16, torch.float32])
def test_rowwise_other_dtypes(tc, dtype):
    x = _x(6, 1024, 7, dtype)
    packed, scale = tc.dynamic_int4_quant(x.cuda())
    codes, s = O.quant_rowwise(x, "activation")
    assert np.array_equal(packed.cpu().numpy(), O.pack_int4(codes))
    assert np.array_equal(scale.cpu().numpy(), s)


@pytest.mark.parametrize("M,K,gs", [(512, 4096, 128), (13, 384, 128), (1, 128, 128), (8, 12288, 128),
                                    (21, 1024, 64), (10, 256, 32), (6, 1536, 256), (300, 768, 128)])
@pytest.mark.parametrize("role", ["activation", "weight"])
def test_grouped_bit_exact(tc, M, K, gs, role):
    x = _x(M, K, seed=M + K + gs, zero_rows=(0,) if M > 2 else ())
    fn = tc.dynamic_int4_quant_grouped if role == "activation" else tc.static_int4_weight_quant_grouped
    packed, scale = fn(x.cuda(), gs)
    codes, s = O.quant_grouped(x, gs, role)
    G = K // gs
    assert packed.shape == (G, M, gs // 2) and scale.shape == (G, M)
    assert np.array_equal(packed.cpu().numpy(), O.pack_int4(codes))
    assert np.array_equal(scale.cpu().numpy(), s)


def test_grouped_fp32_and_strided_input(tc):
    x = _x(12, 1024, 5, torch.float32)
    xs = torch.zeros(12, 2048, dtype=torch.float32)
    xs[:, :1024] = x
    view = xs.cuda()[:, :1024]  # row stride 2048, still 16-byte aligned rows
    packed, scale = tc.dynamic_int4_quant_grouped(view, 128)
    codes, s = O.quant_grouped(x, 128, "activation")
    assert np.array_equal(packed.cpu().numpy(), O.pack_int4(codes))
    assert np.array_equal(scale.cpu().numpy(), s)
    odd = x.cuda()[:, 1:513]  # misaligned view: the op must copy, not fault
    packed, scale = tc.dynamic_int4_quant_grouped(odd, 128)
    codes, s = O.quant_grouped(x[:, 1:513], 128, "activation")
    assert np.array_equal(packed.cpu().numpy(), O.pack_int4(codes))


def test_given_scales_bit_exact(tc):
    x = _x(40, 2048, 11)
    rng = np.random.RandomState(3)
    s_row = (rng.rand(40).astype(np.float32) + 0.05)
    p = tc.int4_quant_with_scales(x.cuda(), torch.from_numpy(s_row).cuda(), 0)
    assert np.array_equal(p.cpu().numpy(), O.pack_int4(O.quant_with_scales(x, s_row)))
    s_grp = (rng.rand(16, 40).astype(np.float32) + 0.05)
    p = tc.int4_quant_with_scales(x.cuda(), torch.from_numpy(s_grp).cuda(), 128)
    assert np.array_equal(p.cpu().numpy(), O.pack_int4(O.quant_with_scales(x, s_grp, 128)))


def test_empty_and_errors(tc):
    p, s = tc.dynamic_int4_quant(torch.zeros(0, 256, dtype=torch.bfloat16, device="cuda"))
    assert p.shape == (0, 128) and s.shape == (0,)
    p, s = tc.dynamic_int4_quant_grouped(torch.zeros(0, 256, dtype=torch.bfloat16, device="cuda"), 128)
    assert p.shape == (2, 0, 64) and s.shape == (2, 0)
    with pytest.raises(RuntimeError, match="even"):
        tc.dynamic_int4_quant(torch.zeros(2, 7, dtype=torch.bfloat16, device="cuda"))
    with pytest.raises(RuntimeError, match="divisible"):
        tc.dynamic_int4_quant_grouped(torch.zeros(2, 200, dtype=torch.bfloat16, device="cuda"), 128)
    with pytest.raises(RuntimeError):
        tc.dynamic_int4_quant_grouped(torch.zeros(2, 192, dtype=torch.bfloat16, device="cuda"), 96)


def test_unpack_kat(tc, golden_dir):
    z = np.load(os.path.join(golden_dir, "kat_unpack_16x256.npz"))
    out = tc.unpack_int4_to_int8(torch.from_numpy(z["packed"]).cuda(), 256)
    assert out.dtype == torch.int8 and out.shape == (16, 256)
    assert np.array_equal(out.cpu().numpy(), z["unpacked"])
    rng = np.random.RandomState(1)
    c = rng.randint(-8, 8, size=(37, 1030)).astype(np.int8)  # odd sizes: tail path
    out = tc.unpack_int4_to_int8(torch.from_numpy(O.pack_int4(c)).cuda(), 1030)
    assert np.array_equal(out.cpu().numpy(), c)


def test_full_size_properties(tc):
    """16384 x 12288 (the largest quantise configuration): sampled rows against the oracle,
    group/row consistency and idempotence under the returned scales."""
    from fp8_inference_toolkit_b200 import synthetic

    M, K = 16384, 12288
    x = synthetic.activations(M, K, seed=2, outlier_frac=0.01, device="cuda")
    pg, sg = tc.dynamic_int4_quant_grouped(x, 128)
    pr, sr = tc.dynamic_int4_quant(x)
    rows = np.random.RandomState(0).choice(M, 48, replace=False)
    xs = x[torch.from_numpy(rows).cuda()].cpu()
    cg, sgo = O.quant_grouped(xs, 128, "activation")
    assert np.array_equal(pg[:, rows].cpu().numpy(), O.pack_int4(cg))
    assert np.array_equal(sg[:, rows].cpu().numpy(), sgo)
    cr, sro = O.quant_rowwise(xs, "activation")
    assert np.array_equal(pr[rows].cpu().numpy(), O.pack_int4(cr))
    assert np.array_equal(sr[rows].cpu().numpy(), sro)
    # idempotence: quantising again with the returned (un-floored here) scales gives the same codes
    assert torch.equal(tc.int4_quant_with_scales(x, sg, 128), pg)
    assert torch.equal(tc.int4_quant_with_scales(x, sr, 0), pr)
    # every row uses the full code range somewhere (absmax element maps to +-7)
    u = tc.unpack_int4_to_int8(pr[:256], K)
    assert (u.abs().amax(dim=1) == 7).all()


@pytest.mark.parametrize("M,K", [(37, 1024), (8, 4096), (130, 256), (5, 1536), (64, 12288)])
def test_rmsnorm_quant_against_oracle(M, K):
    """RMSNorm + grouped quantise against the CPU oracle: the row statistic is a fixed sequence of correctly
    rounded fp32 operations, so codes and scales are compared bit for bit."""
    from fp8_inference_toolkit_b200 import ops
    from oracle import w4a4_oracle as O

    g = torch.Generator().manual_seed(3 * M + K)
    x = (torch.randn(M, K, generator=g) * 1.5).to(torch.bfloat16)
    x[0] = 0  # a zero row: factor = 1 / sqrt(eps), all codes zero
    w = (1.0 + 0.1 * torch.randn(K, generator=g)).to(torch.bfloat16)
    eps = 1e-6
    p, s = ops.rmsnorm_int4_quant_grouped(x.cuda(), w.cuda(), eps, 128)
    codes, so = O.rmsnorm_quant_grouped(x, w, eps, 128)
    assert np.array_equal(p.cpu().numpy(), O.pack_int4(codes))
    assert np.array_equal(s.cpu().numpy(), so)


@pytest.mark.parametrize("M,K", [(37, 1024), (8, 4096), (130, 256)])
def test_rmsnorm_quant_matches_unfused(tc, M, K):
    """RMSNorm fused in front of the grouped quantiser against the unfused pair (fp32 normalisation returning
    bf16, times a bf16 weight, then the grouped quantiser).  The two differ only where the row statistic's last
    bit flips a bf16 rounding, so nearly all codes and all scales agree."""
    from fp8_inference_toolkit_b200 import ops

    g = torch.Generator().manual_seed(M + K)
    x = (torch.randn(M, K, generator=g) * 1.5).to(torch.bfloat16).cuda()
    w = (1.0 + 0.1 * torch.randn(K, generator=g)).to(torch.bfloat16).cuda()
    eps = 1e-6
    xf = x.float()
    y = (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)).to(torch.bfloat16) * w
    p_ref, s_ref = tc.dynamic_int4_quant_grouped(y, 128)
    p, s = ops.rmsnorm_int4_quant_grouped(x, w, eps, 128)
    assert p.shape == p_ref.shape and s.shape == s_ref.shape
    assert torch.allclose(s, s_ref, rtol=1e-2, atol=0)
    assert (s == s_ref).float().mean() > 0.95
    assert (p == p_ref).float().mean() > 0.995
    # a strided view of a wider buffer gives the same result
    wide = torch.zeros(M, K + 64, dtype=torch.bfloat16, device="cuda")
    wide[:, :K] = x
    p2, s2 = ops.rmsnorm_int4_quant_grouped(wide[:, :K], w, eps, 128)
    assert torch.equal(p2, p) and torch.equal(s2, s)
