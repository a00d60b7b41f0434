"""CPU: the oracle against the golden vectors produced by the reference's own CPU helpers
(tests/golden/make_golden.py), plus internal consistency of the oracle."""
import os

import numpy as np
import torch

from oracle import w4a4_oracle as O


def _load(golden_dir, name):
    return np.load(os.path.join(golden_dir, name))


def test_pack_and_gemm_small_kat(golden_dir):
    z = _load(golden_dir, "kat_gemm_4x128x8.npz")
    assert np.array_equal(O.pack_int4(z["a"]), z["a_packed"])
    assert np.array_equal(O.pack_int4(z["b"]), z["b_packed"])
    assert np.array_equal(O.int_gemm(z["a"], z["b"]), z["c"])
    assert np.array_equal(O.unpack_int4(z["a_packed"]), z["a"])


def test_gemm_llm_size_kat(golden_dir):
    z = _load(golden_dir, "kat_gemm_16x2560x2560.npz")
    rng = np.random.RandomState(int(z["seed"]))
    a = rng.randint(-8, 8, size=(16, 2560)).astype(np.int8)
    b = rng.randint(-8, 8, size=(2560, 2560)).astype(np.int8)
    assert np.array_equal(O.pack_int4(a[:1]), z["a_packed_row0"])
    assert np.array_equal(O.pack_int4(b[:1]), z["b_packed_row0"])
    c = O.int_gemm(a, b)
    assert c.dtype == np.int32 and np.array_equal(c, z["c"])
    # the reference's own formulation (int32 torch matmul) agrees with the fast exact path
    ct = O.int_gemm_int32_torch(torch.from_numpy(a), torch.from_numpy(b)).numpy()
    assert np.array_equal(ct, z["c"])


def test_unpack_kat(golden_dir):
    z = _load(golden_dir, "kat_unpack_16x256.npz")
    assert np.array_equal(O.pack_int4(z["codes"]), z["packed"])
    assert np.array_equal(O.unpack_int4(z["packed"]), z["unpacked"])
    assert np.array_equal(z["unpacked"], z["codes"])


def test_scaled_epilogue_kat(golden_dir):
    z = _load(golden_dir, "kat_scaled_8x256x16.npz")
    out = O.linear_per_channel(z["a"], z["b"], z["scale_a"], z["scale_b"]).float().numpy()
    rel = np.abs(out - z["ref"]) / (np.abs(z["ref"]) + 1e-10)
    assert rel.max() < 1e-2  # the reference's bar, int4_native_tc/test_correctness.py:220


def test_native_matmul_kat(golden_dir):
    z = _load(golden_dir, "kat_native_matmul.npz")
    acc = O.int_gemm(z["a"], z["b"])
    f = acc.astype(np.float32) * z["scale_a"][:, None] * z["scale_b"][None, :]  # reference order a then b
    assert np.allclose(f, z["ref"], rtol=1e-6, atol=0)
    g = O.dequant_per_channel(acc, z["scale_a"], z["scale_b"])  # epilogue order b then a
    assert np.allclose(g, z["ref"], rtol=1e-6, atol=0)


def test_quant_formula_kat(golden_dir):
    z = _load(golden_dir, "kat_quant_formula.npz")
    w = torch.from_numpy(z["w_bf16_bits"]).view(torch.bfloat16)
    codes, scale = O.quant_grouped(w, 128, "weight")  # [G,N,gs], [G,N]
    assert np.array_equal(codes.transpose(1, 0, 2), z["codes"])
    assert np.array_equal(scale.T, z["scale"])


def test_quant_edge_cases():
    x = torch.zeros(3, 256, dtype=torch.bfloat16)
    x[1, 5] = 3.0
    x[2, :] = -1.0
    codes, s = O.quant_rowwise(x, "activation")
    assert (codes[0] == 0).all() and s[0] == O.K_MIN_SCALE
    assert codes[1, 5] == 7 and (np.delete(codes[1], 5) == 0).all()
    assert (codes[2] == -7).all()
    _, sw = O.quant_rowwise(x, "weight")
    assert sw[0] == 1.0 and sw[1] == np.float32(3.0) / np.float32(7.0)
    # ties round to even: x/s = 0.5 -> 0, 1.5 -> 2, 2.5 -> 2
    y = torch.tensor([[7.0, 0.5, 1.5, 2.5, -0.5, -1.5, -2.5, 3.5]], dtype=torch.bfloat16)
    c, _ = O.quant_rowwise(y, "weight")
    assert c[0].tolist() == [7, 0, 2, 2, 0, -2, -2, 4]


def test_grouped_layout_and_roundtrip():
    g = torch.Generator().manual_seed(3)
    x = torch.randn(5, 384, generator=g).to(torch.bfloat16)
    codes, s = O.quant_grouped(x, 128, "activation")
    assert codes.shape == (3, 5, 128) and s.shape == (3, 5)
    for gi in range(3):
        cr, sr = O.quant_rowwise(x[:, gi * 128:(gi + 1) * 128], "activation")
        assert np.array_equal(cr, codes[gi]) and np.array_equal(sr, s[gi])
    assert np.array_equal(O.unpack_int4(O.pack_int4(codes)), codes)
    # "given scales" reproduces the codes when handed the un-floored scales
    assert np.array_equal(O.quant_with_scales(x, s, 128), codes)


def test_refcuda_form_rarely_differs():
    g = torch.Generator().manual_seed(4)
    x = torch.randn(64, 4096, generator=g).to(torch.bfloat16).float().numpy()
    am = np.abs(x).max(axis=1, keepdims=True)
    a = O.quant_codes(x, am)
    b = O.quant_codes_refcuda_form(x, am)
    assert (a != b).mean() < 1e-3  # measured 1.4e-4 on bf16 N(0,1) rows (near-ties only)
    assert np.abs(a.astype(int) - b.astype(int)).max() <= 1


def test_linear_grouped_matches_float64():
    g = torch.Generator().manual_seed(5)
    x = torch.randn(7, 512, generator=g).to(torch.bfloat16)
    w = (torch.randn(9, 512, generator=g) * 0.02).to(torch.bfloat16)
    xa, sa = O.quant_grouped(x, 128, "activation")
    wq, sw = O.quant_grouped(w, 128, "weight")
    out = O.linear_grouped(xa, wq, sa, sw).float().numpy()
    ref = sum((xa[i].astype(np.float64) @ wq[i].astype(np.float64).T) * sa[i][:, None] * sw[i][None, :] for i in range(4))
    assert np.abs(out - ref).max() <= np.abs(ref).max() * 2 ** -7
    # and is close to the unquantised product (quality sanity, not a parity claim)
    full = x.float().numpy() @ w.float().numpy().T
    cos = (out * full).sum() / np.sqrt((out ** 2).sum() * (full ** 2).sum())
    assert cos > 0.95


def test_moe_sort_and_layer_shapes():
    ids = np.array([[2, 0], [1, 2], [0, 1], [2, 1]])
    order, off = O.moe_sort(ids, 4)
    assert off.tolist() == [0, 2, 5, 8, 8]
    assert order.tolist() == [1, 4, 2, 5, 7, 0, 3, 6]


def test_w4a8_golden(golden_dir):
    """int8 x int4-as-int8 product and scaled epilogue against the vector made by executing the CPU lines of the
    reference's own test (int4_native_tc/test_correctness.py:551-566)."""
    z = np.load(os.path.join(golden_dir, "kat_w4a8_8x256x64.npz"))
    acc = (z["a"].astype(np.int64) @ z["b"].astype(np.int64).T).astype(np.int32)
    assert np.array_equal(acc, z["acc"])
    out = O.linear_w4a8(z["a"], z["b"], z["scale_a"], z["scale_b"], torch.float32).numpy()
    # the test multiplies by scale_a first, the kernel's epilogue by scale_b first: the same up to fp32 rounding
    np.testing.assert_allclose(out, z["ref"], rtol=3e-7, atol=0)


def test_int8_quantiser_formula():
    x = torch.tensor([[0.0, 0.0, 0.0, 0.0], [1.0, -2.0, 0.5, 127.0], [1e-9, -1e-9, 0.0, 5e-10]], dtype=torch.float32)
    q, s = O.quant_rowwise_int8(x)
    assert np.array_equal(q[0], [0, 0, 0, 0]) and s[0] == O.K_MIN_SCALE_INT8
    assert np.array_equal(q[1], [1, -2, 0, 127]) and s[1] == np.float32(1.0)
    assert np.array_equal(q[2], [127, -127, 0, 64]) and s[2] == O.K_MIN_SCALE_INT8   # codes from the un-floored absmax
