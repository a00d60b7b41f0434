"""GPU parity of the W4A8 path (int8 activations x int4 weights held as int8): the tensor-core kernel with both
operands loaded by TMA straight into its swizzled int8 stages, and the per-token int8 quantiser, against the oracle."""
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


@pytest.fixture()
def ops():
    from fp8_inference_toolkit_b200 import ops as _ops

    yield _ops
    _ops.set_tuning(0, -1)
    _ops.set_cta_pairs(-1)
    _ops.check_status()


def _run(tc, a, b, sa, sb, dtype=torch.bfloat16):
    M, K = a.shape
    N = b.shape[0]
    out = torch.full((M, N), float("nan"), dtype=dtype, device="cuda")
    tc.cutlass_w4a8_scaled_mm(torch.from_numpy(a).cuda(), torch.from_numpy(b).cuda(), torch.from_numpy(sa).cuda(),
                              torch.from_numpy(sb).cuda(), out, M, N, K)
    return out


@pytest.mark.parametrize("tile_n,swap", [(0, -1), (64, 1), (128, 1), (64, 0), (128, 0), (256, 0)])
def test_kat_reference_test_13(tc, ops, golden_dir, tile_n, swap):
    z = np.load(os.path.join(golden_dir, "kat_w4a8_8x256x64.npz"))
    ops.set_tuning(tile_n, swap)
    out = _run(tc, z["a"], z["b"], z["scale_a"], z["scale_b"])
    ops.check_status()
    ref = O.linear_w4a8(z["a"], z["b"], z["scale_a"], z["scale_b"])
    assert torch.equal(out.cpu(), ref)
    rel = np.abs(out.float().cpu().numpy() - z["ref"]) / (np.abs(z["ref"]) + 1e-10)
    assert rel.max() < 1e-2      # the reference test's own bar (test_correctness.py:581)


@pytest.mark.parametrize("M,N,K", [(1, 8, 32), (17, 100, 96), (128, 256, 128), (129, 1000, 2560), (300, 257, 320),
                                   (513, 72, 12288), (40, 24, 65536), (1024, 4096, 4096)])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_ragged_shapes_bit_exact(tc, ops, M, N, K, dtype):
    """Full int8 range on the activation side (sums beyond 2^24 at large K: the int32 accumulator is converted with one
    rounding, as the oracle's astype does)."""
    rng = np.random.RandomState(M + 3 * N + K)
    a = rng.randint(-128, 128, size=(M, K)).astype(np.int8)
    b = rng.randint(-8, 8, size=(N, K)).astype(np.int8)
    sa = (rng.rand(M).astype(np.float32) + 0.01) * 0.01
    sb = (rng.rand(N).astype(np.float32) + 0.01) * 0.1
    out = _run(tc, a, b, sa, sb, dtype)
    ops.check_status()
    assert torch.equal(out.cpu(), O.linear_w4a8(a, b, sa, sb, dtype))


@pytest.mark.parametrize("pairs", [0, 1])
def test_large_m_single_blocks_and_sm_pairs(tc, ops, pairs):
    rng = np.random.RandomState(5)
    M, N, K = 2048, 1024, 1024
    a = rng.randint(-128, 128, size=(M, K)).astype(np.int8)
    b = rng.randint(-128, 128, size=(N, K)).astype(np.int8)      # the op takes any int8 weight
    sa = (rng.rand(M).astype(np.float32) + 0.01) * 0.01
    sb = (rng.rand(N).astype(np.float32) + 0.01) * 0.1
    ops.set_cta_pairs(pairs)
    out = _run(tc, a, b, sa, sb)
    ops.check_status()
    assert torch.equal(out.cpu(), O.linear_w4a8(a, b, sa, sb))


@pytest.mark.parametrize("M,K", [(1, 32), (7, 100), (33, 4096), (300, 12288), (5, 65536)])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
def test_int8_quantiser_bit_exact(tc, M, K, dtype):
    g = torch.Generator().manual_seed(M + K)
    x = (torch.randn(M, K, generator=g) * 3).to(dtype)
    x[0] = 0
    q, s = tc.dynamic_int8_quant(x.cuda())
    qr, sr = O.quant_rowwise_int8(x)
    assert q.dtype == torch.int8 and np.array_equal(q.cpu().numpy(), qr) and np.array_equal(s.cpu().numpy(), sr)


def test_full_path_reference_test_14(tc, ops):
    """bf16 -> int8 activations, bf16 -> int4 weights -> unpacked to int8, W4A8 GEMM (test_correctness.py:589-615),
    every stage against the oracle, and the result close to the bf16 product."""
    from fp8_inference_toolkit_b200 import synthetic

    M, (K, N) = 160, synthetic.QWEN3_8B_SHAPES["o"]
    x = synthetic.activations(M, K, seed=0)
    w = synthetic.weights(N, K, seed=1)
    xq, xs = tc.dynamic_int8_quant(x.cuda())
    wp, ws = tc.static_int4_weight_quant(w.cuda())
    w8 = tc.unpack_int4_to_int8(wp, K)
    out = torch.empty(M, N, dtype=torch.bfloat16, device="cuda")
    tc.cutlass_w4a8_scaled_mm(xq, w8, xs, ws, out, M, N, K)
    ops.check_status()
    xr, xsr = O.quant_rowwise_int8(x)
    wc, wsr = O.quant_rowwise(w, "weight")
    assert np.array_equal(xq.cpu().numpy(), xr) and np.array_equal(w8.cpu().numpy(), wc)
    assert torch.equal(out.cpu(), O.linear_w4a8(xr, wc, xsr, wsr))
    full = x.float() @ w.float().T
    cos = torch.nn.functional.cosine_similarity(out.float().cpu().flatten(), full.flatten(), dim=0)
    assert cos > 0.97
