"""GPU: seeded random shapes through every dense path (weight streaming, split-K, single thread blocks, SM pairs;
ragged M and N, K that ends in half a group) against the oracle: int32 and per-channel outputs bit for bit,
per-group outputs within the tolerance."""
import numpy as np
import pytest
import torch

from oracle import w4a4_oracle as O
from tests.helpers import assert_close_bf16, dev_packed, rand_codes

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
    _ops.check_status()

MS = [1, 2, 3, 7, 8, 9, 15, 16, 17, 31, 64, 100, 128, 129, 255, 256, 300, 511, 512, 513, 700, 1024, 1500]
NS = [1, 8, 31, 64, 100, 128, 255, 256, 257, 384, 500, 512, 640, 1000, 1536]
GS = [1, 2, 3, 5, 8, 16, 33]


def dev_f32(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


@pytest.mark.parametrize("seed", [11, 12, 13])
def test_random_shapes_against_oracle(tc, ops, seed):
    rng = np.random.RandomState(seed)
    for _ in range(14):
        M, N, G = int(rng.choice(MS)), int(rng.choice(NS)), int(rng.choice(GS))
        a, b = rand_codes(rng, (G, M, 128)), rand_codes(rng, (G, N, 128))
        sa = (rng.rand(G, M).astype(np.float32) + 0.01) * 0.1
        sb = (rng.rand(G, N).astype(np.float32) + 0.01) * 0.01
        out = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device="cuda")
        tc.cutlass_int4_fused_grouped_gemm(dev_packed(a), dev_packed(b), dev_f32(sa), dev_f32(sb), out, M, N, 128, G)
        ops.check_status()
        assert_close_bf16(out, O.linear_grouped(a, b, sa, sb), f"per-group {M}x{N}x{G}")
        K = G * 128 - (64 if rng.rand() < 0.25 else 0)
        ar, br = rand_codes(rng, (M, K)), rand_codes(rng, (N, K))
        acc = O.int_gemm(ar, br)
        got = tc.cutlass_int4_gemm(dev_packed(ar), dev_packed(br), M, N, K)
        assert np.array_equal(got.cpu().numpy(), acc), (M, N, K)
        for dtype in (torch.bfloat16, torch.float16):
            oc = torch.full((M, N), float("nan"), dtype=dtype, device="cuda")
            tc.cutlass_int4_scaled_mm(dev_packed(ar), dev_packed(br), dev_f32(sa[0]), dev_f32(sb[0]), oc, M, N, K)
            ops.check_status()
            ref = torch.from_numpy(O.dequant_per_channel(acc, sa[0], sb[0])).to(dtype)
            assert torch.equal(oc.cpu(), ref), (M, N, K, dtype)
