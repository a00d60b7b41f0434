"""Shared helpers of the GPU parity tests."""
import numpy as np
import torch

from oracle import w4a4_oracle as O

REL_TOL = 1e-2      # bf16 outputs: max relative error (reference bar, test_correctness.py:220)
COS_TOL = 0.9999    # bf16 outputs: flat cosine (reference bar, test_v5_correctness.py:50)


def dev_packed(codes: np.ndarray) -> torch.Tensor:
    return torch.from_numpy(O.pack_int4(codes)).cuda()


def dev_f32(a: np.ndarray) -> torch.Tensor:
    return torch.from_numpy(np.ascontiguousarray(a, dtype=np.float32)).cuda()


def rand_codes(rng: np.random.RandomState, shape) -> np.ndarray:
    return rng.randint(-8, 8, size=shape).astype(np.int8)


def assert_close_bf16(out: torch.Tensor, ref: torch.Tensor, what: str = ""):
    """1e-2 relative (against the row-wise scale of the reference) and cosine >= 0.9999."""
    o = out.float().cpu().numpy().astype(np.float64)
    r = ref.float().cpu().numpy().astype(np.float64)
    assert o.shape == r.shape, (o.shape, r.shape)
    denom = np.maximum(np.abs(r), 1e-3 * np.abs(r).max() + 1e-30)
    rel = np.abs(o - r) / denom
    assert rel.max() < REL_TOL, f"{what}: max rel err {rel.max():.3e}"
    cos = (o * r).sum() / (np.sqrt((o * o).sum() * (r * r).sum()) + 1e-300)
    assert cos >= COS_TOL, f"{what}: cosine {cos}"
    return rel.max(), cos
