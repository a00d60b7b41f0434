"""CPU oracle for the int4_native_tc W4A4 hot path.  TEST INFRASTRUCTURE ONLY.

This module restates, in numpy/torch on the CPU, the arithmetic of the
reference's quantise -> pack -> int4 x int4 integer matmul -> fp32 dequant path.
Only tests, the smoke check and the CPU-baseline leg of the benchmark may import
it; the product (the CUDA library and its Python op surface) never does.

Pinning status
--------------
* pack / unpack / integer GEMM: pinned.  Checked against outputs of the
  reference's own CPU helpers (``int4_native_tc/test_correctness.py:20-54``,
  ``benchmark/verify_int4_matmul_precision.py:16-29``) executed on the
  reference's own seeds; see ``tests/golden/make_golden.py``.
* quantiser codes: **parity unpinned** by the reference's tests (they check only
  ranges, ``int4_native_tc/test_correctness.py:61-124``).  The reference CUDA
  kernel multiplies by ``7/absmax`` under fast-math
  (``int4_native_tc/csrc/int4_quant.cu:146,160-163``), which no CPU can
  reproduce; every torch restatement inside the reference divides by
  ``absmax/7`` instead (``benchmark/benchmark_w4a8fp8.py:200-204``,
  ``int4_native_tc/profile_bottleneck.py:21-29``).  The oracle and the CUDA
  kernels both use that second, IEEE-reproducible form (see ``quant_codes``).
* per-group dequant: the reference accumulates ``acc += float(mma) * sx * sw``
  (``int4_native_tc/csrc/int4_gemm.cu:1436,1859-1862``) and is built with
  ``--use_fast_math`` (``int4_native_tc/setup.py:52``), i.e. with multiply-add
  contraction: the compiled statement is ``acc = fma(float(mma) * sx, sw, acc)``.
  ``linear_grouped_f32`` states exactly that (one rounding for the product by
  ``sx``, one for the fused multiply-add), emulated exactly on the CPU by ``fma32``.
* MoE: **parity unpinned** (the reference has no MoE); it is a composition of
  the grouped quantiser and the grouped linear below, with SwiGLU stated as a
  formula of correctly rounded fp32 operations (``silu_mul``) so that a GPU
  kernel can reproduce it bit for bit.
"""
from __future__ import annotations

import numpy as np
import torch

F32 = np.float32
#: activation scale floor, ``int4_native_tc/csrc/int4_quant.cu:97``
K_MIN_SCALE = F32(1.0) / (F32(7.0) * F32(512.0))
GROUP = 128


def fma32(a, b, c) -> np.ndarray:
    """Correctly rounded fp32 fused multiply-add ``round(a * b + c)`` of float32 arrays.

    The product of two fp32 numbers is exact in float64; the sum with ``c`` is formed in float64 rounded to odd
    (error term from TwoSum), which makes the final rounding to fp32 the single rounding of the exact value."""
    a64 = np.asarray(a, dtype=F32).astype(np.float64)
    b64 = np.asarray(b, dtype=F32).astype(np.float64)
    c64 = np.asarray(c, dtype=F32).astype(np.float64)
    p = a64 * b64
    s = p + c64
    bb = s - p
    err = (p - (s - bb)) + (c64 - bb)
    bits = np.asarray(s).view(np.int64)
    need = (err != 0) & ((bits & 1) == 0) & np.isfinite(s)
    toward = np.where(err > 0, np.inf, -np.inf)
    s = np.where(need, np.nextafter(s, toward), s)
    return s.astype(F32)


# --------------------------------------------------------------------------- #
# pack / unpack  (int4_native_tc/test_correctness.py:20-48, int4_quant.cu:49-59)
# --------------------------------------------------------------------------- #
def pack_int4(codes: np.ndarray) -> np.ndarray:
    """[..., K] int codes in [-8, 7] -> [..., K/2] uint8, element 2i in the low nibble."""
    codes = np.asarray(codes)
    assert codes.shape[-1] % 2 == 0
    c = codes.astype(np.int16)
    lo = c[..., 0::2] & 0x0F
    hi = c[..., 1::2] & 0x0F
    return ((hi << 4) | lo).astype(np.uint8)


def unpack_int4(packed: np.ndarray) -> np.ndarray:
    """[..., K/2] uint8 -> [..., K] int8, sign-extending each nibble."""
    p = np.asarray(packed, dtype=np.uint8).astype(np.int16)
    lo = p & 0x0F
    hi = (p >> 4) & 0x0F
    lo = np.where(lo >= 8, lo - 16, lo)
    hi = np.where(hi >= 8, hi - 16, hi)
    out = np.empty(p.shape[:-1] + (p.shape[-1] * 2,), dtype=np.int8)
    out[..., 0::2] = lo
    out[..., 1::2] = hi
    return out


# --------------------------------------------------------------------------- #
# quantise
# --------------------------------------------------------------------------- #
def _to_f32(x) -> np.ndarray:
    """bf16/fp16/fp32 torch tensor or ndarray -> float32 ndarray (exact widening)."""
    if isinstance(x, torch.Tensor):
        return x.detach().to(torch.float32).cpu().numpy()
    return np.asarray(x, dtype=np.float32)


def quant_codes(xf: np.ndarray, absmax: np.ndarray) -> np.ndarray:
    """Canonical code arithmetic shared by the oracle and the CUDA kernels.

    ``q = clamp(rint(x / (absmax / 7)), -8, 7)`` with IEEE fp32 division and
    round-half-to-even; ``q = 0`` where ``absmax == 0``.  The divisor is the
    un-floored ``absmax/7``: the reference derives codes from ``absmax`` and
    applies the floor to the *returned* scale only (``int4_quant.cu:142,146``).
    ``absmax`` broadcasts against ``xf`` along the last axis.
    """
    s = (absmax.astype(F32) / F32(7.0)).astype(F32)
    safe = np.where(s == 0, F32(1.0), s).astype(F32)
    q = np.rint((xf.astype(F32) / safe).astype(F32))
    q = np.clip(q, -8.0, 7.0)
    q = np.where(s == 0, F32(0.0), q)
    return q.astype(np.int8)


def _scale_out(absmax: np.ndarray, role: str) -> np.ndarray:
    s = (absmax.astype(F32) / F32(7.0)).astype(F32)
    if role == "activation":  # int4_quant.cu:142, 789
        return np.maximum(s, K_MIN_SCALE).astype(F32)
    if role == "weight":  # int4_quant.cu:267, 692
        return np.where(absmax == 0, F32(1.0), s).astype(F32)
    raise ValueError(role)


def quant_rowwise(x, role: str = "activation"):
    """Per-row symmetric int4 (``dynamic_int4_quant`` / ``static_int4_weight_quant``,
    ``int4_quant.cu:201,289``).  Returns (codes int8 [R,K], scale f32 [R])."""
    xf = _to_f32(x)
    absmax = np.abs(xf).max(axis=1) if xf.shape[1] else np.zeros(xf.shape[0], F32)
    codes = quant_codes(xf, absmax[:, None])
    return codes, _scale_out(absmax, role)


def quant_grouped(x, group_size: int = GROUP, role: str = "activation"):
    """Per-(row, K-group) symmetric int4 with **group-major** outputs
    (``dynamic_int4_quant_grouped`` / ``static_int4_weight_quant_grouped``,
    ``int4_quant.cu:806,712``; layout ``:678-680,772-774``).
    Returns (codes int8 [G,R,gs], scale f32 [G,R])."""
    xf = _to_f32(x)
    R, K = xf.shape
    assert K % group_size == 0 and group_size % 2 == 0
    G = K // group_size
    xg = xf.reshape(R, G, group_size).transpose(1, 0, 2)  # [G,R,gs]
    absmax = np.abs(xg).max(axis=2)
    codes = quant_codes(xg, absmax[:, :, None])
    return np.ascontiguousarray(codes), _scale_out(absmax, role)


def quant_with_scales(x, scale: np.ndarray, group_size: int | None = None) -> np.ndarray:
    """Quantise with caller-supplied divisors: ``q = clamp(rint(x / scale), -8, 7)``.
    ``scale`` is [R] (row-wise; codes [R,K]) or [G,R] (grouped; codes [G,R,gs])."""
    xf = _to_f32(x)
    scale = np.asarray(scale, dtype=F32)
    if scale.ndim == 1:
        q = np.rint((xf / scale[:, None]).astype(F32))
    else:
        R, K = xf.shape
        G = scale.shape[0]
        gs = group_size or K // G
        xg = xf.reshape(R, G, gs).transpose(1, 0, 2)
        q = np.rint((xg / scale[:, :, None]).astype(F32))
    return np.ascontiguousarray(np.clip(q, -8, 7).astype(np.int8))


def _grouped_view(x, group_size: int, smooth_scale=None) -> np.ndarray:
    """[R,K] -> fp32 [G,R,gs]; divides by ``smooth_scale[k]`` first when given (IEEE fp32)."""
    xf = _to_f32(x)
    if smooth_scale is not None:
        xf = (xf / _to_f32(smooth_scale)[None, :]).astype(F32)
    R, K = xf.shape
    assert K % group_size == 0 and group_size % 2 == 0
    return np.ascontiguousarray(xf.reshape(R, K // group_size, group_size).transpose(1, 0, 2))


def quant_clipped_grouped(x, group_size: int = GROUP, clip_ratio: float = 1.0):
    """Per-(row, group) symmetric int4 whose range is ``absmax * clip_ratio``
    (``dynamic_int4_quant_clipped_grouped``, ``int4_quant.cu:857-903``): values beyond the
    clipped range saturate at -8 / 7 (``:898-901``), the returned scale is floored
    (``:889``).  Division form, like ``quant_codes``.  **Parity unpinned** (the reference has
    no golden vector for it).  Returns (codes int8 [G,R,gs], scale f32 [G,R])."""
    xg = _grouped_view(x, group_size)
    cm = (np.abs(xg).max(axis=2) * F32(clip_ratio)).astype(F32)
    codes = quant_codes(xg, cm[:, :, None])
    s = (cm / F32(7.0)).astype(F32)
    return np.ascontiguousarray(codes), np.maximum(s, K_MIN_SCALE).astype(F32)


def quant_asymmetric_grouped(x, group_size: int = GROUP, clip_ratio: float = 1.0, smooth_scale=None):
    """Per-(row, group) asymmetric int4 (``dynamic_int4_quant_asymmetric_grouped``,
    ``int4_quant.cu:1189-1259``; with clipping and SmoothQuant division
    ``dynamic_int4_quant_asymmetric_clipped_grouped``, ``:1324-1430``):

    ``c = clamp(v, -t, t)``, ``t = max|v| * clip_ratio``; ``s = max((max c - min c)/15, floor)``;
    ``azp = clamp(rint(-min c / s), 0, 15)``; ``u = clamp(rint(c / s + azp), 0, 15)``; the stored
    code is ``u - 8`` (``:1181-1186``) and ``azp_adj = 8 - azp`` (``:1237``).  The kernel multiplies by
    ``1/s`` under fast-math; the reference's torch restatement divides
    (``int4_native_tc/test_enhanced_quantization.py:262-268``) and that IEEE form is used here.
    **Parity unpinned.**  Returns (codes int8 [G,R,gs] in [-8,7], scale f32 [G,R], azp_adj f32 [G,R])."""
    xg = _grouped_view(x, group_size, smooth_scale)
    t = (np.abs(xg).max(axis=2) * F32(clip_ratio)).astype(F32)[:, :, None]
    c = np.minimum(np.maximum(xg, -t), t).astype(F32)
    mn = c.min(axis=2)
    mx = c.max(axis=2)
    s = np.maximum(((mx - mn).astype(F32) / F32(15.0)).astype(F32), K_MIN_SCALE).astype(F32)
    azp = np.clip(np.rint(((-mn).astype(F32) / s).astype(F32)), 0.0, 15.0).astype(F32)
    y = ((c / s[:, :, None]).astype(F32) + azp[:, :, None]).astype(F32)
    u = np.clip(np.rint(y), 0.0, 15.0)
    return np.ascontiguousarray((u - 8.0).astype(np.int8)), s, (F32(8.0) - azp).astype(F32)


def weight_group_sums(b_codes: np.ndarray) -> np.ndarray:
    """``w_col_sum[g,n] = sum_k codes[g,n,k]`` as fp32 (exact; ``int4_gemm.cu:991``)."""
    return np.asarray(b_codes).astype(np.int32).sum(axis=-1).astype(F32)


def linear_grouped_azp_f32(a_codes, b_codes, scale_a, scale_b, azp_adj, w_col_sum) -> np.ndarray:
    """Per-group linear with the zero-point term, before the final cast, in the reference's order:
    ``f = fma((float(acc_g) + azp_adj[g,m] * w_col_sum[g,n]) * sx[g,m], sw[g,n], f)``
    (``int4_gemm.cu:1851-1858``, contracted as the build flags make it; see the module header).
    The bracket is an exact integer below 2**24."""
    G, M, _ = a_codes.shape
    N = b_codes.shape[1]
    f = np.zeros((M, N), dtype=F32)
    for g in range(G):
        acc = int_gemm(a_codes[g], b_codes[g]).astype(F32)
        acc = (acc + (azp_adj[g].astype(F32)[:, None] * w_col_sum[g].astype(F32)[None, :]).astype(F32)).astype(F32)
        t = (acc * scale_a[g].astype(F32)[:, None]).astype(F32)
        f = fma32(t, np.broadcast_to(scale_b[g].astype(F32)[None, :], t.shape), f)
    return f


def quant_codes_refcuda_form(xf: np.ndarray, absmax: np.ndarray) -> np.ndarray:
    """The reference CUDA kernel's formulation ``rint(x * (7/absmax))`` evaluated
    in IEEE fp32 (``int4_quant.cu:146,160-163``).  Informational only: used to
    report how often it differs from ``quant_codes`` on near-tie inputs."""
    inv = np.where(absmax == 0, F32(0.0), F32(7.0) / np.where(absmax == 0, F32(1.0), absmax)).astype(F32)
    q = np.rint((xf.astype(F32) * inv).astype(F32))
    return np.clip(q, -8.0, 7.0).astype(np.int8)


def rmsnorm_quant_grouped(x: torch.Tensor, weight: torch.Tensor, eps: float, group_size: int = GROUP):
    """RMSNorm in front of the grouped activation quantiser, as the fused kernel states it (no reference
    counterpart: the reference quantises the output of a separate normalisation).

    Row statistic: 32 partial sums of squares, partial ``l`` taking elements ``1024 s + 32 l + (0..31)`` of the row
    in ascending order with one fused multiply-add each, added pairwise in a butterfly (distance 16, 8, 4, 2, 1);
    ``factor = 1 / sqrt(sum / K + eps)`` with correctly rounded division, addition and reciprocal square root.
    Value: ``bf16(bf16(x * factor) * weight[k])``, then ``quant_grouped(..., "activation")``.
    ``x`` bf16 [M, K] with K a multiple of 32; returns (codes [G, M, gs] int8, scale [G, M] fp32)."""
    xf = x.float().numpy().astype(F32)
    M, K = xf.shape
    assert K % 32 == 0
    nseg = (K + 1023) // 1024
    pad = np.zeros((M, nseg * 1024), dtype=F32)
    pad[:, :K] = xf
    lanes = pad.reshape(M, nseg, 32, 32)          # [row, segment, lane, element]
    ss = np.zeros((M, 32), dtype=F32)
    for sgm in range(nseg):
        for i in range(32):
            v = lanes[:, sgm, :, i]
            ss = fma32(v, v, ss)
    for o in (16, 8, 4, 2, 1):
        ss = (ss + ss[:, np.arange(32) ^ o]).astype(F32)
    tot = ss[:, 0]
    arg = ((tot / F32(K)).astype(F32) + F32(eps)).astype(F32)
    factor = (1.0 / np.sqrt(arg.astype(np.float64))).astype(F32)     # correctly rounded (float64 has bits to spare)
    y = torch.from_numpy((xf * factor[:, None]).astype(F32)).to(torch.bfloat16).float().numpy()
    y = torch.from_numpy((y * weight.float().numpy()[None, :]).astype(F32)).to(torch.bfloat16)
    return quant_grouped(y, group_size, "activation")


# --------------------------------------------------------------------------- #
# integer GEMM and dequant epilogues
# --------------------------------------------------------------------------- #
def int_gemm(a_codes: np.ndarray, b_codes: np.ndarray) -> np.ndarray:
    """``C[m,n] = sum_k A[m,k] * B[n,k]`` exactly, int32
    (``int4_native_tc/test_correctness.py:51-54``).

    For |code| <= 8 and K <= 2**17 every partial sum is an integer below 2**24,
    so an fp32 BLAS product of the float-cast codes is exact; larger K falls
    back to an int64 product."""
    a = np.asarray(a_codes)
    b = np.asarray(b_codes)
    K = a.shape[-1]
    if K * 64 < (1 << 24):
        return (a.astype(F32) @ b.astype(F32).T).astype(np.int32)
    return (a.astype(np.int64) @ b.astype(np.int64).T).astype(np.int32)


def int_gemm_int32_torch(a_codes: torch.Tensor, b_codes: torch.Tensor) -> torch.Tensor:
    """The reference's own formulation: ``torch.matmul`` on int32 operands
    (``benchmark/verify_int4_matmul_precision.py:23-25``).  This is the *timed*
    CPU baseline; ``int_gemm`` above is the fast exact checker."""
    return torch.matmul(a_codes.to(torch.int32), b_codes.to(torch.int32).T)


def to_bf16(f: np.ndarray) -> torch.Tensor:
    return torch.from_numpy(np.ascontiguousarray(f, dtype=F32)).to(torch.bfloat16)


def dequant_per_channel(acc: np.ndarray, scale_a: np.ndarray, scale_b: np.ndarray) -> np.ndarray:
    """``(float(acc) * scale_b[n]) * scale_a[m]`` in fp32, the order of the
    reference's scaled epilogue (``int4_gemm.cu:137-150``)."""
    t = (acc.astype(F32) * scale_b.astype(F32)[None, :]).astype(F32)
    return (t * scale_a.astype(F32)[:, None]).astype(F32)


def linear_per_channel(a_codes, b_codes, scale_a, scale_b) -> torch.Tensor:
    """Per-channel W4A4 linear -> bf16 [M,N] (``cutlass_int4_scaled_mm``, ``int4_gemm.cu:831``)."""
    return to_bf16(dequant_per_channel(int_gemm(a_codes, b_codes), scale_a, scale_b))


#: int8 activation scale floor, ``int4_native_tc/csrc/int4_quant.cu:423``
K_MIN_SCALE_INT8 = F32(1.0) / (F32(127.0) * F32(512.0))


def quant_rowwise_int8(x):
    """Per-token symmetric int8 (``dynamic_int8_quant``, ``int4_quant.cu:432-537``): ``scale = max(absmax / 127,
    1 / (127 * 512))`` (``:473``), ``q = clamp(rint(x / (absmax / 127)), -128, 127)``, zero rows give zero codes.
    The kernel multiplies by ``127 / absmax`` under fast-math (``:477,486``); as for the int4 quantisers the
    IEEE-reproducible division form is used here.  **Parity unpinned** (the reference's tests check this op only
    through loose end-to-end errors, ``test_correctness.py:589-615``).  Returns (int8 [R,K], fp32 [R])."""
    xf = _to_f32(x)
    absmax = np.abs(xf).max(axis=1) if xf.shape[1] else np.zeros(xf.shape[0], F32)
    s = (absmax.astype(F32) / F32(127.0)).astype(F32)
    safe = np.where(s == 0, F32(1.0), s).astype(F32)
    q = np.clip(np.rint((xf / safe[:, None]).astype(F32)), -128.0, 127.0)
    q = np.where((s == 0)[:, None], F32(0.0), q)
    return q.astype(np.int8), np.maximum(s, K_MIN_SCALE_INT8).astype(F32)


def linear_w4a8(a_int8, b_int8, scale_a, scale_b, dtype=torch.bfloat16) -> torch.Tensor:
    """W4A8 linear (``cutlass_w4a8_scaled_mm``, ``int4_gemm.cu:874-899``): exact int32 product of int8 activations and
    int4 weights held as int8 (``test_correctness.py:564``), then ``(float(acc) * scale_b[n]) * scale_a[m]`` in fp32
    (the scaled epilogue shared with the W4A4 op, ``int4_gemm.cu:137-150``), cast to ``dtype``."""
    acc = (np.asarray(a_int8).astype(np.int64) @ np.asarray(b_int8).astype(np.int64).T).astype(np.int32)
    f = dequant_per_channel(acc, scale_a, scale_b)
    return torch.from_numpy(np.ascontiguousarray(f, dtype=F32)).to(dtype)


def linear_grouped_f32(a_codes, b_codes, scale_a, scale_b) -> np.ndarray:
    """Per-group W4A4 linear before the final cast.  ``a_codes`` [G,M,gs],
    ``b_codes`` [G,N,gs], scales [G,M] / [G,N].  fp32 accumulation in ascending
    group order: ``f = fma(float(acc_g) * sx[g,m], sw[g,n], f)``, the reference's
    ``acc += float(mma) * sx * sw`` as its build flags contract it
    (``int4_gemm.cu:1436,1859-1862,2462``, ``setup.py:52``)."""
    G, M, _ = a_codes.shape
    N = b_codes.shape[1]
    f = np.zeros((M, N), dtype=F32)
    for g in range(G):
        acc = int_gemm(a_codes[g], b_codes[g]).astype(F32)
        t = (acc * scale_a[g].astype(F32)[:, None]).astype(F32)
        f = fma32(t, np.broadcast_to(scale_b[g].astype(F32)[None, :], t.shape), f)
    return f


def linear_grouped(a_codes, b_codes, scale_a, scale_b) -> torch.Tensor:
    """Per-group-128 W4A4 linear -> bf16 [M,N] (``cutlass_int4_fused_grouped_gemm``, ``int4_gemm.cu:4231``)."""
    return to_bf16(linear_grouped_f32(a_codes, b_codes, scale_a, scale_b))


def grouped_int_partials(a_codes, b_codes) -> np.ndarray:
    """int32 partial sums per group, [G,M,N]; the integer accumulators the fused kernel drains."""
    return np.stack([int_gemm(a_codes[g], b_codes[g]) for g in range(a_codes.shape[0])])


# --------------------------------------------------------------------------- #
# MoE composition (no reference counterpart; built from the functions above)
# --------------------------------------------------------------------------- #
def moe_route(logits: torch.Tensor, top_k: int = 8):
    """softmax over experts, top-k, renormalise the k weights to sum to one."""
    p = torch.softmax(logits.float(), dim=-1)
    w, idx = torch.topk(p, top_k, dim=-1)
    w = w / w.sum(dim=-1, keepdim=True)
    return idx.to(torch.int32), w.to(torch.float32)


def moe_sort(expert_ids: np.ndarray, num_experts: int):
    """Stable counting sort of the flattened (token, slot) pairs by expert.
    Returns (sorted_pair_ids [T*k], expert_offsets [E+1])."""
    flat = np.asarray(expert_ids).reshape(-1)
    order = np.argsort(flat, kind="stable").astype(np.int32)
    counts = np.bincount(flat, minlength=num_experts)
    offsets = np.zeros(num_experts + 1, dtype=np.int32)
    offsets[1:] = np.cumsum(counts)
    return order, offsets


_EXP_COEF = [F32(1.0 / 5040.0), F32(1.0 / 720.0), F32(1.0 / 120.0), F32(1.0 / 24.0), F32(1.0 / 6.0), F32(0.5),
             F32(1.0), F32(1.0)]
_LOG2E = F32(1.4426950408889634)
_LN2_HI = F32(0.693145751953125)
_LN2_LO = F32(1.428606765330187045e-06)


def exp_f32(t: np.ndarray) -> np.ndarray:
    """``e**t`` for fp32 ``t`` clamped to [-87, 87], as a fixed sequence of correctly rounded fp32 operations
    (no fused multiply-add): n = rint(t * log2(e)); r = (t - n * ln2_hi) - n * ln2_lo; a degree-7 Taylor polynomial
    of r by Horner's rule; times 2**n.  About 1 ulp; what matters is that a GPU kernel can repeat it exactly."""
    t = np.minimum(np.maximum(np.asarray(t, dtype=F32), F32(-87.0)), F32(87.0))
    n = np.rint((t * _LOG2E).astype(F32)).astype(F32)
    r = ((t - (n * _LN2_HI).astype(F32)).astype(F32) - (n * _LN2_LO).astype(F32)).astype(F32)
    p = np.full_like(r, _EXP_COEF[0])
    for c in _EXP_COEF[1:]:
        p = ((p * r).astype(F32) + c).astype(F32)
    return np.ldexp(p, n.astype(np.int32)).astype(F32)


def silu_mul_f32(g: np.ndarray, u: np.ndarray) -> np.ndarray:
    """``(g * sigmoid(g)) * u`` in fp32 with ``sigmoid(g) = 1 / (1 + exp_f32(-g))`` (IEEE division)."""
    g = np.asarray(g, dtype=F32)
    u = np.asarray(u, dtype=F32)
    sig = (F32(1.0) / (F32(1.0) + exp_f32(-g)).astype(F32)).astype(F32)
    return ((g * sig).astype(F32) * u).astype(F32)


def silu_mul(gate_up: torch.Tensor) -> torch.Tensor:
    """SwiGLU on a bf16 [R, 2I] tensor laid out [gate | up]; fp32 math (``silu_mul_f32``), bf16 result."""
    I = gate_up.shape[1] // 2
    g = gate_up[:, :I].float().numpy()
    u = gate_up[:, I:].float().numpy()
    return to_bf16(silu_mul_f32(g, u))


def moe_layer(x: torch.Tensor, expert_ids, expert_w, w_gate_up_q, w_down_q, num_experts: int):
    """Reference composition for one MoE layer.

    ``x`` bf16 [T,H]; ``expert_ids`` int [T,k]; ``expert_w`` f32 [T,k];
    ``w_gate_up_q[e] = (codes [G1,2I,gs], scale [G1,2I])`` and
    ``w_down_q[e] = (codes [G2,H,gs], scale [G2,H])`` are per-expert grouped
    weight quantisations.  Per expert: grouped-quantise its tokens, grouped
    linear -> bf16, SwiGLU -> bf16, grouped-quantise, grouped linear -> bf16;
    then ``out[t] = sum_j w[t,j] * y_j[t]`` accumulated in fp32 in ascending
    slot order j and cast to bf16."""
    T, H = x.shape
    k = expert_ids.shape[1]
    ids = np.asarray(expert_ids)
    y = torch.zeros(T, k, H, dtype=torch.float32)
    for e in range(num_experts):
        tok, slot = np.nonzero(ids == e)
        if tok.size == 0:
            continue
        xa, sa = quant_grouped(x[tok], GROUP, "activation")
        wq, ws = w_gate_up_q[e]
        h = linear_grouped(xa, wq, sa, ws)
        act = silu_mul(h)
        ha, hs = quant_grouped(act, GROUP, "activation")
        dq, ds = w_down_q[e]
        o = linear_grouped(ha, dq, hs, ds)
        y[tok, slot] = o.float()
    out = np.zeros((T, H), dtype=F32)
    wn = expert_w.float().numpy()
    yn = y.numpy()
    valid = (ids >= 0) & (ids < num_experts)
    for j in range(k):
        term = fma32(np.broadcast_to(wn[:, j : j + 1], (T, H)), yn[:, j], out)   # out = fma(w, y, out)
        out = np.where(valid[:, j : j + 1], term, out)
    return to_bf16(out)
