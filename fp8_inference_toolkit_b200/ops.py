"""PyTorch-facing op surface: same names, argument order, dtypes, shapes and return conventions
as the reference extension ``int4_native_tc_ops`` (``int4_native_tc/csrc/bindings.cpp:208-309``).

PyTorch is only plumbing here: it owns the device memory and the stream; every op is one or more
calls into the C-ABI library.  Quantise ops allocate and return their outputs, scaled GEMMs write
into the caller's ``out`` and return ``None`` -- the reference's ownership rules
(``int4_quant.cu:209-212``, ``int4_gemm.cu:831-837``).
"""
from __future__ import annotations

import torch

from . import _cabi
from ._cabi import check, lib

_DTYPES = {torch.bfloat16: _cabi.BF16, torch.float16: _cabi.FP16, torch.float32: _cabi.FP32}


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def _dev(t: torch.Tensor) -> int:
    return t.device.index if t.device.index is not None else torch.cuda.current_device()


def _stream(t: torch.Tensor) -> int:
    """Handle of torch's current stream on the tensor's device (the stream the reference launches on)."""
    if _raw_stream is not None:
        return _raw_stream(_dev(t))
    return torch.cuda.current_stream(t.device).cuda_stream


def _require(cond: bool, msg: str) -> None:
    if not cond:
        raise RuntimeError(msg)


def _cuda2d(t: torch.Tensor, name: str) -> None:
    _require(isinstance(t, torch.Tensor) and t.is_cuda, f"{name} must be CUDA tensor")
    _require(t.dim() == 2, f"{name} must be 2D")


def _float_input(t: torch.Tensor, name: str) -> torch.Tensor:
    _require(t.dtype in _DTYPES, f"{name} must be bfloat16, float16 or float32")
    if t.stride(1) != 1 or (t.stride(0) * t.element_size()) % 16 != 0 or t.data_ptr() % 16 != 0:
        t = t.contiguous()
    return t


def _same_device(*ts: torch.Tensor) -> None:
    d = ts[0].device
    for t in ts[1:]:
        _require(t.device == d, "all tensors must be on the same device")


def _packed(t: torch.Tensor, name: str) -> torch.Tensor:
    _require(t.is_cuda, f"{name} must be CUDA tensor")
    _require(t.dtype == torch.uint8, f"{name} must be uint8")
    _require(t.is_contiguous(), f"{name} must be contiguous")
    return t


def _f32(t: torch.Tensor, name: str, numel: int) -> torch.Tensor:
    _require(t.is_cuda and t.dtype == torch.float32, f"{name} must be a float32 CUDA tensor")
    _require(t.is_contiguous(), f"{name} must be contiguous")
    _require(t.numel() == numel, f"{name} has {t.numel()} elements, expected {numel}")
    return t


# --------------------------------------------------------------------------- #
# quantise / pack
# --------------------------------------------------------------------------- #
def _quant_rowwise(x: torch.Tensor, role: int, who: str):
    _cuda2d(x, "input" if role == _cabi.ROLE_ACTIVATION else "weight")
    R, K = x.shape
    _require(K % 2 == 0, "K must be even for INT4 packing")
    x = _float_input(x, who)
    packed = torch.empty((R, K // 2), dtype=torch.uint8, device=x.device)
    scale = torch.empty((R,), dtype=torch.float32, device=x.device)
    check(lib.i4tc_quant_rowwise(x.data_ptr(), _DTYPES[x.dtype], R, K, x.stride(0), packed.data_ptr(),
                                 scale.data_ptr(), role, _dev(x), _stream(x)), who)
    return packed, scale


def _quant_grouped(x: torch.Tensor, group_size: int, role: int, who: str):
    _cuda2d(x, "input" if role == _cabi.ROLE_ACTIVATION else "weight")
    R, K = x.shape
    group_size = int(group_size)
    _require(group_size > 0 and K % group_size == 0, "K must be divisible by group_size")
    _require(group_size % 2 == 0, "group_size must be even")
    x = _float_input(x, who)
    G = K // group_size
    packed = torch.empty((G, R, group_size // 2), dtype=torch.uint8, device=x.device)
    scale = torch.empty((G, R), dtype=torch.float32, device=x.device)
    check(lib.i4tc_quant_grouped(x.data_ptr(), _DTYPES[x.dtype], R, K, x.stride(0), group_size,
                                 packed.data_ptr(), scale.data_ptr(), role, _dev(x), _stream(x)), who)
    return packed, scale


def dynamic_int4_quant(input: torch.Tensor):
    """[M,K] -> (packed u8 [M,K/2], scale f32 [M]).  Reference: ``int4_quant.cu:201``."""
    return _quant_rowwise(input, _cabi.ROLE_ACTIVATION, "dynamic_int4_quant")


def static_int4_weight_quant(weight: torch.Tensor):
    """[N,K] -> (packed u8 [N,K/2], scale f32 [N]).  Reference: ``int4_quant.cu:289``."""
    return _quant_rowwise(weight, _cabi.ROLE_WEIGHT, "static_int4_weight_quant")


def dynamic_int4_quant_grouped(input: torch.Tensor, group_size: int):
    """[M,K] -> (packed u8 [G,M,gs/2], scale f32 [G,M]).  Reference: ``int4_quant.cu:806``."""
    return _quant_grouped(input, group_size, _cabi.ROLE_ACTIVATION, "dynamic_int4_quant_grouped")


def static_int4_weight_quant_grouped(weight: torch.Tensor, group_size: int):
    """[N,K] -> (packed u8 [G,N,gs/2], scale f32 [G,N]).  Reference: ``int4_quant.cu:712``."""
    return _quant_grouped(weight, group_size, _cabi.ROLE_WEIGHT, "static_int4_weight_quant_grouped")


def _ext_input(input: torch.Tensor, group_size: int, who: str):
    _cuda2d(input, "input")
    _require(input.dtype in (torch.bfloat16, torch.float16), f"{who}: input must be bfloat16 or float16")
    M, K = input.shape
    _require(group_size > 0 and K % group_size == 0, "K must be divisible by group_size")
    _require(group_size % 2 == 0, "group_size must be even")
    if input.stride(1) != 1:
        input = input.contiguous()
    return input, M, K, K // group_size


def dynamic_int4_quant_clipped_grouped(input: torch.Tensor, group_size: int, clip_ratio: float):
    """[M,K] -> (packed u8 [G,M,gs/2], scale f32 [G,M]) with the range ``absmax * clip_ratio`` per group.
    Reference: ``int4_quant.cu:906`` (checks ``:909-916``)."""
    x, M, K, G = _ext_input(input, group_size, "dynamic_int4_quant_clipped_grouped")
    _require(0.0 < clip_ratio <= 1.0, "clip_ratio must be in (0, 1]")
    packed = torch.empty((G, M, group_size // 2), dtype=torch.uint8, device=x.device)
    scale = torch.empty((G, M), dtype=torch.float32, device=x.device)
    check(lib.i4tc_quant_clipped_grouped(x.data_ptr(), _DTYPES[x.dtype], M, K, x.stride(0), int(group_size),
                                         float(clip_ratio), packed.data_ptr(), scale.data_ptr(), _dev(x),
                                         _stream(x)), "dynamic_int4_quant_clipped_grouped")
    return packed, scale


def dynamic_int4_quant_asymmetric_clipped_grouped(input: torch.Tensor, group_size: int, clip_ratio: float,
                                                  smooth_scale: torch.Tensor | None = None):
    """[M,K] -> (packed u8 [G,M,gs/2], scale f32 [G,M], azp_adj f32 [G,M]); asymmetric codes stored as
    ``u - 8``, optional division by ``smooth_scale`` [K] (same dtype as the input) and symmetric clipping first.
    Reference: ``int4_quant.cu:1433`` (checks ``:1437-1470``)."""
    who = "dynamic_int4_quant_asymmetric_clipped_grouped"
    x, M, K, G = _ext_input(input, group_size, who)
    _require(0.0 < clip_ratio <= 1.0, "clip_ratio must be in (0, 1]")
    sm_ptr = None
    if smooth_scale is not None:
        _require(smooth_scale.is_cuda and smooth_scale.dtype == x.dtype, "smooth_scale must match the input's dtype")
        _require(smooth_scale.numel() == K, "smooth_scale must be [K]")
        _same_device(x, smooth_scale)
        smooth_scale = smooth_scale.contiguous()
        sm_ptr = smooth_scale.data_ptr()
    packed = torch.empty((G, M, group_size // 2), dtype=torch.uint8, device=x.device)
    scale = torch.empty((G, M), dtype=torch.float32, device=x.device)
    azp_adj = torch.empty((G, M), dtype=torch.float32, device=x.device)
    check(lib.i4tc_quant_asymmetric_grouped(x.data_ptr(), _DTYPES[x.dtype], M, K, x.stride(0), int(group_size),
                                            float(clip_ratio), sm_ptr, packed.data_ptr(), scale.data_ptr(),
                                            azp_adj.data_ptr(), _dev(x), _stream(x)), who)
    return packed, scale, azp_adj


def dynamic_int4_quant_asymmetric_grouped(input: torch.Tensor, group_size: int):
    """[M,K] -> (packed, scale, azp_adj) without clipping or smoothing.  Reference: ``int4_quant.cu:1262``."""
    return dynamic_int4_quant_asymmetric_clipped_grouped(input, group_size, 1.0, None)


def int4_weight_group_sums(b_packed: torch.Tensor) -> torch.Tensor:
    """Group-major packed weights u8 [G,N,gs/2] -> ``w_col_sum`` f32 [G,N], the sum of each group's codes (the
    operand the reference's callers build in torch, ``int4_native_tc/profile_layer.py:96-119``)."""
    _packed(b_packed, "b_packed")
    _require(b_packed.dim() == 3 and b_packed.shape[2] % 4 == 0, "b_packed must be [G, N, gs/2] with gs % 8 == 0")
    G, N, half = b_packed.shape
    out = torch.empty((G, N), dtype=torch.float32, device=b_packed.device)
    check(lib.i4tc_weight_group_sums(b_packed.data_ptr(), G * N, 2 * half, out.data_ptr(), _dev(out),
                                     _stream(out)), "int4_weight_group_sums")
    return out


def rmsnorm_int4_quant_grouped(input: torch.Tensor, norm_weight: torch.Tensor, eps: float, group_size: int = 128):
    """RMSNorm fused in front of the grouped quantiser (no reference op; the reference's report names the fusion as
    its follow-up).  bf16 [M,K], bf16 [K] -> (packed u8 [G,M,gs/2], scale f32 [G,M]) of
    ``bf16(bf16(x * rsqrt(mean(x^2) + eps)) * norm_weight)``."""
    _cuda2d(input, "input")
    _require(input.dtype == torch.bfloat16 and norm_weight.dtype == torch.bfloat16, "input and norm_weight must be bfloat16")
    _require(input.stride(1) == 1, "input rows must be contiguous")
    _same_device(input, norm_weight)
    M, K = input.shape
    _require(norm_weight.is_contiguous() and norm_weight.numel() == K, "norm_weight must be a contiguous [K] tensor")
    _require(group_size > 0 and K % group_size == 0, "K must be divisible by group_size")
    G = K // group_size
    packed = torch.empty((G, M, group_size // 2), dtype=torch.uint8, device=input.device)
    scale = torch.empty((G, M), dtype=torch.float32, device=input.device)
    check(lib.i4tc_rmsnorm_quant_grouped(input.data_ptr(), M, K, input.stride(0), norm_weight.data_ptr(), float(eps),
                                         int(group_size), packed.data_ptr(), scale.data_ptr(), _dev(input),
                                         _stream(input)), "rmsnorm_int4_quant_grouped")
    return packed, scale


def int4_quant_with_scales(input: torch.Tensor, scale: torch.Tensor, group_size: int = 0):
    """Quantise with caller-supplied divisors (no reference op; the "identical scales" form used to
    compare codes bit for bit).  ``scale`` [M] -> packed [M,K/2]; ``scale`` [G,M] -> packed [G,M,gs/2]."""
    _cuda2d(input, "input")
    R, K = input.shape
    x = _float_input(input, "int4_quant_with_scales")
    _same_device(x, scale)
    if group_size:
        G = K // group_size
        _f32(scale, "scale", G * R)
        packed = torch.empty((G, R, group_size // 2), dtype=torch.uint8, device=x.device)
    else:
        _f32(scale, "scale", R)
        packed = torch.empty((R, K // 2), dtype=torch.uint8, device=x.device)
    check(lib.i4tc_quant_with_scales(x.data_ptr(), _DTYPES[x.dtype], R, K, x.stride(0), int(group_size),
                                     scale.data_ptr(), packed.data_ptr(), _dev(x), _stream(x)),
          "int4_quant_with_scales")
    return packed


def unpack_int4_to_int8(packed: torch.Tensor, K: int) -> torch.Tensor:
    """packed u8 [N,K/2] -> int8 [N,K].  Reference: ``int4_quant.cu:593``."""
    _require(packed.is_cuda, "packed must be CUDA tensor")
    _require(packed.dim() == 2, "packed must be 2D [N, K/2]")
    _require(packed.dtype == torch.uint8, "packed must be uint8")
    _require(packed.size(1) * 2 == K, "packed.size(1) must equal K/2")
    packed = packed.contiguous()
    N = packed.size(0)
    out = torch.empty((N, K), dtype=torch.int8, device=packed.device)
    check(lib.i4tc_unpack_int4_to_int8(packed.data_ptr(), N, K, out.data_ptr(), _dev(packed), _stream(packed)),
          "unpack_int4_to_int8")
    return out


# --------------------------------------------------------------------------- #
# GEMMs
# --------------------------------------------------------------------------- #
def cutlass_int4_gemm(a_packed: torch.Tensor, b_packed: torch.Tensor, M: int, N: int, K: int) -> torch.Tensor:
    """int32 [M,N] = A[M,K] . B[N,K]^T over packed int4.  Reference: ``int4_gemm.cu:779``."""
    _packed(a_packed, "a_packed")
    _packed(b_packed, "b_packed")
    _same_device(a_packed, b_packed)
    _require(K % 64 == 0, "K must be a multiple of 64")
    _require(a_packed.numel() == M * (K // 2), "a_packed does not have M*K/2 bytes")
    _require(b_packed.numel() == N * (K // 2), "b_packed does not have N*K/2 bytes")
    out = torch.empty((M, N), dtype=torch.int32, device=a_packed.device)
    check(lib.i4tc_gemm_int32(a_packed.data_ptr(), b_packed.data_ptr(), out.data_ptr(), M, N, K,
                              _dev(a_packed), _stream(a_packed)), "cutlass_int4_gemm")
    return out


def cutlass_int4_scaled_mm(a_packed, b_packed, scale_a, scale_b, out, M: int, N: int, K: int) -> None:
    """out[m,n] = cast((acc * scale_b[n]) * scale_a[m]) into the caller's bf16/fp16 ``out``.
    Reference: ``int4_gemm.cu:831``."""
    _packed(a_packed, "a_packed")
    _packed(b_packed, "b_packed")
    _same_device(a_packed, b_packed, scale_a, scale_b, out)
    _require(K % 64 == 0, "K must be a multiple of 64")
    _require(out.dtype in (torch.bfloat16, torch.float16), "out must be bfloat16 or float16")
    _require(out.is_contiguous() and out.numel() == M * N, "out must be a contiguous [M,N] tensor")
    _require(a_packed.numel() == M * (K // 2), "a_packed does not have M*K/2 bytes")
    _require(b_packed.numel() == N * (K // 2), "b_packed does not have N*K/2 bytes")
    _f32(scale_a, "scale_a", M)
    _f32(scale_b, "scale_b", N)
    check(lib.i4tc_gemm_scaled(a_packed.data_ptr(), b_packed.data_ptr(), scale_a.data_ptr(), scale_b.data_ptr(),
                               out.data_ptr(), _DTYPES[out.dtype], M, N, K, _dev(out), _stream(out)),
          "cutlass_int4_scaled_mm")


def dynamic_int8_quant(input: torch.Tensor):
    """[M,K] float -> (int8 [M,K], fp32 scale [M]): per-token symmetric int8, ``scale = max(absmax / 127, 1/(127*512))``.
    Reference: ``int4_quant.cu:511`` (kernel ``:432``)."""
    _cuda2d(input, "input")
    x = _float_input(input, "input")
    M, K = x.shape
    q = torch.empty((M, K), dtype=torch.int8, device=x.device)
    scale = torch.empty((M,), dtype=torch.float32, device=x.device)
    check(lib.i4tc_quant_rowwise_int8(x.data_ptr(), _DTYPES[x.dtype], M, K, x.stride(0), q.data_ptr(), scale.data_ptr(),
                                      _dev(x), _stream(x)), "dynamic_int8_quant")
    return q, scale


def cutlass_w4a8_scaled_mm(a, b_int8, scale_a, scale_b, out, M: int, N: int, K: int) -> None:
    """``out[m,n] = cast((sum_k a[m,k] * b_int8[n,k]) * scale_b[n] * scale_a[m])`` with int8 ``a`` [M,K] and the int4
    weight held as int8 ``b_int8`` [N,K] (``unpack_int4_to_int8``).  Reference: ``int4_gemm.cu:874-899``."""
    _require(a.is_cuda and b_int8.is_cuda, "Inputs must be CUDA")
    _require(scale_a.is_cuda and scale_b.is_cuda, "Scales must be CUDA")
    _require(out.is_cuda, "Output must be CUDA")
    _require(K % 32 == 0, "K must be multiple of 32 for INT8 alignment")
    _require(a.dtype == torch.int8, "a must be int8")
    _require(b_int8.dtype == torch.int8, "b_int8 must be int8")
    _require(out.dtype in (torch.bfloat16, torch.float16),
             "cutlass_w4a8_scaled_mm: unsupported output dtype, must be bfloat16 or float16")
    _same_device(a, b_int8, scale_a, scale_b, out)
    _require(a.is_contiguous() and a.numel() == M * K, "a must be a contiguous [M,K] tensor")
    _require(b_int8.is_contiguous() and b_int8.numel() == N * K, "b_int8 must be a contiguous [N,K] tensor")
    _require(out.is_contiguous() and out.numel() == M * N, "out must be a contiguous [M,N] tensor")
    _f32(scale_a, "scale_a", M)
    _f32(scale_b, "scale_b", N)
    check(lib.i4tc_gemm_w4a8_scaled(a.data_ptr(), b_int8.data_ptr(), scale_a.data_ptr(), scale_b.data_ptr(),
                                    out.data_ptr(), _DTYPES[out.dtype], M, N, K, _dev(out), _stream(out)),
          "cutlass_w4a8_scaled_mm")


def cutlass_int4_fused_grouped_gemm(a_packed, b_packed, scale_a, scale_b, out, M: int, N: int,
                                    group_size: int, num_groups: int) -> None:
    """Per-group-128 fused linear into the caller's bf16 ``out`` [M,N].
    Reference: ``int4_gemm.cu:4231`` (checks at ``:4243-4252``)."""
    _packed(a_packed, "a_packed")
    _packed(b_packed, "b_packed")
    _same_device(a_packed, b_packed, scale_a, scale_b, out)
    _require(group_size == 128, "fused grouped GEMM only supports group_size=128")
    _require(out.dtype == torch.bfloat16, "fused grouped GEMM only supports BF16 output")
    _require(out.is_contiguous() and out.numel() == M * N, "out must be a contiguous [M,N] tensor")
    _require(a_packed.numel() == num_groups * M * 64, "a_packed must be [G, M, 64]")
    _require(b_packed.numel() == num_groups * N * 64, "b_packed must be [G, N, 64]")
    _f32(scale_a, "scale_a", num_groups * M)
    _f32(scale_b, "scale_b", num_groups * N)
    check(lib.i4tc_gemm_grouped(a_packed.data_ptr(), b_packed.data_ptr(), scale_a.data_ptr(),
                                scale_b.data_ptr(), out.data_ptr(), M, N, group_size, num_groups,
                                _dev(out), _stream(out)), "cutlass_int4_fused_grouped_gemm")


# Same contract, different kernels in the reference (int4_gemm.cu:3751, 4073, 4007, 3932).
cutlass_int4_fused_grouped_gemm_v5 = cutlass_int4_fused_grouped_gemm
cutlass_int4_fused_grouped_gemm_v7 = cutlass_int4_fused_grouped_gemm
cutlass_int4_fused_grouped_gemm_v8 = cutlass_int4_fused_grouped_gemm
cutlass_int4_fused_grouped_gemm_v9 = cutlass_int4_fused_grouped_gemm


def cutlass_int4_scaled_mm_grouped(a_packed, b_packed, scale_a, scale_b, out, M: int, N: int, group_size: int,
                                   num_groups: int) -> None:
    """The reference's per-group loop of scaled GEMMs (``int4_gemm.cu:929-992``), served here by the fused kernel:
    a narrower contract -- ``group_size`` 128 and bf16 output only, and no rounding of each group's product to the
    output type before the fp32 accumulation (the reference's loop accepts any multiple of 64 and fp16)."""
    _require(group_size == 128, "cutlass_int4_scaled_mm_grouped: this build serves group_size=128 only "
                                f"(got {group_size}; the reference accepts any multiple of 64)")
    _require(out.dtype == torch.bfloat16, "cutlass_int4_scaled_mm_grouped: this build writes bfloat16 only "
                                         f"(got {out.dtype}; the reference also accepts float16)")
    cutlass_int4_fused_grouped_gemm(a_packed, b_packed, scale_a, scale_b, out, M, N, group_size, num_groups)


def cutlass_int4_fused_grouped_gemm_azp(a_packed, b_packed, scale_a, scale_b, out, azp_adj, w_col_sum, M: int,
                                        N: int, group_size: int, num_groups: int) -> None:
    """Per-group-128 fused linear with the zero-point term of asymmetric activations into the caller's bf16
    ``out`` [M,N]: ``sum_g sa*sb*(acc_g + azp_adj[g,m]*w_col_sum[g,n])``.  Reference: ``int4_gemm.cu:4298``."""
    _packed(a_packed, "a_packed")
    _packed(b_packed, "b_packed")
    _same_device(a_packed, b_packed, scale_a, scale_b, out, azp_adj, w_col_sum)
    _require(group_size == 128, "fused grouped GEMM only supports group_size=128")
    _require(out.dtype == torch.bfloat16, "cutlass_int4_fused_grouped_gemm_azp currently supports BF16 output only")
    _require(out.is_contiguous() and out.numel() == M * N, "out must be a contiguous [M,N] tensor")
    _require(a_packed.numel() == num_groups * M * 64, "a_packed must be [G, M, 64]")
    _require(b_packed.numel() == num_groups * N * 64, "b_packed must be [G, N, 64]")
    _f32(scale_a, "scale_a", num_groups * M)
    _f32(scale_b, "scale_b", num_groups * N)
    _f32(azp_adj, "azp_adj", num_groups * M)
    _f32(w_col_sum, "w_col_sum", num_groups * N)
    check(lib.i4tc_gemm_grouped_azp(a_packed.data_ptr(), b_packed.data_ptr(), scale_a.data_ptr(),
                                    scale_b.data_ptr(), azp_adj.data_ptr(), w_col_sum.data_ptr(), out.data_ptr(),
                                    M, N, group_size, num_groups, _dev(out), _stream(out)),
          "cutlass_int4_fused_grouped_gemm_azp")


# Same contract, different kernels in the reference (int4_gemm.cu:3838, 4149).
cutlass_int4_fused_grouped_gemm_v5_azp = cutlass_int4_fused_grouped_gemm_azp
cutlass_int4_fused_grouped_gemm_v7_azp = cutlass_int4_fused_grouped_gemm_azp


def cutlass_int4_scaled_mm_azp_grouped(a_packed, b_packed, scale_a, scale_b, out, azp_adj, w_col_sum, M: int, N: int,
                                       group_size: int, num_groups: int) -> None:
    """The reference's per-group loop with the zero-point term (``int4_gemm.cu:994-1000``), served by the fused
    kernel under the same narrower contract as ``cutlass_int4_scaled_mm_grouped``."""
    _require(group_size == 128, "cutlass_int4_scaled_mm_azp_grouped: this build serves group_size=128 only "
                                f"(got {group_size}; the reference accepts any multiple of 64)")
    _require(out.dtype == torch.bfloat16, "cutlass_int4_scaled_mm_azp_grouped: this build writes bfloat16 only "
                                         f"(got {out.dtype}; the reference also accepts float16)")
    cutlass_int4_fused_grouped_gemm_azp(a_packed, b_packed, scale_a, scale_b, out, azp_adj, w_col_sum, M, N, group_size,
                                        num_groups)


def int4_grouped_partials(a_packed, b_packed, M: int, N: int, num_groups: int) -> torch.Tensor:
    """int32 [G,M,N]: the per-group integer accumulators of the fused kernel (no reference op)."""
    _packed(a_packed, "a_packed")
    _packed(b_packed, "b_packed")
    _same_device(a_packed, b_packed)
    _require(a_packed.numel() == num_groups * M * 64, "a_packed must be [G, M, 64]")
    _require(b_packed.numel() == num_groups * N * 64, "b_packed must be [G, N, 64]")
    out = torch.empty((num_groups, M, N), dtype=torch.int32, device=a_packed.device)
    check(lib.i4tc_gemm_grouped_int32(a_packed.data_ptr(), b_packed.data_ptr(), out.data_ptr(), M, N,
                                      num_groups, _dev(out), _stream(out)), "int4_grouped_partials")
    return out


def set_tuning(tile_n: int = 0, swap: int = -1) -> None:
    """Force the GEMM tile width / operand orientation (tests); ``set_tuning()`` restores automatic."""
    check(lib.i4tc_set_tuning(tile_n, swap), "set_tuning")


def set_split_k(splits: int = 0) -> None:
    """Force the number of K ranges of the small-M per-group GEMM (tests); 0 restores automatic."""
    check(lib.i4tc_set_split_k(splits), "set_split_k")


def set_cta_pairs(mode: int = -1) -> None:
    """Force (1) or forbid (0) 256 x 256 tiles on SM pairs for large dense GEMMs (tests); -1 restores automatic."""
    check(lib.i4tc_set_cta_pairs(mode), "set_cta_pairs")


def set_small_m_path(path: int = 0) -> None:
    """Test / tuning hook: 0 = automatic, 1 = CUDA-core kernel only, 2 = register-fed tensor-core kernel wherever it
    applies (1..32 tokens), 3 = always the tile kernel."""
    check(lib.i4tc_set_small_m_path(path), "set_small_m_path")


def set_epilogue_warps(warps: int = 0) -> None:
    """Force 8 or 16 epilogue warps per thread block of the tensor-core GEMM (tests); 0 restores automatic."""
    check(lib.i4tc_set_epilogue_warps(warps), "set_epilogue_warps")


def reserve_workspace(nbytes: int, device=None, stream=None) -> None:
    """Make the split-K workspace of (device, stream) at least ``nbytes`` large now, so that no small-M GEMM on that
    stream allocates later (call before capturing a CUDA graph).  Defaults: current device, its current stream."""
    dev = torch.cuda.current_device() if device is None else torch.device(device).index
    st = torch.cuda.current_stream(dev) if stream is None else stream
    check(lib.i4tc_reserve_workspace(dev, st.cuda_stream, int(nbytes)), "reserve_workspace")


def workspace_bytes(device=None, stream=None) -> int:
    """Current size of the split-K workspace of (device, stream); 0 if none was needed yet."""
    dev = torch.cuda.current_device() if device is None else torch.device(device).index
    st = torch.cuda.current_stream(dev) if stream is None else stream
    return int(lib.i4tc_workspace_bytes(dev, st.cuda_stream))


def check_status(device=None) -> None:
    """Raise if any kernel gave up on a bounded wait since the last call (synchronises the stream)."""
    dev = torch.cuda.current_device() if device is None else torch.device(device).index
    check(lib.i4tc_check_status(dev, torch.cuda.current_stream(dev).cuda_stream), "check_status")
