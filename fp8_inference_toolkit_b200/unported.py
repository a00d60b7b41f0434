"""Ops of the reference surface that are outside the W4A4 hot path (grouped W4A8, W4A16, FP8 and
grouped int8-activation variants; ``int4_native_tc/int4_native_tc/__init__.py:86-122``).  They are exported so
that ``from int4_native_tc import *`` keeps working, and raise when called."""
from __future__ import annotations

UNPORTED = [
    "cutlass_w4a16_mm_grouped",
    "cutlass_w4a8_scaled_mm_grouped",
    "dequant_int4_to_bf16",
    "dequant_int4_to_fp16",
    "dynamic_int8_quant_grouped",
    "dynamic_int8_quant_asymmetric_grouped",
    "cutlass_int4_dequant_gemm_grouped",
    "dequant_int4_grouped_to_bf16",
    "unpack_int4_grouped_to_int8_contiguous",
    "unpack_int4_grouped_to_int8_weight",
    "progressive_int4_gemm_grouped",
    "dequant_int4_grouped_to_fp8",
    "dequant_int4_grouped_to_fp8_with_scales",
]


def _make(name: str):
    def _stub(*args, **kwargs):
        raise NotImplementedError(f"{name} is not part of the B200 W4A4 hot path and has not been ported")

    _stub.__name__ = name
    return _stub


for _n in UNPORTED:
    globals()[_n] = _make(_n)
