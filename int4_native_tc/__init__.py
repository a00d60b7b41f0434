"""Drop-in for the reference's ``int4_native_tc`` package
(``int4_native_tc/int4_native_tc/__init__.py:48-122``): re-exports the op surface."""
import int4_native_tc_ops as _ops

__all__ = [
    "cutlass_int4_gemm", "cutlass_int4_scaled_mm", "cutlass_w4a8_scaled_mm", "cutlass_w4a16_mm_grouped",
    "cutlass_int4_scaled_mm_grouped", "cutlass_int4_scaled_mm_azp_grouped", "cutlass_w4a8_scaled_mm_grouped",
    "cutlass_int4_fused_grouped_gemm", "cutlass_int4_fused_grouped_gemm_azp",
    "cutlass_int4_fused_grouped_gemm_v5", "cutlass_int4_fused_grouped_gemm_v5_azp",
    "cutlass_int4_fused_grouped_gemm_v7", "cutlass_int4_fused_grouped_gemm_v7_azp",
    "cutlass_int4_fused_grouped_gemm_v8", "cutlass_int4_fused_grouped_gemm_v9",
    "dynamic_int4_quant", "dynamic_int8_quant", "static_int4_weight_quant", "unpack_int4_to_int8",
    "dequant_int4_to_bf16", "dequant_int4_to_fp16", "static_int4_weight_quant_grouped",
    "dynamic_int4_quant_grouped", "dynamic_int4_quant_clipped_grouped",
    "dynamic_int4_quant_asymmetric_grouped", "dynamic_int4_quant_asymmetric_clipped_grouped",
    "dynamic_int8_quant_grouped", "dynamic_int8_quant_asymmetric_grouped",
    "cutlass_int4_dequant_gemm_grouped", "dequant_int4_grouped_to_bf16",
    "unpack_int4_grouped_to_int8_contiguous", "unpack_int4_grouped_to_int8_weight",
    "progressive_int4_gemm_grouped", "dequant_int4_grouped_to_fp8", "dequant_int4_grouped_to_fp8_with_scales",
    # additions without a reference counterpart
    "moe_sort_tokens", "moe_w4a4_grouped_gemm", "int4_quant_with_scales", "int4_grouped_partials",
    "int4_weight_group_sums",
]
for _n in __all__:
    globals()[_n] = getattr(_ops, _n)
