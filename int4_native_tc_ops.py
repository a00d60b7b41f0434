"""Drop-in for the reference's pybind11 module of the same name
(``int4_native_tc/csrc/bindings.cpp:208-309``): the 35 op names, plus the MoE ops."""
from fp8_inference_toolkit_b200.ops import (  # noqa: F401
    cutlass_int4_gemm,
    cutlass_int4_scaled_mm,
    cutlass_int4_scaled_mm_grouped,
    cutlass_w4a8_scaled_mm,
    dynamic_int8_quant,
    cutlass_int4_fused_grouped_gemm,
    cutlass_int4_fused_grouped_gemm_v5,
    cutlass_int4_fused_grouped_gemm_v7,
    cutlass_int4_fused_grouped_gemm_v8,
    cutlass_int4_fused_grouped_gemm_v9,
    cutlass_int4_fused_grouped_gemm_azp,
    cutlass_int4_fused_grouped_gemm_v5_azp,
    cutlass_int4_fused_grouped_gemm_v7_azp,
    cutlass_int4_scaled_mm_azp_grouped,
    dynamic_int4_quant,
    static_int4_weight_quant,
    unpack_int4_to_int8,
    static_int4_weight_quant_grouped,
    dynamic_int4_quant_grouped,
    dynamic_int4_quant_clipped_grouped,
    dynamic_int4_quant_asymmetric_grouped,
    dynamic_int4_quant_asymmetric_clipped_grouped,
    int4_weight_group_sums,
    int4_quant_with_scales,
    int4_grouped_partials,
)
from fp8_inference_toolkit_b200.moe import moe_sort_tokens, moe_w4a4_grouped_gemm  # noqa: F401
from fp8_inference_toolkit_b200.unported import *  # noqa: F401,F403
from fp8_inference_toolkit_b200.unported import UNPORTED as _UNPORTED

for _n in _UNPORTED:
    globals()[_n] = getattr(__import__("fp8_inference_toolkit_b200.unported", fromlist=[_n]), _n)
