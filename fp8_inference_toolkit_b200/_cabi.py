"""ctypes binding of ``libint4tc_b200.so`` (the C ABI declared in ``include/int4tc_b200.h``).

There is no fallback: if the library has not been built, importing this module raises.
"""
from __future__ import annotations

import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "csrc", "libint4tc_b200.so")

BF16, FP16, FP32, INT32 = 0, 1, 2, 3
ROLE_ACTIVATION, ROLE_WEIGHT = 0, 1

_p = C.c_void_p
_i = C.c_int
_l = C.c_int64
_f = C.c_float
_d = C.c_double

#: name -> (restype, argtypes); must list every symbol of include/int4tc_b200.h
SIGNATURES = {
    "i4tc_version": (_i, []),
    "i4tc_last_error": (C.c_char_p, []),
    "i4tc_sm_count": (_i, [_i]),
    "i4tc_set_tuning": (_i, [_i, _i]),
    "i4tc_set_split_k": (_i, [_i]),
    "i4tc_set_cta_pairs": (_i, [_i]),
    "i4tc_set_epilogue_warps": (_i, [_i]),
    "i4tc_set_small_m_path": (_i, [_i]),
    "i4tc_reserve_workspace": (_i, [_i, _p, _l]),
    "i4tc_workspace_bytes": (_l, [_i, _p]),
    "i4tc_release_workspaces": (_i, [_i]),
    "i4tc_quant_rowwise": (_i, [_p, _i, _l, _l, _l, _p, _p, _i, _i, _p]),
    "i4tc_quant_grouped": (_i, [_p, _i, _l, _l, _l, _l, _p, _p, _i, _i, _p]),
    "i4tc_quant_with_scales": (_i, [_p, _i, _l, _l, _l, _l, _p, _p, _i, _p]),
    "i4tc_quant_clipped_grouped": (_i, [_p, _i, _l, _l, _l, _l, _d, _p, _p, _i, _p]),
    "i4tc_quant_asymmetric_grouped": (_i, [_p, _i, _l, _l, _l, _l, _d, _p, _p, _p, _p, _i, _p]),
    "i4tc_weight_group_sums": (_i, [_p, _l, _l, _p, _i, _p]),
    "i4tc_unpack_int4_to_int8": (_i, [_p, _l, _l, _p, _i, _p]),
    "i4tc_gemm_int32": (_i, [_p, _p, _p, _l, _l, _l, _i, _p]),
    "i4tc_gemm_scaled": (_i, [_p, _p, _p, _p, _p, _i, _l, _l, _l, _i, _p]),
    "i4tc_gemm_w4a8_scaled": (_i, [_p, _p, _p, _p, _p, _i, _l, _l, _l, _i, _p]),
    "i4tc_quant_rowwise_int8": (_i, [_p, _i, _l, _l, _l, _p, _p, _i, _p]),
    "i4tc_gemm_grouped": (_i, [_p, _p, _p, _p, _p, _l, _l, _l, _l, _i, _p]),
    "i4tc_gemm_grouped_azp": (_i, [_p, _p, _p, _p, _p, _p, _p, _l, _l, _l, _l, _i, _p]),
    "i4tc_gemm_grouped_int32": (_i, [_p, _p, _p, _l, _l, _l, _i, _p]),
    "i4tc_moe_sort_scratch_bytes": (_l, [_l, _l]),
    "i4tc_moe_sort": (_i, [_p, _l, _l, _p, _p, _p, _p, _l, _i, _p]),
    "i4tc_moe_sort_noalloc_max_scratch_ints": (_l, []),
    "i4tc_moe_sort_noalloc": (_i, [_p, _l, _l, _p, _p, _p, _i, _p]),
    "i4tc_moe_sort_noalloc_prepare": (_i, [_i]),
    "i4tc_moe_ep_plan": (_i, [_p, _p, _l, _l, _l, _l, _l, _p, _p, _p, _p, _p, _l, _i, _p]),
    "i4tc_moe_ep_dispatch_quant": (_i, [_p, _l, _l, _l, _p, _l, _l, _p, _p, _l, _p, _l, _l, _i, _p]),
    "i4tc_peer_signal": (_i, [_p, _l, C.c_uint32, _i, _p]),
    "i4tc_peer_wait": (_i, [_p, _l, C.c_uint32, _i, _p]),
    "i4tc_peer_signal_counter": (_i, [_p, _l, _p, _i, _i, _p]),
    "i4tc_peer_wait_counter": (_i, [_p, _l, _p, _i, _p]),
    "i4tc_moe_ep_meta_ints": (_l, [_l, _l]),
    "i4tc_moe_ep_unpack": (_i, [_p, _l, _l, _l, _l, _l, _p, _p, _p, _p, _p, _p, _i, _p]),
    "i4tc_moe_silu_mul_quant_rows": (_i, [_p, _l, _p, _l, _p, _p, _i, _p]),
    "i4tc_moe_ep_pack_return": (_i, [_p, _p, _l, _l, _p, _p, _p, _l, _l, _l, _i, _p]),
    "i4tc_moe_gather_packed": (_i, [_p, _p, _l, _l, _p, _l, _l, _p, _p, _p, _l, _p, _l, _l, _i, _p]),
    "i4tc_moe_gather_quant": (_i, [_p, _i, _l, _l, _l, _p, _l, _l, _p, _p, _i, _p]),
    "i4tc_moe_grouped_gemm": (_i, [_p, _p, _p, _p, _p, _p, _l, _l, _l, _l, _i, _p]),
    "i4tc_moe_grouped_gemm_rows": (_i, [_p, _p, _p, _p, _p, _p, _l, _l, _l, _l, _i, _p]),
    "i4tc_moe_ep_return_rows": (_i, [_p, _l, _l, _p, _p, _l, _l, _l, _p, _i, _p]),
    "i4tc_moe_silu_mul_quant": (_i, [_p, _l, _l, _p, _p, _i, _p]),
    "i4tc_rmsnorm_quant_grouped": (_i, [_p, _l, _l, _l, _p, _f, _l, _p, _p, _i, _p]),
    "i4tc_moe_combine": (_i, [_p, _p, _p, _l, _l, _l, _p, _i, _p]),
    "i4tc_check_status": (_i, [_i, _p]),
}


def _load() -> C.CDLL:
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            f"{LIB_PATH} is missing: build it with `python fp8_inference_toolkit_b200/build.py` "
            "(needs nvcc). There is no CPU or PyTorch fallback for these ops."
        )
    lib = C.CDLL(LIB_PATH)
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)  # AttributeError if the library does not export it
        fn.restype = res
        fn.argtypes = args
    return lib


lib = _load()


def last_error() -> str:
    msg = lib.i4tc_last_error()
    return msg.decode("utf-8", "replace") if msg else ""


def check(rc: int, what: str) -> None:
    """Turn a C-ABI status into the ``RuntimeError`` the reference's TORCH_CHECK would raise."""
    if rc != 0:
        raise RuntimeError(f"{what}: {last_error()} (status {rc})")
