"""CPU: the C-ABI library builds, loads without a GPU and exports every symbol the header declares."""
import ctypes
import os
import re

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared_symbols():
    text = open(os.path.join(ROOT, "include", "int4tc_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(i4tc_[a-z0-9_]+)\s*\(", text)))


def test_header_symbols_exported(lib_built):
    lib = ctypes.CDLL(lib_built)
    names = _declared_symbols()
    assert len(names) >= 18
    for n in names:
        assert hasattr(lib, n), f"{n} declared in include/int4tc_b200.h but not exported"


def test_binding_table_matches_header(lib_built):
    from fp8_inference_toolkit_b200 import _cabi

    assert sorted(_cabi.SIGNATURES) == _declared_symbols()
    assert _cabi.lib.i4tc_version() >= 100


def test_argument_errors_need_no_gpu(lib_built):
    from fp8_inference_toolkit_b200 import _cabi

    lib = _cabi.lib
    # rejected before any CUDA call
    assert lib.i4tc_quant_rowwise(None, 0, 4, 7, 7, None, None, 0, 0, None) == -1
    assert "even" in _cabi.last_error()
    assert lib.i4tc_gemm_grouped(None, None, None, None, None, 4, 4, 64, 2, 0, None) == -3
    assert "group_size=128" in _cabi.last_error()
    assert lib.i4tc_gemm_int32(None, None, None, 4, 4, 100, 0, None) == -1
    assert lib.i4tc_set_tuning(96, 0) == -1
    assert lib.i4tc_moe_sort_scratch_bytes(4096 * 8, 128) == 32 * 128 * 4


def test_ops_reject_cpu_tensors(lib_built):
    import int4_native_tc

    with pytest.raises(RuntimeError, match="CUDA"):
        int4_native_tc.dynamic_int4_quant(torch.zeros(2, 8, dtype=torch.bfloat16))
    with pytest.raises(RuntimeError, match="CUDA"):
        int4_native_tc.static_int4_weight_quant_grouped(torch.zeros(2, 128), 128)
    with pytest.raises(NotImplementedError):
        int4_native_tc.cutlass_w4a8_scaled_mm_grouped()
    # the whole reference surface is importable
    import int4_native_tc_ops

    for n in int4_native_tc.__all__:
        assert callable(getattr(int4_native_tc_ops, n))
