"""Drop-in for the reference's ``calibration`` package (``int4_native_tc/calibration/__init__.py``)."""
from fp8_inference_toolkit_b200.calibration import (  # noqa: F401
    ActivationStatsCollector,
    LayerStats,
    apply_smoothing_to_weight,
    compute_smoothing_factors,
)

__all__ = ["ActivationStatsCollector", "LayerStats", "apply_smoothing_to_weight", "compute_smoothing_factors"]
