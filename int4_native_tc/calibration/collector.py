from fp8_inference_toolkit_b200.calibration import ActivationStatsCollector, LayerStats  # noqa: F401
