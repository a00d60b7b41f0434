from fp8_inference_toolkit_b200.calibration import apply_smoothing_to_weight, compute_smoothing_factors  # noqa: F401
