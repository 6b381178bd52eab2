"""``training_engine_tensor.config``: model spec, FLOP accounting and muP helpers under the
reference's module name (its config.py:53-202). The reference keeps one model's constants at module
level; here they are fields of a :class:`ModelSpec`, and the helper functions take the spec."""
from forgetrain_b200.config import (  # noqa: F401
    ModelSpec, compute_training_flops, compute_training_flops_standard, forward_flops_per_token,
    load_model_spec, peak_tflops, validate_spec)


def mup_width_scale(spec: ModelSpec) -> float:
    """hidden / base width: logit divisor and hidden-matrix LR divisor."""
    return spec.mup_width_scale


def mup_residual_scale(spec: ModelSpec) -> float:
    """depth_scale / sqrt(layers): multiplier of every residual branch."""
    return spec.mup_residual_scale


def mtp_per_layer_loss_scale(factor: float, num_layers: int) -> float:
    return factor / num_layers if num_layers > 0 else 0.0


__all__ = ["ModelSpec", "load_model_spec", "validate_spec", "compute_training_flops",
           "compute_training_flops_standard", "forward_flops_per_token", "peak_tflops",
           "mup_width_scale", "mup_residual_scale", "mtp_per_layer_loss_scale"]
