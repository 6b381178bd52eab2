"""``training_engine_tensor.entry``: the 8B engine's gate entry points under its module name
(entry.py:47-194)."""
from forgetrain_b200.entry import megatron_grad_names, run_forward, run_forward_backward  # noqa: F401
from forgetrain_b200.trainer import run_training_loop as run_training  # noqa: F401

__all__ = ["run_forward", "run_forward_backward", "run_training", "megatron_grad_names"]
