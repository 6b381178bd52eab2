"""``training_engine_tensor.kernels``: the functional op layer under the reference's module name
(0.5B kernels.py, 8B kernels.py). CUDA tensors run the sm_100a kernels, CPU tensors the plain
PyTorch statement of the same op."""
from forgetrain_b200.ops import (  # noqa: F401
    add_rmsnorm_fwd, attention_bwd, attention_fwd, cross_entropy_fwd_bwd, embedding_bwd, embedding_fwd,
    linear_dgrad, linear_fwd, linear_swiglu_fwd, linear_wgrad, rmsnorm_bwd, rope_, rope_tables,
    swiglu_bwd, swiglu_fwd)

__all__ = ["embedding_fwd", "embedding_bwd", "add_rmsnorm_fwd", "rmsnorm_bwd", "rope_", "rope_tables",
           "attention_fwd", "attention_bwd", "swiglu_fwd", "swiglu_bwd", "linear_fwd",
           "linear_swiglu_fwd", "linear_dgrad", "linear_wgrad", "cross_entropy_fwd_bwd"]
