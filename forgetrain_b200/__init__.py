"""forgetrain_b200: a Blackwell-native (sm_100a) LLM pretraining engine.

PyTorch is the framework layer (process groups, memory, streams); every hot op is a
hand-written CUDA kernel in ``csrc/`` (tcgen05 / TMEM / TMA GEMM and FlashAttention, fused
memory-bound kernels, peer-memory collectives) loaded from an in-tree shared library.
"""
from .config import ModelSpec, load_model_spec  # noqa: F401
from .engine_config import EngineConfig, get_config, set_global_config  # noqa: F401

__all__ = ["ModelSpec", "load_model_spec", "EngineConfig", "get_config", "set_global_config"]
__version__ = "0.1.0"
