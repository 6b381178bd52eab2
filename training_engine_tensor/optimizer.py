"""``training_engine_tensor.optimizer``: schedule and sharded AdamW under the reference's module name
(0.5B optimizer.py:9-24, 8B optimizer.py:16-25)."""
from forgetrain_b200.optim.adamw import ShardedAdamW  # noqa: F401
from forgetrain_b200.optim.lr import compute_lr  # noqa: F401

__all__ = ["compute_lr", "ShardedAdamW"]
