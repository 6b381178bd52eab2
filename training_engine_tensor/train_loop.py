"""``training_engine_tensor.train_loop``: the training loop under the reference's module name (its
train_loop.py:400-1061 and, for the 8B engine, entry.py:126-780)."""
from forgetrain_b200.trainer import Trainer, run_training_loop  # noqa: F401

__all__ = ["run_training_loop", "Trainer"]
