"""Alias package: keeps the reference's entry point ``python -m training_engine_tensor
pretrain ...`` working on top of :mod:`forgetrain_b200`."""
from forgetrain_b200 import *  # noqa: F401,F403
