"""Learning-rate schedules.

WSD (warmup - stable - decay) exactly as the reference's ``compute_lr``
(exports/train_engine_0.5B/src/training_engine_tensor/optimizer.py:162-195):
linear warmup to ``max_lr``; constant until ``decay_iters - wsd_decay_iters``; then
``min + (2 * 0.5**r - 1) * (max - min)`` with ``r`` the fraction of the decay window done;
``min_lr`` after ``decay_iters``. ``it`` is the optimizer step count before its increment.
With ``wsd_decay_iters == 0`` this is the 8B engine's warmup-then-constant schedule.
"""
from __future__ import annotations


def compute_lr(it: int, max_lr: float, min_lr: float, warmup_iters: int, lr_decay_iters: int,
               wsd_decay_iters: int) -> float:
    if warmup_iters > 0 and it < warmup_iters:
        return max_lr * it / warmup_iters
    if wsd_decay_iters <= 0:
        return max_lr if it <= lr_decay_iters else min_lr
    stable_end = lr_decay_iters - wsd_decay_iters
    if it <= stable_end:
        return max_lr
    if it > lr_decay_iters:
        return min_lr
    r = (it - stable_end) / wsd_decay_iters
    return min_lr + (2.0 * 0.5 ** r - 1.0) * (max_lr - min_lr)
