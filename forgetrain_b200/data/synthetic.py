"""Seeded synthetic token source: uniform ids in ``[0, vocab)``, labels = inputs shifted by
one, loss mask all ones. Batches are produced on the host (pinned when CUDA is present) so the
training loop pays the same host-to-device copy a real loader would. Each data-parallel rank
draws from its own stream (``seed + 1000003 * dp_rank``); the stream position is the only
state, so resuming from ``state_dict()`` continues the exact sequence.

The reference prints "using synthetic random data" but has no such path
(exports/train_engine_0.5B/src/training_engine_tensor/__main__.py:479-481 vs
train_loop.py:489-491); this is the one it lacks.
"""
from __future__ import annotations

import torch


class SyntheticTokenSource:
    def __init__(self, vocab_size: int, micro_batch_size: int, seq_length: int, seed: int = 1234,
                 dp_rank: int = 0, pin: bool | None = None, distinct_batches: int = 0):
        self.vocab_size = vocab_size
        self.mbs = micro_batch_size
        self.seq = seq_length
        self.seed = seed
        self.dp_rank = dp_rank
        self.gen = torch.Generator(device="cpu")
        self.gen.manual_seed(seed + 1000003 * dp_rank)
        self.batches_drawn = 0
        self.pin = torch.cuda.is_available() if pin is None else pin
        # > 0: cycle over that many fixed batches (memorisation runs / loss-decrease checks)
        self.distinct = distinct_batches
        self._cache: list[torch.Tensor] = []

    def __iter__(self):
        return self

    def __next__(self) -> dict[str, torch.Tensor]:
        if self.distinct > 0 and len(self._cache) == self.distinct:
            chunk = self._cache[self.batches_drawn % self.distinct]
        else:
            chunk = torch.randint(0, self.vocab_size, (self.mbs, self.seq + 1), generator=self.gen,
                                  dtype=torch.int64)
            if self.distinct > 0:
                self._cache.append(chunk)
        self.batches_drawn += 1
        batch = {
            "tokens": chunk[:, :-1].contiguous(),
            "labels": chunk[:, 1:].contiguous(),
            "loss_mask": torch.ones(self.mbs, self.seq, dtype=torch.float32),
        }
        if self.pin:
            batch = {k: v.pin_memory() for k, v in batch.items()}
        return batch

    def state_dict(self) -> dict:
        return {"kind": "synthetic", "seed": self.seed, "dp_rank": self.dp_rank,
                "batches_drawn": self.batches_drawn}

    def load_state_dict(self, st: dict) -> None:
        if not st or st.get("kind") != "synthetic":
            return
        self.gen.manual_seed(self.seed + 1000003 * self.dp_rank)
        self.batches_drawn = 0
        for _ in range(int(st.get("batches_drawn", 0))):
            torch.randint(0, self.vocab_size, (self.mbs, self.seq + 1), generator=self.gen,
                          dtype=torch.int64)
            self.batches_drawn += 1
