"""Pre-tokenised inputs: one fixed global batch replayed every step.

The reference's ``checkpoint-train-loop`` subcommand trains from a checkpoint on a ``.pt`` file of
already tokenised rows (``tokens``, ``labels``, ``loss_mask`` and optionally ``position_ids``, each
``[rows, seq]``); data-parallel rank ``r`` takes rows ``[r * mbs, (r + 1) * mbs)`` and the same rows
are used for every requested step, which is what makes the run comparable tensor by tensor with
another engine fed the same file (0.5B train_loop.py:487-505, __main__.py:140-146). With several
local micro-batches the rank's rows follow each other: micro-batch ``j`` of rank ``r`` is row block
``(r * n_mb + j)``.
"""
from __future__ import annotations

import torch


class FixedBatchSource:
    def __init__(self, path_or_dict, micro_batch_size: int, dp_rank: int = 0, dp_size: int = 1,
                 num_local_microbatches: int = 1, pin: bool = False):
        data = path_or_dict if isinstance(path_or_dict, dict) else \
            torch.load(path_or_dict, map_location="cpu", weights_only=False)
        for key in ("tokens", "labels"):
            if key not in data:
                raise KeyError(f"tokenised inputs lack {key!r} (have {sorted(data)})")
        rows = data["tokens"].shape[0]
        need = micro_batch_size * dp_size * num_local_microbatches
        if rows < need:
            raise ValueError(f"tokenised inputs hold {rows} rows; micro-batch {micro_batch_size} x "
                             f"{num_local_microbatches} micro-batches x {dp_size} ranks needs {need}")
        self.batches: list[dict[str, torch.Tensor]] = []
        for j in range(num_local_microbatches):
            lo = (dp_rank * num_local_microbatches + j) * micro_batch_size
            hi = lo + micro_batch_size
            b = {"tokens": data["tokens"][lo:hi].long().contiguous(),
                 "labels": data["labels"][lo:hi].long().contiguous()}
            mask = data.get("loss_mask")
            b["loss_mask"] = (mask[lo:hi].float() if mask is not None
                              else torch.ones(hi - lo, b["tokens"].shape[1])).contiguous()
            if "position_ids" in data:
                b["position_ids"] = data["position_ids"][lo:hi].to(torch.int32).contiguous()
            if pin and torch.cuda.is_available():
                b = {k: v.pin_memory() for k, v in b.items()}
            self.batches.append(b)
        self.seq_length = int(data["tokens"].shape[1])
        self.cursor = 0

    def __iter__(self):
        return self

    def __next__(self) -> dict[str, torch.Tensor]:
        b = self.batches[self.cursor % len(self.batches)]
        self.cursor += 1
        return b

    def state_dict(self) -> dict:
        return {"kind": "fixed", "cursor": self.cursor}

    def load_state_dict(self, st: dict) -> None:
        if st and st.get("kind") == "fixed":
            self.cursor = int(st.get("cursor", 0))
