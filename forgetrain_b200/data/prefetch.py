"""Host-to-device batch prefetcher on a dedicated copy stream.

Keeps up to ``depth`` (1..4) batches in flight: each batch is copied with non-blocking
transfers on the copy stream and carries an event; ``next()`` makes the compute stream wait
for that event only and records the consuming stream on every tensor it hands out. Batches whose loss mask is entirely zero are skipped. On CPU it degrades
to a pass-through FIFO so the state machine can be unit-tested without a GPU. Behavioural
spec: exports/train_engine_0.5B/src/training_engine_tensor/data.py:37-185.
"""
from __future__ import annotations

from collections import deque
from typing import Iterable, Iterator

import torch


class DataPrefetcher:
    def __init__(self, source: Iterable[dict], device, depth: int = 2, skip_all_masked: bool = True,
                 stream_factory=None, event_factory=None):
        if not 1 <= depth <= 4:
            raise ValueError("depth must be in 1..4")
        self.source: Iterator[dict] = iter(source)
        self.device = torch.device(device)
        self.depth = depth
        self.skip_all_masked = skip_all_masked
        self.cuda = self.device.type == "cuda"
        if stream_factory is not None:
            self.stream = stream_factory()
        else:
            self.stream = torch.cuda.Stream(device=self.device) if self.cuda else None
        self._event_factory = event_factory or ((lambda: torch.cuda.Event()) if self.cuda else None)
        self.queue: deque = deque()
        self.exhausted = False
        self.skipped = 0
        self.bytes_last = 0
        # batches taken from the source so far (skipped ones included), and how many of them lie
        # at or before the batch handed out last: the position a checkpoint has to record
        self.drawn = 0
        self.consumed_from_source = 0

    def _fetch_one(self) -> bool:
        while True:
            try:
                host = next(self.source)
            except StopIteration:
                self.exhausted = True
                return False
            self.drawn += 1
            m = host.get("loss_mask")
            if self.skip_all_masked and m is not None and float(m.sum()) == 0.0:
                self.skipped += 1
                continue
            break
        nbytes = sum(v.numel() * v.element_size() for v in host.values() if torch.is_tensor(v))
        if self.stream is not None:
            ctx = torch.cuda.stream(self.stream) if self.cuda else _Null()
            with ctx:
                dev = {k: (v.to(self.device, non_blocking=True) if torch.is_tensor(v) else v)
                       for k, v in host.items()}
                ev = self._event_factory() if self._event_factory else None
                if ev is not None:
                    ev.record(self.stream) if self.cuda else ev.record()
        else:
            dev = {k: (v.to(self.device) if torch.is_tensor(v) else v) for k, v in host.items()}
            ev = None
        self.queue.append((dev, ev, host, nbytes, self.drawn))
        return True

    def _fill(self) -> None:
        while len(self.queue) < self.depth and not self.exhausted:
            if not self._fetch_one():
                break

    def __iter__(self):
        return self

    def __next__(self) -> dict:
        self._fill()
        if not self.queue:
            raise StopIteration
        dev, ev, host, nbytes, position = self.queue.popleft()
        self.consumed_from_source = position
        if ev is not None:
            if self.cuda:
                cur = torch.cuda.current_stream()
                cur.wait_event(ev)
                # The tensors were allocated on the copy stream and are consumed on the compute
                # stream: tell the caching allocator, or it may hand a batch's block to the next
                # host-to-device copy while a kernel of the consuming step (the embedding
                # backward runs last) has not read it yet. Same discipline as the reference's
                # reducer buffers (nccl.py:1077-1084).
                for v in dev.values():
                    if torch.is_tensor(v):
                        v.record_stream(cur)
            else:
                ev.wait()
                self._record(dev)
        self.bytes_last = nbytes
        self._keepalive = host  # pinned source must outlive the async copy
        self._fill()
        return dev


    def _record(self, dev: dict) -> None:
        """CPU stand-in of the record_stream step (counted so the state machine is testable)."""
        self.recorded_tensors = getattr(self, "recorded_tensors", 0) + sum(
            1 for v in dev.values() if torch.is_tensor(v))


class _Null:
    def __enter__(self):
        return self

    def __exit__(self, *a):
        return False
