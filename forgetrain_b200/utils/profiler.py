"""Event-segment step profiler.

Opt-in through ``profile_range="start,end"`` + ``profile_output`` (both or neither). Inside the
range every ``mark(name)`` records a CUDA event (a ``perf_counter_ns`` stamp on CPU); marks are
"closing" marks: the segment called ``name`` is the time between the previous mark and this
one. Events are resolved only after the step's synchronisation, so profiling adds no sync of
its own. ``write()`` dumps ``{schema_version: 2, range, deep_mode, records, summary{n, mean,
median, p90, std, total}}`` atomically from rank 0. Same contract as the reference's
``StepProfiler`` (exports/train_engine_0.5B/src/training_engine_tensor/profiling.py:207-662).
"""
from __future__ import annotations

import json
import os
import statistics
import time
from pathlib import Path

import torch

# closing-mark names of the main loop and of a micro-batch in deep mode (the reference's
# SEG_* / DEEP_PHASE_* constants, profiling.py:180-204)
SEG_STEP_START, SEG_MICROBATCHES, SEG_REDUCE_SCATTER = "step_start", "microbatches", "reduce_scatter"
SEG_GRAD_NORM, SEG_OPTIMIZER, SEG_LOSS_ALLREDUCE, SEG_ALLGATHER = \
    "grad_norm", "optimizer", "loss_allreduce", "allgather"
DEEP_PHASE_DATA, DEEP_PHASE_FWD, DEEP_PHASE_CE, DEEP_PHASE_BWD, DEEP_PHASE_ACCUM = \
    "mb_data", "mb_fwd", "mb_ce", "mb_bwd", "mb_accum"
SEGMENTS = (SEG_STEP_START, SEG_MICROBATCHES, SEG_REDUCE_SCATTER, SEG_GRAD_NORM, SEG_OPTIMIZER,
            SEG_LOSS_ALLREDUCE, SEG_ALLGATHER)
DEEP_SEGMENTS = DEEP_PHASE_ORDER = (DEEP_PHASE_DATA, DEEP_PHASE_FWD, DEEP_PHASE_CE, DEEP_PHASE_BWD,
                                    DEEP_PHASE_ACCUM)


def _bucket_summary(records: list[dict], key: str, total_key: str | None = None) -> dict:
    names: dict[str, list[float]] = {}
    for r in records:
        for k, v in (r.get(key) or {}).items():
            names.setdefault(k, []).append(v)
        if total_key is not None and total_key in r:
            names.setdefault("total", []).append(r[total_key])
    out = {}
    for k, vals in names.items():
        s = sorted(vals)
        out[k] = {"n": len(s), "mean": statistics.fmean(s), "median": statistics.median(s),
                  "p90": s[min(len(s) - 1, int(0.9 * len(s)))],
                  "std": statistics.pstdev(s) if len(s) > 1 else 0.0, "total": sum(s)}
    return out


def summarize_segments(records: list[dict]) -> dict:
    """``{segment: {n, mean, median, p90, std, total}}`` over step records (those of a written
    profile or any subset of them, e.g. without the first steps); ``"total"`` is the whole step.
    No records give ``{}``. Counterpart of the reference's ``summarize_segments``
    (profiling.py:592-606)."""
    return _bucket_summary(records, "segments_ms", "total_ms")


def summarize_host_phases(records: list[dict]) -> dict:
    """The same statistics over the host-side intervals (``host_timer``); records without them
    are skipped (reference profiling.py:609-621)."""
    return _bucket_summary(records, "host_ms")


class _HostEvent:
    def __init__(self, clock):
        self.t = None
        self._clock = clock

    def record(self):
        self.t = self._clock()

    def elapsed_time(self, other: "_HostEvent") -> float:
        return (other.t - self.t) / 1e6


class StepProfiler:
    def __init__(self, start: int, end: int, output: str, deep: bool = False, host_timer: bool = False,
                 rank: int = 0, use_cuda: bool | None = None, event_factory=None, clock=None):
        if end <= start:
            raise ValueError(f"empty profile range {start},{end}")
        self.start, self.end, self.output = start, end, output
        self.deep, self.host_timer, self.rank = deep, host_timer, rank
        self.use_cuda = torch.cuda.is_available() if use_cuda is None else use_cuda
        self._clock = clock or time.perf_counter_ns
        if event_factory is not None:
            self._new_event = event_factory
        elif self.use_cuda:
            self._new_event = lambda: torch.cuda.Event(enable_timing=True)
        else:
            self._new_event = lambda: _HostEvent(self._clock)
        self.records: list[dict] = []
        self._step = None
        self._marks: list[tuple[str, object]] = []
        self._host: list[tuple[str, int]] = []
        self.active = False

    def begin_step(self, step: int) -> None:
        self._step = step
        self.active = self.start <= step < self.end
        self._marks, self._host = [], []
        if self.active:
            self.mark("step_start")

    def mark(self, name: str) -> None:
        if not self.active:
            return
        ev = self._new_event()
        ev.record()
        self._marks.append((name, ev))
        if self.host_timer:
            self._host.append((name, self._clock()))

    def deep_mark(self, name: str) -> None:
        if self.deep:
            self.mark(name)

    def end_step(self) -> None:
        """Call after the step's device synchronisation."""
        if not self.active or len(self._marks) < 2:
            self.active = False
            return
        seg: dict[str, float] = {}
        for (_, e0), (name, e1) in zip(self._marks[:-1], self._marks[1:]):
            seg[name] = seg.get(name, 0.0) + float(e0.elapsed_time(e1))
        rec = {"step": self._step, "segments_ms": seg,
               "total_ms": float(self._marks[0][1].elapsed_time(self._marks[-1][1]))}
        if self.host_timer and len(self._host) >= 2:
            rec["host_ms"] = {n1: (t1 - t0) / 1e6 for (_, t0), (n1, t1) in zip(self._host[:-1], self._host[1:])}
        self.records.append(rec)
        self.active = False

    def summary(self) -> dict:
        return summarize_segments(self.records)

    def write(self) -> str | None:
        if self.rank != 0:
            return None
        doc = {"schema_version": 2, "range": [self.start, self.end], "deep_mode": self.deep,
               "records": self.records, "summary": self.summary()}
        host = summarize_host_phases(self.records)
        if host:
            doc["host_summary"] = host
        path = Path(self.output)
        path.parent.mkdir(parents=True, exist_ok=True)
        tmp = path.with_suffix(path.suffix + ".tmp")
        tmp.write_text(json.dumps(doc, indent=1))
        os.replace(tmp, path)
        return str(path)


def parse_profile_range(text: str) -> tuple[int, int]:
    parts = [p.strip() for p in text.split(",")]
    if len(parts) != 2:
        raise ValueError(f"PROFILE_RANGE must be 'start,end', got {text!r}")
    a, b = int(parts[0]), int(parts[1])
    if a < 0 or b <= a:
        raise ValueError(f"PROFILE_RANGE needs 0 <= start < end, got {text!r}")
    return a, b


def profiler_from_config(cfg, rank: int = 0) -> StepProfiler | None:
    if bool(cfg.profile_range) != bool(cfg.profile_output):
        raise ValueError("PROFILE_RANGE and PROFILE_OUTPUT must be given together")
    if not cfg.profile_range:
        return None
    a, b = parse_profile_range(cfg.profile_range)
    return StepProfiler(a, b, cfg.profile_output, deep=cfg.profile_deep, host_timer=cfg.host_timer,
                        rank=rank)
