"""Data-parallel gradient reduction over the flat fp32 gradient buffer (ZeRO-1 style).

Weight gradients are written in place into the flat buffer by the backward pass, so there is
no pack / cast step: when the last parameter of a bucket reports ready on the last micro-batch
the bucket is averaged over the data-parallel group and reduce-scattered *in place* (each rank
ends up with the reduced values of its own shard inside the same buffer), on a side stream, so
the reduction overlaps the rest of the backward pass. The squared norm of the reduced shard is
accumulated for gradient clipping.

Two backends do the reduction:

* ``fused``: one sm_100a kernel per bucket over NVLink peer memory
  (:mod:`forgetrain_b200.parallel.fused_dp`): loads of every peer's slice (or an in-switch
  ``multimem`` reduction), the 1/W scale and the squared-norm partial in a single pass.
* ``nccl`` (``gloo`` on CPU): ``torch.distributed`` reduce-scatter; the selectable baseline.

Behavioural spec: the reference's ``BucketedGradReducer``
(exports/train_engine_0.5B/src/training_engine_tensor/nccl.py:654-1152, 1454-1513).
"""
from __future__ import annotations

import torch
import torch.distributed as dist

from .buckets import Bucket, compute_grad_buckets


class BucketedGradReducer:
    def __init__(self, flat_grads: torch.Tensor, entries, world: int, rank: int, group,
                 target_elems: int, backend: str = "nccl", overlap: bool = True,
                 norm_exclude: list[tuple[int, int]] | None = None, fused=None,
                 all_reduce: bool = False):
        self.flat = flat_grads
        self.world, self.rank, self.group = world, rank, group
        self.backend = backend
        self.buckets: list[Bucket] = compute_grad_buckets(entries, world, target_elems)
        self.bucket_of: dict[str, int] = {n: b.index for b in self.buckets for n in b.params}
        self.is_cuda = flat_grads.is_cuda
        self.overlap = overlap and self.is_cuda and world > 1
        self.comm_stream = torch.cuda.Stream(device=flat_grads.device) if self.overlap else None
        self.done_events: list = [None] * len(self.buckets)
        self.pending = [0] * len(self.buckets)
        self.seen: set[str] = set()
        self.fused = fused
        # True: every rank ends up with the WHOLE reduced bucket (unsharded optimizer); the norm
        # is still accumulated over this rank's shard only, so the sum over ranks stays correct
        self.all_reduce = all_reduce
        # ranges (absolute offsets) left out of the norm on this rank (TP-duplicated params)
        self.norm_exclude = norm_exclude or []
        self.sumsq = torch.zeros(1, dtype=torch.float32, device=flat_grads.device)
        self._active = False

    # ------------------------------------------------------------------ lifecycle
    def start_step(self) -> None:
        for b in self.buckets:
            self.pending[b.index] = len(b.params)
            self.done_events[b.index] = None
        self.seen.clear()
        self.sumsq.zero_()
        self._active = True

    def on_grad_ready(self, name: str) -> None:
        """Called by the backward pass of the LAST micro-batch when ``name``'s gradient is
        complete in the flat buffer."""
        if not self._active:
            raise RuntimeError("on_grad_ready outside start_step()/wait_all()")
        bi = self.bucket_of.get(name)
        if bi is None:
            raise KeyError(f"unknown parameter {name!r}")
        if name in self.seen:
            raise RuntimeError(f"gradient of {name!r} reported twice in one step")
        self.seen.add(name)
        self.pending[bi] -= 1
        if self.pending[bi] == 0:
            self._issue_bucket_reduce(self.buckets[bi])

    def shard_view(self, b: Bucket) -> torch.Tensor:
        lo, hi = b.shard_range(self.rank, self.world)
        return self.flat[lo:hi]

    def bucket_view(self, b: Bucket) -> torch.Tensor:
        return self.flat[b.start:b.start + b.size]

    def _issue_bucket_reduce(self, b: Bucket) -> None:
        if self.world == 1:
            self._accumulate_norm(b)
            return
        if self.overlap:
            ev = torch.cuda.Event()
            ev.record()
            self.comm_stream.wait_event(ev)
            ctx = torch.cuda.stream(self.comm_stream)
        else:
            ctx = _null_ctx()
        with ctx:
            if self.fused is not None:
                self.fused.reduce_scatter_bucket(b, self.sumsq)
            else:
                view = self.bucket_view(b)
                view.mul_(1.0 / self.world)
                if self.is_cuda and not self.all_reduce:
                    dist.reduce_scatter_tensor(self.shard_view(b), view, group=self.group)
                else:
                    dist.all_reduce(view, group=self.group)
                self._accumulate_norm(b)
            if self.overlap:
                done = torch.cuda.Event()
                done.record()
                self.done_events[b.index] = done

    def _accumulate_norm(self, b: Bucket) -> None:
        sh = self.shard_view(b)
        if self.is_cuda:
            from ..ops import cuda_ops
            cuda_ops.sumsq_into(sh, self.sumsq)
        else:
            self.sumsq += sh.pow(2).sum()

    def wait_all(self) -> None:
        """Make the current stream wait for every issued reduction (no host sync)."""
        if not self._active:
            return
        missing = [b.index for b in self.buckets if self.pending[b.index] != 0]
        if missing:
            raise RuntimeError(f"buckets {missing} never became ready: "
                               f"{sum(self.pending[i] for i in missing)} gradients not reported")
        if self.overlap:
            for ev in self.done_events:
                if ev is not None:
                    torch.cuda.current_stream().wait_event(ev)
        self._active = False

    # ------------------------------------------------------------------ gradient norm
    def local_sumsq(self) -> torch.Tensor:
        """Sum of squares of this rank's reduced shards minus the excluded ranges."""
        out = self.sumsq.clone()
        for lo, hi in self.norm_exclude:
            for b in self.buckets:
                s_lo, s_hi = b.shard_range(self.rank, self.world)
                a, z = max(lo, s_lo), min(hi, s_hi)
                if z > a:
                    out -= self.flat[a:z].pow(2).sum()
        return out


class _null_ctx:
    def __enter__(self):
        return self

    def __exit__(self, *a):
        return False
