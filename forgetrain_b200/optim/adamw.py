"""ZeRO-1 sharded AdamW over the flat buffers.

Each data-parallel rank keeps fp32 master weights and both moments only for its shard of every
gradient bucket. One fused kernel launch per bucket applies clip * grad, the moment updates,
bias correction, decoupled weight decay and the per-parameter muP learning-rate multiplier
(from a small segment table), and writes the new bf16 value directly at the shard's position in
the flat parameter buffer, which is the all-gather destination, so the all-gather runs in
place with no packing; with the peer-memory collectives the update kernel itself stores the
bf16 results into every rank's parameter buffer (``multimem.st`` or peer stores), so update and
all-gather are one launch. Every per-step scalar (lr, bias corrections, clip coefficient) lives in
a device vector, which keeps the launches graph-capturable.

The buckets are updated and gathered in the order in which the next forward pass reads them
(embedding first, head last: the reverse of the flat-buffer order), on a side stream, with one
event per bucket; the next forward waits for a bucket's event only right before the first
layer that reads a parameter of it, so the update and the gather of everything but the first
bucket overlap the forward pass (the reference's per-bucket Adam -> all-gather pipeline,
exports/train_engine_8b/src/training_engine_tensor/entry.py:681-710, forward.py:150-158).

Numerics follow the reference's fused kernel
(exports/train_engine_0.5B/src/training_engine_tensor/triton_kernels.py:414-607) and its
sharded driver (optimizer.py:633-748): beta = (0.9, 0.95), eps 1e-8, weight decay only on
matrices, hidden matrices at lr / (hidden / 256) under muP.
"""
from __future__ import annotations

import os

import torch
import torch.distributed as dist

from ..ops import reference as ref_ops
from ..parallel.buckets import Bucket


class ShardedAdamW:
    def __init__(self, store, buckets: list[Bucket], world: int, rank: int, group, *,
                 beta1=0.9, beta2=0.95, eps=1e-8, weight_decay=0.1, max_grad_norm=1.0,
                 mup_lr_scaling=True, norm_reduce=None, comm_stream=None, fused=None):
        self.store = store
        self.buckets = buckets
        self.world, self.rank, self.group = world, rank, group
        self.beta1, self.beta2, self.eps = beta1, beta2, eps
        self.weight_decay = weight_decay
        self.max_grad_norm = max_grad_norm
        self.norm_reduce = norm_reduce    # callable summing the squared norm over all ranks
        self.step_count = 0
        self.fused = fused
        dev = store.device
        self.is_cuda = dev.type == "cuda"
        self.comm_stream = comm_stream
        total_shard = sum(b.shard_size(world) for b in buckets)
        self.master = torch.empty(total_shard, dtype=torch.float32, device=dev)
        self.exp_avg = torch.zeros(total_shard, dtype=torch.float32, device=dev)
        self.exp_avg_sq = torch.zeros(total_shard, dtype=torch.float32, device=dev)
        self.shard_off: list[int] = []
        off = 0
        for b in buckets:
            self.shard_off.append(off)
            off += b.shard_size(world)
        lr_div = store.spec.mup_width_scale if (mup_lr_scaling and store.spec.mup_enabled) else 1.0
        # per-bucket segment tables over the shard
        self.segments: list[list[tuple[int, float, float, str]]] = []
        self.seg_dev: list[tuple[torch.Tensor, torch.Tensor, torch.Tensor]] = []
        for b in buckets:
            s_lo, s_hi = b.shard_range(rank, world)
            segs = []
            for name in b.params:
                p_lo = b.start + b.param_offsets[name]
                p_hi = p_lo + b.param_sizes[name]
                a, z = max(p_lo, s_lo), min(p_hi, s_hi)
                if z <= a:
                    continue
                ps = store.by_name[name]
                wd = weight_decay if ps.has_weight_decay else 0.0
                lrm = 1.0 / lr_div if ps.mup_lr_scaled else 1.0
                segs.append((z - s_lo, wd, lrm, name))
            if not segs:
                segs.append((s_hi - s_lo, 0.0, 1.0, ""))
            self.segments.append(segs)
            if self.is_cuda:
                self.seg_dev.append((
                    torch.tensor([s[0] for s in segs], dtype=torch.int64, device=dev),
                    torch.tensor([s[1] for s in segs], dtype=torch.float32, device=dev),
                    torch.tensor([s[2] for s in segs], dtype=torch.float32, device=dev)))
        self.hyper = torch.zeros(8, dtype=torch.float32, device=dev)
        self.hyper_host = torch.zeros(8, dtype=torch.float32)
        if self.is_cuda:
            self.hyper_host = self.hyper_host.pin_memory()
        # fused peer-memory path: update + all-gather in one kernel (FT_FUSE_ADAM_AG=0: two)
        self.fuse_update_gather = os.environ.get("FT_FUSE_ADAM_AG", "1") != "0"
        self.sched = None        # device schedule vector, see set_schedule()
        self.step_dev = None
        self.grad_norm = torch.zeros(1, dtype=torch.float32, device=dev)
        self.sumsq_total = torch.zeros(1, dtype=torch.float32, device=dev)
        self.ag_events: list = [None] * len(buckets)
        # True: apply() leaves the per-bucket events pending for wait_bucket(); False: apply()
        # joins the side stream before it returns (CUDA-graph capture, serial streams)
        self.overlap_forward = False
        self.opt_stream = comm_stream
        self.sync_master_from_params()

    def set_schedule(self, max_lr: float, min_lr: float, warmup_iters: int, lr_decay_iters: int,
                     wsd_decay_iters: int) -> None:
        """Keep the step counter and the learning-rate schedule on the device (CUDA only): each
        :meth:`apply` then derives its own scalars in a one-thread kernel instead of copying
        them from the host, which is what lets a captured step be replayed without any
        per-step host data and keeps a host that runs ahead from overwriting scalars the
        device has not consumed yet. The ``lr`` passed to :meth:`step` must be the same
        schedule evaluated at ``step_count`` (it is only used for reporting then)."""
        if not self.is_cuda:
            return
        dev = self.hyper.device
        self.sched = torch.tensor([max_lr, min_lr, warmup_iters, lr_decay_iters, wsd_decay_iters,
                                   self.beta1, self.beta2, self.eps], dtype=torch.float32,
                                  device=dev)
        self.step_dev = torch.tensor([self.step_count], dtype=torch.int32, device=dev)

    # ------------------------------------------------------------------ state plumbing
    def master_view(self, i: int) -> torch.Tensor:
        o = self.shard_off[i]
        return self.master[o:o + self.buckets[i].shard_size(self.world)]

    def _views(self, i: int):
        o = self.shard_off[i]
        n = self.buckets[i].shard_size(self.world)
        return self.master[o:o + n], self.exp_avg[o:o + n], self.exp_avg_sq[o:o + n]

    def sync_master_from_params(self) -> None:
        for i, b in enumerate(self.buckets):
            lo, hi = b.shard_range(self.rank, self.world)
            self.master_view(i).copy_(self.store.flat_params[lo:hi].float())

    def sync_params_from_master(self) -> None:
        for i, b in enumerate(self.buckets):
            lo, hi = b.shard_range(self.rank, self.world)
            self.store.flat_params[lo:hi].copy_(self.master_view(i).to(self.store.dtype))
        self.all_gather_params()

    # ------------------------------------------------------------------ one step
    def compute_clip(self, local_sumsq: torch.Tensor) -> None:
        """All-reduce the squared norm, derive ``clip = min(1, max/(norm+1e-6))`` on device."""
        self.sumsq_total.copy_(local_sumsq)
        if self.norm_reduce is not None:
            self.norm_reduce(self.sumsq_total)
        if self.is_cuda:
            from ..ops import cuda_ops
            cuda_ops.clip_coef(self.sumsq_total, float(self.max_grad_norm), self.hyper,
                               self.grad_norm)
        else:
            nrm = self.sumsq_total.sqrt()
            self.grad_norm.copy_(nrm)
            clip = 1.0 if self.max_grad_norm <= 0 else min(1.0, self.max_grad_norm / (float(nrm) + 1e-6))
            self.hyper[6] = clip

    def step(self, lr: float) -> None:
        """Update this rank's shard of every bucket, then all-gather the bf16 parameters."""
        self.prepare_host(lr)
        self.apply()

    def prepare_host(self, lr: float) -> None:
        """Host half of a step: advance the step count and stage this step's scalars in the
        pinned hyper-parameter vector. Nothing is launched, so a captured :meth:`apply` can be
        replayed after it."""
        self.step_count += 1
        t = self.step_count
        self._lr = lr
        h = self.hyper_host
        h[0], h[1], h[2], h[3] = lr, self.beta1, self.beta2, self.eps
        h[4], h[5] = 1.0 - self.beta1 ** t, 1.0 - self.beta2 ** t

    def apply(self) -> None:
        """Device half of a step (capturable in a CUDA graph): derive the step's scalars and run
        the fused AdamW kernel and the parameter all-gather bucket by bucket, in forward-
        consumption order, on the side stream when there is one."""
        lr, t = self._lr, self.step_count
        side = self.opt_stream if (self.is_cuda and self.opt_stream is not None) else None
        if side is not None:
            ready = torch.cuda.Event()
            ready.record()                 # gradients reduced, clip coefficient written
            side.wait_event(ready)
            ctx = torch.cuda.stream(side)
        else:
            ctx = _null_ctx()
        with ctx:
            if self.sched is not None:
                from ..ops import cuda_ops
                cuda_ops.adam_hyper_step(self.step_dev, self.sched, self.hyper)
            else:
                # slots 6 (clip) and 7 are device-owned: copy only the first six
                self.hyper[:6].copy_(self.hyper_host[:6], non_blocking=True)
            for i in reversed(range(len(self.buckets))):
                self._update_bucket(i, lr, t)
                if side is not None:
                    done = torch.cuda.Event()
                    done.record()
                    self.ag_events[i] = done
        if side is not None and not self.overlap_forward:
            self.wait_all_gathers()

    def _update_bucket(self, i: int, lr: float, t: int) -> None:
        b = self.buckets[i]
        flat_g, flat_p = self.store.flat_grads, self.store.flat_params
        lo, hi = b.shard_range(self.rank, self.world)
        p32, m, v = self._views(i)
        if self.is_cuda and self.fused is not None and self.world > 1 and self.fuse_update_gather \
                and (hi - lo) % 8 == 0:
            se, sw, sl = self.seg_dev[i]
            self.fused.adamw_all_gather(b, p32, m, v, flat_g[lo:hi], self.hyper, se, sw, sl)
            return
        if self.is_cuda:
            from ..ops import cuda_ops
            se, sw, sl = self.seg_dev[i]
            cuda_ops.adamw_flat(p32, m, v, flat_g[lo:hi], flat_p[lo:hi], self.hyper, se, sw, sl)
        else:
            clip = float(self.hyper[6])
            a = 0
            for end, wd, lrm, _ in self.segments[i]:
                ref_ops.adamw_step(p32[a:end], m[a:end], v[a:end], flat_g[lo + a:lo + end],
                                   flat_p[lo + a:lo + end], lr * lrm, self.beta1, self.beta2,
                                   self.eps, wd, t, clip)
                a = end
        self._all_gather_bucket(i, b)

    def _all_gather_bucket(self, i: int, b: Bucket) -> None:
        """Gather bucket ``b`` on the current stream (apply() has already switched to the side
        stream when there is one)."""
        if self.world == 1:
            return
        lo, hi = b.shard_range(self.rank, self.world)
        full = self.store.flat_params[b.start:b.start + b.size]
        shard = self.store.flat_params[lo:hi]
        if self.fused is not None:
            self.fused.all_gather_bucket(b)
        elif self.is_cuda:
            dist.all_gather_into_tensor(full, shard, group=self.group)
        else:
            parts = [torch.empty_like(shard) for _ in range(self.world)]
            dist.all_gather(parts, shard.clone(), group=self.group)
            full.copy_(torch.cat(parts))

    def all_gather_params(self) -> None:
        """Gather every bucket now (after a load or a manual change of the shards). The pushes
        of the peer-memory gather land in the peers' parameter buffers without asking, so all
        ranks first meet in a barrier: nobody may still be reading the values being replaced.
        Inside a training step that guarantee comes from the gradient-norm all-reduce, which
        every rank passes between its last read of the old parameters and :meth:`apply`."""
        if self.fused is not None and self.world > 1:
            self.fused.barrier()
        for i, b in enumerate(self.buckets):
            self._all_gather_bucket(i, b)
        self.wait_all_gathers()

    def wait_bucket(self, i: int) -> None:
        """Make the current stream wait until bucket ``i`` holds this step's parameters."""
        ev = self.ag_events[i]
        if ev is not None:
            torch.cuda.current_stream().wait_event(ev)
            self.ag_events[i] = None

    def wait_all_gathers(self) -> None:
        if self.fused is not None:
            self.fused.wait_all_gathers()
        for i in range(len(self.ag_events)):
            self.wait_bucket(i)

    # ------------------------------------------------------------------ checkpoint support
    def gather_full_state(self, keep: bool = True) -> dict[str, dict[str, torch.Tensor]]:
        """Rank-count independent optimizer state: per-parameter fp32 tensors on CPU. A collective
        over the data-parallel group: every rank must call it. A rank that will not write the
        checkpoint passes ``keep=False``: it takes part in the gathers and returns empty
        dictionaries instead of holding a host copy of the whole state (three fp32 tensors per
        parameter, 48 GB for one tensor-parallel half of the 8B model)."""
        out = {"master_weights": {}, "exp_avg": {}, "exp_avg_sq": {}}
        for field, flat in (("master_weights", self.master), ("exp_avg", self.exp_avg),
                            ("exp_avg_sq", self.exp_avg_sq)):
            for i, b in enumerate(self.buckets):
                n = b.shard_size(self.world)
                shard = flat[self.shard_off[i]:self.shard_off[i] + n]
                if self.world > 1:
                    if self.is_cuda:
                        full = torch.empty(b.size, dtype=torch.float32, device=shard.device)
                        dist.all_gather_into_tensor(full, shard.contiguous(), group=self.group)
                    else:
                        parts = [torch.empty_like(shard) for _ in range(self.world)]
                        dist.all_gather(parts, shard.contiguous(), group=self.group)
                        full = torch.cat(parts)
                else:
                    full = shard
                if not keep:
                    continue
                for name in b.params:
                    o = b.param_offsets[name]
                    n_el = self.store.numel(name)
                    out[field][name] = full[o:o + n_el].view(self.store.shapes[name]).cpu().clone()
        return out

    def load_full_state(self, state: dict, step_count: int) -> None:
        for field, flat in (("master_weights", self.master), ("exp_avg", self.exp_avg),
                            ("exp_avg_sq", self.exp_avg_sq)):
            src = state[field]
            for i, b in enumerate(self.buckets):
                s_lo, s_hi = b.shard_range(self.rank, self.world)
                base = self.shard_off[i]
                for name in b.params:
                    p_lo = b.start + b.param_offsets[name]
                    n_el = self.store.numel(name)
                    a, z = max(p_lo, s_lo), min(p_lo + n_el, s_hi)
                    if z <= a:
                        continue
                    dst = flat[base + a - s_lo:base + z - s_lo]
                    if name not in src:
                        # a parameter the source run did not have (an untied output table, a new
                        # MTP head): master weights from the loaded parameters, moments at zero
                        if field == "master_weights":
                            dst.copy_(self.store.flat_params[a:z].float())
                        else:
                            dst.zero_()
                        continue
                    dst.copy_(src[name].reshape(-1)[a - p_lo:z - p_lo].to(flat.device))
        self.step_count = int(step_count)
        if self.step_dev is not None:
            self.step_dev.fill_(self.step_count)


class _null_ctx:
    def __enter__(self):
        return self

    def __exit__(self, *a):
        return False
