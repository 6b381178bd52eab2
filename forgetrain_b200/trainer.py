"""Training engine: one object that owns parameters, model, gradient reducer and optimizer,
and a loop around it.

``Trainer.train_step`` is the public per-step call: micro-batch loop (forward, fused
cross-entropy, backward writing gradients into the flat buffer), bucket reductions overlapped
with the last backward, device-side gradient norm and clip coefficient, sharded fused AdamW and
the in-place bf16 parameter all-gather. Nothing in the step synchronises the host; the returned
loss and gradient norm are device tensors. ``run_training_loop`` wraps it with the data
pipeline, logging (same line formats as the reference), MFU accounting, the segment profiler
and periodic asynchronous checkpoints. Counterpart of the reference's
``run_training_loop`` (exports/train_engine_0.5B/src/training_engine_tensor/train_loop.py:400-1061)
and ``_run_training_distributed`` (exports/train_engine_8b/src/training_engine_tensor/entry.py:298-780).
"""
from __future__ import annotations

import json
import math
import os
import time
from pathlib import Path

import torch
import torch.distributed as dist

from . import config as cfgmod
from .ckpt import checkpoint as ckpt
from .config import ModelSpec
from .data.prefetch import DataPrefetcher
from .data.synthetic import SyntheticTokenSource
from .engine_config import EngineConfig
from .models.minicpm4 import MiniCPM4
from .models.params import ALIGN_ELEMS, ParamStore
from .optim.adamw import ShardedAdamW
from .optim.lr import compute_lr
from .parallel.dp import BucketedGradReducer
from .parallel.topology import Topology
from .parallel.tp import TPContext
from .utils.profiler import StepProfiler, profiler_from_config


def _dtype_of(cfg: EngineConfig, device: torch.device) -> torch.dtype:
    return torch.bfloat16 if cfg.dtype == "bf16" else torch.float32


class Trainer:
    def __init__(self, spec: ModelSpec, cfg: EngineConfig, topo: Topology, *, seq_length: int,
                 micro_batch_size: int, seed: int = 1234, max_seq_len: int | None = None):
        self.spec, self.cfg, self.topo = spec, cfg, topo
        self.seq_length, self.mbs = seq_length, micro_batch_size
        dev = topo.device
        self.device = dev
        self.dtype = _dtype_of(cfg, dev)
        if dev.type == "cuda" and self.dtype != torch.bfloat16:
            raise ValueError("the CUDA path is bf16-only; use --dtype bf16 on GPUs")
        dp, tp = topo.dp_size, topo.tp_size
        # Peer memory only reaches the GPUs of this node. On several nodes the tensor-parallel
        # groups (consecutive ranks) stay inside a node when the TP degree divides the ranks per
        # node, so their fused kernels stay; the data-parallel groups span nodes and fall back
        # to the NCCL reducer / all-gather.
        from .parallel.topology import node_layout
        per_node = int(os.environ.get("LOCAL_WORLD_SIZE", "0") or 0) or topo.world
        multi_node, tp_in_node = node_layout(topo.world, per_node, tp)
        if multi_node and cfg.comm == "fused" and topo.rank == 0:
            print(f"[engine] {topo.world} ranks on nodes of {per_node}: data-parallel collectives "
                  f"use NCCL; tensor-parallel kernels stay fused: {tp_in_node and tp > 1}", flush=True)
        if (cfg.comm == "fused" and dev.type == "cuda" and tp > 1 and cfg.sequence_parallel
                and tp_in_node
                and (micro_batch_size * seq_length) % (128 * tp) == 0):
            from .parallel.fused_tp import FusedTPContext
            n_slots = 2 * (spec.num_layers + cfg.mtp_num_layers) + 4
            self.tp_ctx = FusedTPContext(topo.tp_group, tp, topo.tp_rank, dev,
                                         micro_batch_size * seq_length, spec.hidden_size, n_slots,
                                         topo.replica_group, topo.replica_size)
        else:
            self.tp_ctx = TPContext(topo.tp_group, tp, topo.tp_rank, cfg.sequence_parallel,
                                    topo.replica_group, topo.replica_size)
        # --- fused peer-memory communication (GPU, >1 rank, comm == "fused")
        self.fused_dp = None
        self.symm = None
        grad_buffer = param_buffer = None
        # SHARDED_OPTIMIZER=0: every rank keeps the whole optimizer state and updates every
        # parameter itself; gradients are all-reduced by the library and nothing is gathered
        # (the reference's non-ZeRO path, 0.5B optimizer.py:569-630). Costs dp x the state memory.
        sharded = cfg.sharded_optimizer or dp == 1
        want_fused = (cfg.comm == "fused" and dev.type == "cuda" and dp > 1 and not multi_node
                      and sharded)
        pad = ALIGN_ELEMS * dp
        if want_fused:
            from .parallel import fused_dp
            total = ParamStore.layout_total(spec, cfg.mtp_num_layers, tp, pad)
            self.symm = fused_dp.SymmetricBuffers(total, dev, topo.dp_group, topo.dp_rank, dp)
            grad_buffer, param_buffer = self.symm.grads, self.symm.params
        self.store = ParamStore(spec, dev, self.dtype, cfg.mtp_num_layers, topo.tp_rank, tp,
                                pad_to=pad, grad_buffer=grad_buffer, align=pad,
                                param_buffer=param_buffer)
        if cfg.random_init:
            self.store.init_random(seed, cfg.init_scheme, cfg.init_std)
        self.model = MiniCPM4(spec, self.store, self.tp_ctx, max_seq_len=max_seq_len or seq_length,
                              recompute_attn=cfg.recompute_attn, recompute_mlp=cfg.recompute_mlp)
        self.model.mask_vocab_padding = cfg.mask_vocab_padding
        self.mtp = None
        if cfg.mtp_num_layers > 0:
            from .models.mtp import MTPHead
            self.mtp = MTPHead(self.model, cfg.mtp_num_layers, cfg.mtp_loss_scaling_factor)
        target = cfg.wgrad_bucket_target_elems
        if cfg.rs_buckets > 0 and tp > 1:
            target = max(1, self.store.total // cfg.rs_buckets)
        norm_exclude = []
        if tp > 1 and topo.tp_rank > 0:
            for ps in self.store.order:
                if ps.is_norm:
                    o = self.store.offsets[ps.name]
                    norm_exclude.append((o, o + self.store.numel(ps.name)))
        if topo.replica_size > 1 and topo.tp_rank % topo.replica_size != 0:
            # k / v rows of wqkv are replicated inside a KV group: count them on one rank only
            D = spec.head_dim
            for ps in self.store.order:
                if ps.name.endswith("attention.wqkv.weight"):
                    o = self.store.offsets[ps.name]
                    rows, cols = self.store.shapes[ps.name]
                    norm_exclude.append((o + (rows - 2 * D) * cols, o + rows * cols))
        if want_fused:
            from .parallel import fused_dp
            self.fused_dp = fused_dp.FusedDPComm(self.symm)
        self.reducer = BucketedGradReducer(
            self.store.flat_grads, self.store.entries(), dp, topo.dp_rank, topo.dp_group, target,
            backend=cfg.comm, overlap=cfg.wgrad_overlap and not cfg.serial_streams,
            norm_exclude=norm_exclude, fused=self.fused_dp, all_reduce=not sharded)
        norm_reduce = None
        if topo.world > 1:
            if self.fused_dp is not None and tp == 1:
                norm_reduce = self.fused_dp.all_reduce_small
            else:
                norm_reduce = (lambda t: dist.all_reduce(t))  # world: DP shards x TP shards
        opt_buckets, opt_world, opt_rank = self.reducer.buckets, dp, topo.dp_rank
        if not sharded:
            from .parallel.buckets import compute_grad_buckets
            opt_buckets, opt_world, opt_rank = compute_grad_buckets(self.store.entries(), 1, target), 1, 0
        self.opt = ShardedAdamW(
            self.store, opt_buckets, opt_world, opt_rank, topo.dp_group if sharded else None,
            beta1=cfg.adam_beta1, beta2=cfg.adam_beta2, eps=cfg.adam_eps,
            weight_decay=cfg.weight_decay,
            max_grad_norm=0.0 if cfg.no_grad_clip else cfg.max_grad_norm,
            mup_lr_scaling=cfg.mup_lr_scaling, norm_reduce=norm_reduce,
            comm_stream=self._optimizer_stream(cfg, dev),
            fused=self.fused_dp)
        self.opt.set_schedule(cfg.max_lr, cfg.min_lr, cfg.warmup_iters, cfg.lr_decay_iters,
                              cfg.wsd_decay_iters)
        self.num_samples = 0
        self.loss_buf = torch.zeros(1, dtype=torch.float32, device=dev)
        # per-layer losses of the multi-token-prediction head, averaged like the main loss
        self.mtp_loss_buf = (torch.zeros(cfg.mtp_num_layers, dtype=torch.float32, device=dev)
                             if cfg.mtp_num_layers > 0 else None)
        self.graph = None
        self.full_graph = None
        self._fwd_graph = None
        graphable_comm = topo.world == 1 or (self.fused_dp is not None and tp == 1)
        uses_graph = dev.type == "cuda" and (cfg.full_step_cuda_graph or cfg.step_cuda_graph)
        # Weight-gradient GEMMs of the decoder blocks on a side stream: the tail of one GEMM's last
        # wave then overlaps the start of the next kernel, and with tensor parallelism over NCCL they
        # run while the collective that follows the data gradient is in flight. Not with the fused
        # all-gather -> GEMM kernel: a second full-grid GEMM on another stream only delays that
        # kernel's own CTAs, which wait for one another's copies.
        fused_tp = tp > 1 and cfg.comm == "fused"
        if cfg.wgrad_side_stream and dev.type == "cuda" and not uses_graph \
                and not cfg.serial_streams and not fused_tp:
            self.model.wgrad_stream = torch.cuda.Stream(device=dev)
        if self.opt.opt_stream is not None and not uses_graph:
            self.opt.overlap_forward = True
            self._install_param_gate()
        if cfg.full_step_cuda_graph and dev.type == "cuda" and graphable_comm:
            from .graph.step_graph import GraphedFullStep
            self.full_graph = GraphedFullStep(self, cfg.step_cuda_graph_warmup)
        elif (cfg.step_cuda_graph or cfg.full_step_cuda_graph) and dev.type == "cuda" \
                and self.mtp is None:
            from .graph.step_graph import GraphedComputeStep
            self.graph = GraphedComputeStep(self.model, cfg.step_cuda_graph_warmup,
                                            cfg.step_cuda_graph_sanity, cfg.step_cuda_graph_tol)

    # ------------------------------------------------------------------ helpers
    def _optimizer_stream(self, cfg: EngineConfig, dev):
        """Stream of the AdamW + all-gather pipeline: the reducer's communication stream (the
        peer-memory kernels of one process must all run in one order), else a stream of its
        own; none with ``opt_allgather_overlap`` off, serial streams or on CPU."""
        if dev.type != "cuda" or not cfg.opt_allgather_overlap or cfg.serial_streams:
            return None
        return self.reducer.comm_stream or torch.cuda.Stream(device=dev)

    def _install_param_gate(self) -> None:
        """The forward pass waits for a bucket of the previous optimizer step right before the
        first layer that reads one of its parameters, and not earlier."""
        by_prefix: dict[str, list[int]] = {}
        for b in self.opt.buckets:
            for name in b.params:
                parts = name.split(".")
                pre = ".".join(parts[:2]) if parts[0] == "layers" else \
                    (".".join(parts[:3]) if parts[0] == "mtp" else parts[0])
                if b.index not in by_prefix.setdefault(pre, []):
                    by_prefix[pre].append(b.index)
        opt = self.opt

        def gate(prefix: str) -> None:
            for i in by_prefix.get(prefix, ()):
                opt.wait_bucket(i)
        self.model.param_gate = gate

    def loss_to_host_async(self) -> "LossReadback":
        """Start a device-to-host copy of the last step's loss (and gradient norm) into pinned
        memory on the current stream and return a handle; ``handle.value()`` waits for that
        copy only. Reading step i's loss after step i+1 has been enqueued keeps the host one
        step ahead of the device instead of draining the GPU at every step."""
        return LossReadback(self.loss_buf, self.opt.grad_norm)

    def finish_step(self) -> None:
        """Make the current stream wait for everything the last step left running on side
        streams (the tail of the optimizer / all-gather pipeline)."""
        self.opt.wait_all_gathers()

    def _grad_ready(self, name: str) -> None:
        """The gradient of ``name`` is complete on this rank (last micro-batch): finish it over
        the tensor-parallel group where that is needed, then hand it to the bucket reducer."""
        self.model.finalize_grad(name)
        self.reducer.on_grad_ready(name)

    @torch.no_grad()
    def forward_logits(self, tokens: torch.Tensor, position_ids=None) -> torch.Tensor:
        """Forward pass only (evaluation); replayed from a CUDA graph per input shape when
        ``forward_cuda_graph`` is set."""
        if self.cfg.forward_cuda_graph and tokens.is_cuda:
            if self._fwd_graph is None:
                from .graph.step_graph import GraphedForward
                self._fwd_graph = GraphedForward(self.model)
            return self._fwd_graph(tokens, position_ids)
        return self.model.forward(tokens, position_ids)

    def nonfinite_report(self, limit: int = 6) -> str:
        """Which parameters and gradients hold NaN / Inf on this rank (after a non-finite loss: the
        first thing one wants to know; the reference has a NaN diagnostic inside its norm backward
        kernel for the same purpose, triton_kernels.py:725-803). Synchronises."""
        bad = []
        for kind, views in (("parameter", self.store.params), ("gradient", self.store.grads)):
            for name, t in views.items():
                n = int((~torch.isfinite(t.float())).sum())
                if n:
                    bad.append(f"{kind} {name}: {n} of {t.numel()} values")
        if not bad:
            return "parameters and gradients of this rank are finite (the loss itself overflowed)"
        more = f" and {len(bad) - limit} more" if len(bad) > limit else ""
        return "non-finite values in " + "; ".join(bad[:limit]) + more

    def current_lr(self) -> float:
        c = self.cfg
        return compute_lr(self.opt.step_count, c.max_lr, c.min_lr, c.warmup_iters, c.lr_decay_iters,
                          c.wsd_decay_iters)

    def _grad_norm_diag(self) -> None:
        """``GRAD_NORM_DIAG``: this rank's full gradient norm before any reduction and the
        twelve largest per-parameter norms (reference train_loop.py:829-856). Synchronises."""
        rows = sorted(((float(self.store.grads[ps.name].float().norm()), ps.name)
                       for ps in self.store.specs), reverse=True)
        total = sum(g * g for g, _ in rows) ** 0.5
        print(f"[grad-norm-diag] pre_reduce_rank{self.topo.rank}_full={total:.10f}", flush=True)
        print("[grad-norm-top] " + " | ".join(f"{g:.6f}:{n}" for g, n in rows[:12]), flush=True)

    def _micro_batch(self, batch, loss_scale: float, accumulate: bool, last: bool, prof=None):
        diag = self.cfg.grad_norm_diag and last and self.topo.dp_rank == 0
        hold = self.cfg.grad_norm_diag and last   # every rank holds its buckets back alike
        grad_ready = self._grad_ready if (last and not hold) else None
        tokens, labels = batch["tokens"], batch["labels"]
        mask = batch.get("loss_mask")
        pos = batch.get("position_ids")
        m = self.model
        if self.graph is not None:
            loss = self.graph(batch, loss_scale, accumulate)
            if last:      # gradients are complete only after the replay: release every bucket now
                for ps in self.store.order:
                    self._grad_ready(ps.name)
            return loss
        if self.mtp is not None:
            loss = self.mtp.forward_backward(tokens, labels, mask, loss_scale, accumulate,
                                             grad_ready, pos)
        elif prof is not None and prof.deep and prof.active:
            # PROFILE_DEEP: the phases of a micro-batch as separate segments (reference
            # profiling.py:180-191, hooks train_loop.py:584-585,643-648). Gradient accumulation
            # happens inside the weight-gradient GEMM epilogue here, so ``mb_accum`` closes at
            # once after ``mb_bwd``; it is kept for the record layout.
            logits = m.forward(tokens, pos)
            prof.deep_mark("mb_fwd")
            loss, dlogits = m.loss_and_dlogits(logits, labels, mask, loss_scale)
            del logits
            prof.deep_mark("mb_ce")
            m.backward(tokens, dlogits, accumulate, grad_ready, pos)
            prof.deep_mark("mb_bwd")
            prof.deep_mark("mb_accum")
        else:
            loss = m.forward_backward(tokens, labels, mask, loss_scale, accumulate, grad_ready, pos)
        if hold:   # diagnostics look at the local gradients, so the buckets are released after
            if diag:
                self._grad_norm_diag()
            for ps in self.store.order:
                self._grad_ready(ps.name)
        return loss

    # ------------------------------------------------------------------ the step
    def train_step(self, micro_batches: list[dict], profiler: StepProfiler | None = None) -> dict:
        """One optimizer step over ``micro_batches`` (device tensors). Returns device-side
        ``loss`` (mean over micro-batches and DP ranks) and ``grad_norm`` plus the ``lr`` used."""
        lr = self.current_lr()
        self.opt.prepare_host(lr)
        for batch in micro_batches:
            self.num_samples += batch["tokens"].shape[0] * self.topo.dp_size
        if self.full_graph is not None and profiler is None:
            self.full_graph(micro_batches)
        else:
            self._device_step(micro_batches, profiler)
        out = {"loss": self.loss_buf, "grad_norm": self.opt.grad_norm, "lr": lr}
        if self.mtp_loss_buf is not None:
            out["mtp_loss_per_layer"] = self.mtp_loss_buf
        return out

    def _device_step(self, micro_batches: list[dict], prof: StepProfiler | None = None) -> None:
        """Everything of a step that runs on the device: micro-batches, bucket reductions,
        gradient norm and clip coefficient, AdamW, parameter all-gather, loss average. With one
        process (or device-side collectives) it issues no host synchronisation."""
        n = len(micro_batches)
        if prof:
            prof.mark("step_start")
        if not self.opt.overlap_forward:
            self.opt.wait_all_gathers()
        self.reducer.start_step()
        self.loss_buf.zero_()
        if self.mtp_loss_buf is not None:
            self.mtp_loss_buf.zero_()
        for i, batch in enumerate(micro_batches):
            if prof:
                prof.deep_mark("mb_data")
            loss = self._micro_batch(batch, 1.0 / n, accumulate=i > 0, last=(i == n - 1), prof=prof)
            self.loss_buf += loss.detach().reshape(1) / n
            if self.mtp_loss_buf is not None:   # mean over micro-batches, per MTP layer
                self.mtp_loss_buf += torch.stack(
                    [l.detach().reshape(()) for l in self.mtp.last_mtp_losses]).float() / n
        if prof:
            prof.mark("microbatches")
        self.reducer.wait_all()
        if prof:
            prof.mark("reduce_scatter")
        self.opt.compute_clip(self.reducer.local_sumsq())
        if prof:
            prof.mark("grad_norm")
        self.opt.apply()
        if prof:
            prof.mark("optimizer")
        if self.topo.dp_size > 1:
            # mean over the data-parallel ranks, of the loss and of the per-layer MTP losses
            # (reference train_loop.py:326-364, 767-772)
            for buf in (self.loss_buf, self.mtp_loss_buf):
                if buf is None:
                    continue
                if self.fused_dp is not None:
                    self.fused_dp.all_reduce_small(buf)
                else:
                    dist.all_reduce(buf, group=self.topo.dp_group)
                buf /= self.topo.dp_size
        if prof:
            prof.mark("loss_allreduce")
            if prof.active:   # on profiled steps the parameter gather is closed inside the step
                self.opt.wait_all_gathers()
            prof.mark("allgather")

    # ------------------------------------------------------------------ checkpoint
    def save(self, save_dir, step: int, dataloader_state=None, async_io=True):
        """Rank-count independent checkpoint: DP shards of the optimizer state are gathered;
        with TP > 1 every TP rank of DP rank 0 writes its own ``rank_<R>.pt`` shard."""
        self.finish_step()        # the parameters read below are complete on this stream
        # only the ranks that write a file keep the gathered state on the host
        writes = self.topo.rank == 0 if self.topo.tp_size == 1 else self.topo.dp_rank == 0
        opt_state = self.opt.gather_full_state(keep=writes)
        opt_state["step_count"] = self.opt.step_count
        opt_state["num_samples"] = self.num_samples
        names = [ps.name for ps in self.store.specs]
        params = {n: self.store.params[n] for n in names}
        if self.topo.tp_size == 1:
            return ckpt.save_checkpoint(save_dir, step, params=params, param_names=names,
                                        optimizer_state=opt_state, num_samples=self.num_samples,
                                        dataloader_state=dataloader_state, rank=self.topo.rank,
                                        async_io=async_io)
        writer = 0 if self.topo.dp_rank == 0 else 1
        return ckpt.save_checkpoint(save_dir, step, params=params, param_names=names,
                                    optimizer_state=opt_state, num_samples=self.num_samples,
                                    dataloader_state=dataloader_state, rank=writer,
                                    async_io=async_io, filename=f"rank_{self.topo.tp_rank}.pt",
                                    extra={"tp_size": self.topo.tp_size, "tp_rank": self.topo.tp_rank,
                                           "vocab_size": self.spec.vocab_size})

    def load(self, path) -> dict:
        p = Path(path)
        note = (lambda m: print(f"[load] {m}", flush=True)) if self.topo.rank == 0 else (lambda m: None)
        from .ckpt import megatron_import as mg
        if mg.is_megatron_root(p):
            # a Megatron export: full tensors by Megatron names (+ optional Adam state); every
            # rank reads the file and keeps its tensor-parallel shard
            log = print if self.topo.rank == 0 else (lambda *_: None)
            n_mtp = self.cfg.mtp_num_layers
            tensors = mg.load_megatron_checkpoint(p, self.spec, n_mtp, log=log)
            self.store.load_named(tensors, full_tensors=True, keep_missing=("mtp.",), log=log)
            ost = mg.load_megatron_optimizer_state(p, log=log)
            if ost is not None:
                from .models.params import shard_for_tp
                L = self.spec.num_layers
                by_name = {ps.name: ps for ps in self.store.specs}
                tp, tpr = self.topo.tp_size, self.topo.tp_rank
                for k in ("master_weights", "exp_avg", "exp_avg_sq"):
                    ost[k] = mg.rename_state(ost[k], L, n_mtp)
                    if tp > 1:       # full tensors in the export: keep this rank's shard
                        ost[k] = {n: shard_for_tp(by_name[n], t, self.spec, tpr, tp)
                                  for n, t in ost[k].items() if n in by_name}
                self.opt.load_full_state(ost, ost["step_count"])
                self.num_samples = ost["num_samples"]
            else:
                self.opt.sync_master_from_params()
            return {"step": 0, "num_samples": self.num_samples, "dataloader_state": None}
        from .ckpt import hf_import
        if hf_import.is_hf_folder(p):
            # a HuggingFace export: full tensors, no optimizer state; every rank keeps its shard
            self.store.load_named(hf_import.load_hf_folder(p, self.spec), full_tensors=True,
                                  keep_missing=("mtp.",), log=note)
            self.opt.sync_master_from_params()
            return {"step": 0, "num_samples": 0, "dataloader_state": None}
        if p.is_dir() and not any(p.glob("rank_*.pt")) and not (p / "training_state.pt").exists():
            from .ckpt.checkpoint import latest_step_dir
            p = latest_step_dir(p, "rank_*.pt") or p
        rank_files = sorted(p.glob("rank_*.pt"), key=lambda q: int(q.stem.split("_")[1])) \
            if p.is_dir() else []
        tp, tpr = self.topo.tp_size, self.topo.tp_rank
        if rank_files and len(rank_files) == tp and tp > 1:
            # same tensor-parallel degree: every rank reads its own shard
            state = torch.load(p / f"rank_{tpr}.pt", map_location="cpu", weights_only=False)
            self.store.load_named(state["params"], full_tensors=False, keep_missing=("mtp.",), log=note)
        else:
            # a checkpoint of another tensor-parallel degree (or of none): rebuild the full
            # tensors, then keep this rank's shard of parameters and optimizer state
            from .models.params import merge_tp_shards, shard_for_tp
            if rank_files:
                shards = [torch.load(q, map_location="cpu", weights_only=False) for q in rank_files]
                if len(shards) != int(shards[0].get("tp_size", len(shards))):
                    raise ValueError(f"{p}: {len(shards)} rank files for tp_size {shards[0].get('tp_size')}")
                state = dict(shards[0])
                state["params"] = merge_tp_shards(self.spec, [sh["params"] for sh in shards],
                                                  self.store.specs)
                osts = [sh.get("optimizer_state") for sh in shards]
                if all(osts):
                    merged = dict(osts[0])
                    for k in ("master_weights", "exp_avg", "exp_avg_sq"):
                        merged[k] = merge_tp_shards(self.spec, [o[k] for o in osts], self.store.specs)
                    state["optimizer_state"] = merged
            else:
                state = ckpt.load_resume_checkpoint(p, expected_vocab=self.spec.vocab_size)
            self.store.load_named(state["params"], full_tensors=True, keep_missing=("mtp.",), log=note)
            ost = state.get("optimizer_state")
            if ost and tp > 1:
                by_name = {ps.name: ps for ps in self.store.specs}
                ost = dict(ost)
                for k in ("master_weights", "exp_avg", "exp_avg_sq"):
                    ost[k] = {n: shard_for_tp(by_name[n], t, self.spec, tpr, tp)
                              for n, t in ost[k].items() if n in by_name}
                state["optimizer_state"] = ost
        ost = state.get("optimizer_state")
        if ost:
            self.opt.load_full_state(ost, ost.get("step_count", state.get("step", 0)))
            self.num_samples = int(ost.get("num_samples", state.get("num_samples", 0)))
        else:
            self.opt.sync_master_from_params()
        return state


class _StopRequest:
    """SIGTERM (a scheduler's pre-emption notice, also what ``torch.distributed.run`` forwards to its
    workers) and SIGUSR1 ask the loop to stop: the running step is finished, every rank learns of
    the request in the step's own all-reduce, a checkpoint is written when there is a
    ``save_dir``, and the loop returns normally, so the job can be continued with ``--resume``
    (or by the launcher's ``AUTO_RESUME``).

    The same signal also reaches the survivors of a job that lost a rank, and those sit in a
    collective that will never return, where no Python-level handler runs. So the signal is taken
    from the interpreter's wake-up descriptor by a watcher thread: it raises the flag and, if the
    ranks have not agreed on a stopping step within the grace period (``max(5 s, 3 steps)``), ends
    the process the way the signal would have. Installed in the main thread only; ``restore``
    puts the previous handlers back."""

    GRACE_S = 5.0
    _live = None                 # the instance whose handlers are installed, if any

    def __init__(self):
        import signal
        import socket
        import threading
        if _StopRequest._live is not None:      # a loop that ended in an exception left its own
            _StopRequest._live.restore()
        self.requested = False
        self.agreed = False          # set by the loop once all ranks know of the request
        self.step_s = 0.0            # duration of the last step, for the grace period
        self._old, self._old_fd, self._pair = {}, None, None
        if threading.current_thread() is not threading.main_thread():
            return
        try:
            r, w = socket.socketpair()
            r.setblocking(True)
            w.setblocking(False)
            self._old_fd = signal.set_wakeup_fd(w.fileno(), warn_on_full_buffer=False)
            self._pair = (r, w)
            for sig in (signal.SIGTERM, signal.SIGUSR1):
                self._old[sig] = signal.signal(sig, self._handler)
        except (ValueError, OSError):
            return
        self._watch = {int(signal.SIGTERM), int(signal.SIGUSR1)}
        _StopRequest._live = self
        threading.Thread(target=self._watcher, name="stop-request", daemon=True).start()

    def _handler(self, signum, frame):
        self.requested = True

    def _watcher(self):
        import time
        r = self._pair[0]
        while True:
            try:
                data = r.recv(16)
            except OSError:
                return
            if not data:
                return
            if not any(b in self._watch for b in data):
                continue
            self.requested = True
            deadline = time.monotonic() + max(self.GRACE_S, 3.0 * self.step_s)
            while time.monotonic() < deadline:
                if self.agreed or self._pair is None:
                    return
                time.sleep(0.05)
            if not self.agreed and self._pair is not None:
                os._exit(143)        # the others are not coming: leave as the signal asked

    def restore(self):
        import signal
        if _StopRequest._live is self:
            _StopRequest._live = None
        pair, self._pair = self._pair, None
        for sig, old in self._old.items():
            try:
                signal.signal(sig, old)
            except (ValueError, OSError):
                pass
        self._old = {}
        if pair is not None:
            try:
                signal.set_wakeup_fd(self._old_fd if self._old_fd is not None else -1)
            except (ValueError, OSError):
                pass
            for sock in pair:
                sock.close()


class LossReadback:
    """Asynchronous read-back of (loss, grad_norm): 8 bytes, device -> pinned host."""
    nbytes = 8

    def __init__(self, loss: torch.Tensor, grad_norm: torch.Tensor):
        self._cuda = loss.is_cuda
        if self._cuda:
            self._host = torch.empty(2, dtype=torch.float32, pin_memory=True)
            self._host[0:1].copy_(loss.reshape(1), non_blocking=True)
            self._host[1:2].copy_(grad_norm.reshape(1), non_blocking=True)
            self._event = torch.cuda.Event()
            self._event.record()
        else:
            self._host = torch.stack([loss.reshape(()), grad_norm.reshape(())]).float().clone()

    def value(self) -> tuple[float, float]:
        if self._cuda:
            self._event.synchronize()
        return float(self._host[0]), float(self._host[1])


# ---------------------------------------------------------------------------------------------
# loop
# ---------------------------------------------------------------------------------------------
def _log(topo: Topology, msg: str) -> None:
    if topo.rank == 0:
        print(msg, flush=True)


def run_training_loop(*, spec: ModelSpec, cfg: EngineConfig, topo: Topology, num_steps: int,
                      micro_batch_size: int, seq_length: int, num_local_microbatches: int = 1,
                      seed: int = 1234, save_dir: str | None = None, save_interval: int = 0,
                      resume: str | None = None, data_source=None, dump_inputs_dir: str | None = None,
                      report_path: str | None = None, log_every: int = 1) -> dict:
    """Train ``num_steps`` optimizer steps; returns ``{"steps": [per-step dicts], ...}``."""
    trainer = Trainer(spec, cfg, topo, seq_length=seq_length, micro_batch_size=micro_batch_size,
                      seed=seed)
    start_step = 0
    source = data_source or SyntheticTokenSource(spec.vocab_size, micro_batch_size, seq_length,
                                                 seed=seed, dp_rank=topo.dp_rank,
                                                 pin=topo.device.type == "cuda")
    if resume:
        state = trainer.load(resume)
        start_step = int(state.get("step", 0))
        if hasattr(source, "load_state_dict"):
            from .data.hf_dataloader import select_rank_state
            source.load_state_dict(select_rank_state(state.get("dataloader_state"), topo.dp_rank,
                                                     topo.dp_size, log=lambda m: _log(topo, m)))
        _log(topo, f"resumed from {resume} at step {start_step}")
    consumed_at_start = consumed = int(getattr(source, "batches_drawn", 0))
    prefetch = DataPrefetcher(source, topo.device, depth=cfg.data_prefetch_depth)
    profiler = profiler_from_config(cfg, rank=topo.rank)
    tokens_per_step = micro_batch_size * seq_length * num_local_microbatches * topo.dp_size
    flops_hw = cfgmod.compute_training_flops(spec, tokens_per_step, seq_length, cfg.mtp_num_layers)
    flops_std = cfgmod.compute_training_flops_standard(spec, tokens_per_step, seq_length,
                                                       cfg.mtp_num_layers)
    peak = cfgmod.peak_tflops() * 1e12 * topo.world
    cuda = topo.device.type == "cuda"
    results = []
    _log(topo, f"[engine] model={spec.name} params={spec.num_parameters(cfg.mtp_num_layers)/1e6:.1f}M "
               f"world={topo.world} dp={topo.dp_size} tp={topo.tp_size} mbs={micro_batch_size} "
               f"seq={seq_length} microbatches={num_local_microbatches} dtype={cfg.dtype} "
               f"comm={cfg.comm} data={'synthetic' if data_source is None else 'custom'}")
    from .utils.fault_injection import maybe_fail
    stop = _StopRequest()                    # SIGTERM / SIGUSR1: checkpoint after the running step
    for step in range(start_step, start_step + num_steps):
        maybe_fail(step + 1, topo.rank)      # recovery tests: FT_INJECT_FAILURE, host side only
        if cuda:
            ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            ev0.record()
        t0 = time.perf_counter()
        if profiler:
            profiler.begin_step(step)
        mbs = [next(prefetch) for _ in range(num_local_microbatches)]
        # position in the source of the last batch the model sees this step (all-masked batches
        # that the prefetcher dropped on the way count, what it has read ahead does not)
        consumed = consumed_at_start + prefetch.consumed_from_source
        if dump_inputs_dir and topo.rank == 0:
            Path(dump_inputs_dir).mkdir(parents=True, exist_ok=True)
            torch.save({k: v.cpu() for k, v in mbs[0].items()},
                       Path(dump_inputs_dir) / f"inputs_step{step:07d}.pt")
        out = trainer.train_step(mbs, profiler)
        if cuda:
            ev1.record()
            torch.cuda.synchronize()
            dt = ev0.elapsed_time(ev1) / 1e3
            from .ops import _lib
            _lib.check_status(topo.device)
        else:
            dt = time.perf_counter() - t0
        stopping = stop.requested
        if topo.world > 1:  # step time = max over ranks; a stop request of any rank is everybody's
            tt = torch.tensor([dt, float(stopping)], dtype=torch.float64, device=topo.device)
            dist.all_reduce(tt, op=dist.ReduceOp.MAX)
            dt, stopping = float(tt[0]), bool(tt[1] > 0)
        stop.step_s = dt
        if stopping:
            stop.agreed = True
        if profiler:
            profiler.end_step()
        loss, gnorm = float(out["loss"]), float(out["grad_norm"])
        rec = {"step": step + 1, "loss": loss, "local_loss": loss, "grad_norm": gnorm,
               "lr": out["lr"], "total_step_time": dt, "mfu_e2e": flops_hw / dt / peak,
               "mfu_e2e_standard": flops_std / dt / peak,
               "tokens_per_sec_per_gpu": tokens_per_step / dt / topo.world}
        mtp_suffix = ""
        if "mtp_loss_per_layer" in out:
            per_layer = [float(v) for v in out["mtp_loss_per_layer"].tolist()]
            rec["mtp_loss_per_layer"] = per_layer
            rec["mtp_loss"] = sum(per_layer) / len(per_layer)
            mtp_suffix = " | mtp loss: " + ", ".join(f"{v:.6e}" for v in per_layer)
        results.append(rec)
        if (step + 1) % log_every == 0:
            _log(topo, f" iteration {step + 1:8d} | loss {loss:.6E} | local_loss {loss:.6E} | "
                       f"grad norm {gnorm:.4f} | lr {out['lr']:.4E} | time(ms) {dt * 1e3:.1f} | "
                       f"tok/s/gpu {rec['tokens_per_sec_per_gpu']:.0f} | mfu {rec['mfu_e2e_standard'] * 100:.2f}%"
                       f"{mtp_suffix}")
            if cfg.emit_loss_lines:
                _log(topo, f"[LOSS] step={step + 1} global_loss={loss:.8f} grad_norm={gnorm:.6f} "
                           f"time_s={dt:.4f} mfu_e2e_standard={rec['mfu_e2e_standard']:.4f}")
        if not math.isfinite(loss):
            raise FloatingPointError(f"non-finite loss at step {step + 1}; {trainer.nonfinite_report()}")
        done = step + 1
        if save_dir and (stopping or ckpt.should_save_after_step(done, start_step + num_steps,
                                                                  save_interval, start_step)):
            if hasattr(source, "state_dict_at"):   # a stream cannot be rewound by a count alone
                ds = source.state_dict_at(consumed)
            else:
                ds = dict(getattr(source, "state_dict", dict)())
                if "batches_drawn" in ds:   # the prefetcher reads ahead: record what was consumed
                    ds["batches_drawn"] = consumed
            if topo.dp_size > 1 and isinstance(ds, dict):
                # every data-parallel rank may be somewhere else in its own data: a streamed
                # dataset always is, any source is once a rank has dropped an all-masked batch
                from .data.hf_dataloader import pack_rank_states
                states = [None] * topo.dp_size
                dist.all_gather_object(states, ds, group=topo.dp_group)
                ds = pack_rank_states(states)
            trainer.save(save_dir, done, dataloader_state=ds)
        if stopping:
            _log(topo, f"[signal] stop requested: {'checkpoint written at' if save_dir else 'no --save-dir, leaving at'} "
                       f"step {done} of {start_step + num_steps}")
            break
    stop.restore()
    ckpt.wait_for_async_save()
    if profiler:
        profiler.write()
    report = {"steps": results, "model": spec.name, "world": topo.world,
              "tokens_per_step": tokens_per_step}
    if report_path and topo.rank == 0:
        Path(report_path).parent.mkdir(parents=True, exist_ok=True)
        tmp = Path(report_path).with_suffix(".tmp")
        tmp.write_text(json.dumps(report, indent=1))
        os.replace(tmp, report_path)
    report["trainer"] = trainer
    return report
