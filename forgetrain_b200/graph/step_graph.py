"""Whole micro-batch (forward + fused cross-entropy + backward) captured in a CUDA graph.

Every kernel of the compute step is launched on the current stream with device-resident
operands, so the step is capturable as it is: inputs are copied into static buffers, the graph
is replayed, the loss is read from a static scalar and the gradients land in the flat gradient
buffer as in eager mode. Two graphs are kept per input shape: "store" (first micro-batch of a
step) and "accumulate" (later micro-batches). Collectives and the optimizer stay outside the
graph (their per-step scalars and epochs are host-side), so bucket reductions are issued right
after the replay instead of during backward.

Warm-up iterations run before capture on a side stream (they only produce gradients, which the
captured step overwrites, so they do not train). An optional sanity check replays once and
compares the loss with an eager run. Counterpart of the reference's ``graphed_compute_step``
(exports/train_engine_0.5B/src/training_engine_tensor/step_graph.py:143-430) and
``forward_graph`` (forward_graph.py:66-272).
"""
from __future__ import annotations

import torch


class GraphedComputeStep:
    def __init__(self, model, warmup: int = 3, sanity: bool = False, tol: float = 1e-3):
        self.model = model
        self.warmup = max(1, warmup)
        self.sanity = sanity
        self.tol = tol
        self._graphs: dict = {}
        self.replays = 0

    def _key(self, batch: dict, loss_scale: float, accumulate: bool):
        t = batch["tokens"]
        return (tuple(t.shape), str(t.device), float(loss_scale), bool(accumulate),
                "loss_mask" in batch and batch["loss_mask"] is not None, "position_ids" in batch)

    def _capture(self, key, batch: dict, loss_scale: float, accumulate: bool):
        m = self.model
        static = {k: v.clone() for k, v in batch.items() if torch.is_tensor(v)}

        def run():
            return m.forward_backward(static["tokens"], static["labels"], static.get("loss_mask"),
                                      loss_scale, accumulate, None, static.get("position_ids"))
        keep = m.store.flat_grads.clone() if accumulate else None
        side = torch.cuda.Stream(device=static["tokens"].device)
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            for _ in range(self.warmup):
                eager_loss = run()
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        eager_val = float(eager_loss)
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            loss = run()
        if keep is not None:           # warm-up and capture must not leave their sums behind
            m.store.flat_grads.copy_(keep)
        entry = {"graph": g, "static": static, "loss": loss}
        if self.sanity:
            saved = m.store.flat_grads.clone()
            g.replay()
            torch.cuda.synchronize()
            got = float(loss)
            m.store.flat_grads.copy_(saved)
            if abs(got - eager_val) > self.tol * max(1.0, abs(eager_val)):
                raise RuntimeError(f"graph replay loss {got} differs from eager loss {eager_val}")
        self._graphs[key] = entry
        return entry

    def __call__(self, batch: dict, loss_scale: float, accumulate: bool) -> torch.Tensor:
        key = self._key(batch, loss_scale, accumulate)
        e = self._graphs.get(key)
        if e is None:
            e = self._capture(key, batch, loss_scale, accumulate)
        for k, v in e["static"].items():
            v.copy_(batch[k], non_blocking=True)
        e["graph"].replay()
        self.replays += 1
        return e["loss"]


class GraphedFullStep:
    """A whole optimizer step in ONE CUDA graph: every micro-batch's forward + loss + backward,
    the gradient-norm partials, the clip coefficient, the fused AdamW update of the master
    weights and the bf16 parameter write-back.

    What changes from step to step is either device state the graph itself advances (weights,
    moments, gradients) or a handful of scalars (learning rate, bias corrections) that the host
    stages in a pinned vector before the replay; the captured copy node reads them at replay
    time. The first ``warmup`` calls run eagerly (they are real training steps and also warm
    the allocator and the tensor-map cache); the next call captures (capture launches nothing)
    and replays. One graph is kept per (number of micro-batches, input shape).

    Plays the role of the reference's ``step_graph_full`` / ``step_graph_optimizer`` wrappers
    (exports/train_engine_0.5B/src/training_engine_tensor/step_graph_full.py:147-482,
    step_graph_nccl_opt.py:116-261, step_graph_optimizer.py:112-272). With data parallelism over
    the peer-memory collectives (bucket reduce-scatter, fused AdamW + all-gather, small
    all-reduces) those kernels are part of the graph: their barrier epochs are relative launch
    arguments plus a device-side base that the last node of the graph advances, and every rank
    replays the same graph in the same step.
    """

    def __init__(self, trainer, warmup: int = 3):
        self.trainer = trainer
        self.warmup = max(1, warmup)
        self.calls = 0
        self.replays = 0
        self._graphs: dict = {}

    @staticmethod
    def _key(micro_batches):
        return tuple((tuple(b["tokens"].shape), tuple(sorted(k for k, v in b.items()
                                                             if torch.is_tensor(v))))
                     for b in micro_batches)

    def __call__(self, micro_batches: list[dict]) -> None:
        tr = self.trainer
        self.calls += 1
        if self.calls <= self.warmup:
            tr._device_step(micro_batches)
            return
        key = self._key(micro_batches)
        e = self._graphs.get(key)
        if e is None:
            static = [{k: v.clone() for k, v in b.items() if torch.is_tensor(v)}
                      for b in micro_batches]
            torch.cuda.synchronize()
            symm = getattr(tr, "symm", None)   # peer-memory collectives: epochs go device-side
            if symm is not None:
                symm.begin_capture()
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                tr._device_step(static)
                if symm is not None:
                    symm.end_capture()
            e = {"graph": g, "static": static}
            self._graphs[key] = e
        for st, b in zip(e["static"], micro_batches):
            for k, v in st.items():
                v.copy_(b[k], non_blocking=True)
        e["graph"].replay()
        self.replays += 1


class GraphedForward:
    """Forward pass (logits) of a fixed input shape in a CUDA graph, for evaluation loops.
    Counterpart of the reference's ``forward_graph`` wrapper
    (exports/train_engine_0.5B/src/training_engine_tensor/forward_graph.py:66-272)."""

    def __init__(self, model, warmup: int = 2):
        self.model = model
        self.warmup = max(1, warmup)
        self._graphs: dict = {}
        self.replays = 0

    def __call__(self, tokens: torch.Tensor, position_ids: torch.Tensor | None = None):
        key = (tuple(tokens.shape), position_ids is not None)
        e = self._graphs.get(key)
        if e is None:
            st_tok = tokens.clone()
            st_pos = None if position_ids is None else position_ids.clone()
            side = torch.cuda.Stream(device=tokens.device)
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):
                for _ in range(self.warmup):
                    self.model.forward(st_tok, st_pos)
            torch.cuda.current_stream().wait_stream(side)
            torch.cuda.synchronize()
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                logits = self.model.forward(st_tok, st_pos)
            e = {"graph": g, "tokens": st_tok, "pos": st_pos, "logits": logits}
            self._graphs[key] = e
        e["tokens"].copy_(tokens, non_blocking=True)
        if e["pos"] is not None:
            e["pos"].copy_(position_ids, non_blocking=True)
        e["graph"].replay()
        self.replays += 1
        return e["logits"]
