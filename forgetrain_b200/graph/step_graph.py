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
