"""An in-process stand-in for ``torch.distributed``: W threads are the ranks, collectives meet at a
barrier. Lets the host-side data-parallel logic (bucket reduction, sharded optimizer, state
gathering) run at any world size in one CPU process, without sockets or child processes."""
from __future__ import annotations

import threading

import torch
import torch.distributed as real_dist


class SimDist:
    ReduceOp = real_dist.ReduceOp

    def __init__(self, world: int):
        self.world = world
        self._barrier = threading.Barrier(world)
        self._slots: list = [None] * world
        self._tls = threading.local()
        self.calls: list[str] = []          # collectives seen by rank 0, in order

    # -- rank identity ---------------------------------------------------------------------
    def rank(self) -> int:
        return self._tls.rank

    def _exchange(self, value):
        """Every rank deposits ``value``; returns the list of all ranks' values."""
        self._slots[self.rank()] = value
        self._barrier.wait()
        got = list(self._slots)
        self._barrier.wait()                # nobody overwrites a slot before all have read
        return got

    # -- the collectives the engine's CPU path uses ---------------------------------------------
    def all_reduce(self, t: torch.Tensor, op=None, group=None):
        if self.rank() == 0:
            self.calls.append(f"all_reduce[{t.numel()}]")
        parts = self._exchange(t.detach().clone())
        if op == self.ReduceOp.MAX:
            out = torch.stack(parts).amax(0)
        else:
            out = torch.stack(parts).sum(0)
        t.copy_(out)

    def all_gather(self, out_list, t: torch.Tensor, group=None):
        if self.rank() == 0:
            self.calls.append(f"all_gather[{t.numel()}]")
        parts = self._exchange(t.detach().clone())
        for dst, src in zip(out_list, parts):
            dst.copy_(src)

    def barrier(self, group=None):
        self._exchange(None)

    # -- running the ranks -------------------------------------------------------------------
    def run(self, fn):
        """Run ``fn(rank)`` on every rank; returns the results in rank order. The first
        exception of any rank is re-raised here (the others are released from the barrier)."""
        results: list = [None] * self.world
        errors: list = []

        def body(r):
            self._tls.rank = r
            try:
                results[r] = fn(r)
            except threading.BrokenBarrierError:
                pass
            except BaseException as e:          # noqa: BLE001 - re-raised below
                errors.append(e)
                self._barrier.abort()

        threads = [threading.Thread(target=body, args=(r,)) for r in range(self.world)]
        for th in threads:
            th.start()
        for th in threads:
            th.join(timeout=120)
        if errors:
            raise errors[0]
        assert not any(th.is_alive() for th in threads), "a simulated rank did not finish"
        return results
