"""Host model of the epoch-flag protocol of the peer-memory collectives (csrc/comm.cu:
``signal_peers`` / ``wait_peers`` and the entry / exit barriers of ``bucket_reduce_scatter_kernel``).

Every rank owns a board ``flags[slot][src]``; ``signal`` stores the caller's epoch into its column
of EVERY rank's board, ``wait`` polls the caller's own board until every column has reached the
epoch (signed 32-bit difference, so it survives wrap-around) or a time limit passes, in which
case it reports failure instead of blocking. Ranks are threads; the model exists so that late,
missing and wrapped-around signals can be tested without a GPU."""
from __future__ import annotations

import threading
import time

import numpy as np

ERR_WAIT_PEER = 6      # any non-zero code; the value is not part of the protocol


def _i32(x: int) -> int:
    x &= 0xFFFFFFFF
    return x - (1 << 32) if x & 0x80000000 else x


class FlagBoards:
    def __init__(self, world: int, slots: int = 8):
        self.world, self.slots = world, slots
        self.flags = np.zeros((world, slots, world), dtype=np.uint32)   # [owner][slot][src]
        self.base = np.zeros((world, slots), dtype=np.uint32)           # device-side epoch base
        self.status = [0] * world

    def signal(self, rank: int, slot: int, epoch: int) -> None:
        e = (epoch + int(self.base[rank, slot])) & 0xFFFFFFFF
        for peer in range(self.world):
            self.flags[peer, slot, rank] = e

    def wait(self, rank: int, slot: int, epoch: int, limit_s: float) -> bool:
        e = (epoch + int(self.base[rank, slot])) & 0xFFFFFFFF
        t0 = time.monotonic()
        while True:
            if all(_i32(int(self.flags[rank, slot, src]) - e) >= 0 for src in range(self.world)):
                return True
            if time.monotonic() - t0 > limit_s:
                if self.status[rank] == 0:
                    self.status[rank] = ERR_WAIT_PEER
                return False
            time.sleep(0.0005)


def reduce_scatter(boards: FlagBoards, bufs: list[np.ndarray], rank: int, epoch: int,
                   limit_s: float = 1.0, delay_s: float = 0.0, skip_signal: bool = False) -> float:
    """One rank's part of the in-place bucket reduce-scatter: entry barrier (slot 0), read every
    peer's copy of this rank's shard, write the mean into the own copy, exit barrier (slot 1).
    Returns the squared norm of the reduced shard (0 when a wait ran out)."""
    w = boards.world
    n = bufs[rank].size // w
    if delay_s:
        time.sleep(delay_s)
    if not skip_signal:
        boards.signal(rank, 0, epoch)
    if not boards.wait(rank, 0, epoch, limit_s):
        return 0.0
    lo, hi = rank * n, (rank + 1) * n
    acc = np.zeros(n, dtype=np.float32)
    for peer in range(w):
        acc += bufs[peer][lo:hi]
    acc /= w
    bufs[rank][lo:hi] = acc
    boards.signal(rank, 1, epoch)
    boards.wait(rank, 1, epoch, limit_s)     # peers may still be reading this rank's buffer
    return float((acc * acc).sum())


def run_ranks(world: int, fn):
    out = [None] * world
    th = [threading.Thread(target=lambda r=r: out.__setitem__(r, fn(r))) for r in range(world)]
    for t in th:
        t.start()
    for t in th:
        t.join(timeout=30)
    assert not any(t.is_alive() for t in th)
    return out
