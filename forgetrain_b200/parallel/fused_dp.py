"""Data-parallel collectives as hand-written peer-memory kernels (``csrc/comm.cu``).

The flat fp32 gradient buffer and the flat bf16 parameter buffer live in symmetric memory
(``torch.distributed._symmetric_memory``: the same allocation on every rank of the
data-parallel group, every peer mapped into this process, plus an NVLS multicast mapping when
the fabric offers one). On top of the raw pointers:

* ``reduce_scatter_bucket``: ONE kernel per bucket does entry barrier, in-switch (``multimem``)
  or peer-load reduction of this rank's shard, the 1/W scale, the squared-norm partial and the
  exit barrier: no separate scale / norm kernels and no staging copy;
* ``all_gather_bucket``: one kernel pushes the freshly updated bf16 shard into every peer's
  parameter buffer (``multimem.st`` or peer stores) and waits for every peer's push;
* ``all_reduce_small``: a one-CTA all-reduce for a handful of floats (gradient norm, loss).

Every device-side wait is bounded (``timeout_ms``); a wait that runs out sets the status word
that :func:`forgetrain_b200.ops._lib.check_status` reports. ``use_multimem=False`` keeps all
traffic on plain peer loads / stores (used by the failure-handling tests).
"""
from __future__ import annotations

import ctypes
import os

import torch
import torch.distributed as dist

from ..ops import _lib

NUM_FLAG_SLOTS = 8
SCRATCH_FLOATS = 64 * 16


def _as_i32(e: int) -> int:
    """The bit pattern of a 32-bit epoch as the signed value an int32 tensor holds."""
    e &= 0xFFFFFFFF
    return e - (1 << 32) if e & 0x80000000 else e


def bump_epoch(e: int) -> int:
    """The epoch after ``e``. Full 32-bit counters: the device compares
    ``(int32)(flag - epoch) >= 0``, which is wrap-safe only when host and device count
    modulo 2^32 alike (a counter that wrapped at 2^31 would find the stale flag already
    "ahead" and pass every wait on that slot without waiting)."""
    return (e + 1) & 0xFFFFFFFF


class SymmetricBuffers:
    """Symmetric allocations shared by the ranks of one process group."""

    def __init__(self, n_elems: int, device: torch.device, group, rank: int, world: int,
                 use_multimem: bool | None = None):
        import torch.distributed._symmetric_memory as symm_mem
        self.group, self.rank, self.world = group, rank, world
        self.n = n_elems
        gname = group.group_name if group is not None else dist.group.WORLD.group_name
        self.grads = symm_mem.empty(n_elems, dtype=torch.float32, device=device)
        self.params = symm_mem.empty(n_elems, dtype=torch.bfloat16, device=device)
        self.flags = symm_mem.empty(NUM_FLAG_SLOTS * 16, dtype=torch.int32, device=device)
        self.scratch = symm_mem.empty(SCRATCH_FLOATS, dtype=torch.float32, device=device)
        self.grads.zero_()
        self.params.zero_()
        self.flags.zero_()
        self.scratch.zero_()
        torch.cuda.synchronize(device)
        self.h_grads = symm_mem.rendezvous(self.grads, gname)
        self.h_params = symm_mem.rendezvous(self.params, gname)
        self.h_flags = symm_mem.rendezvous(self.flags, gname)
        self.h_scratch = symm_mem.rendezvous(self.scratch, gname)
        if use_multimem is None:
            use_multimem = os.environ.get("FT_COMM_MULTIMEM", "1") != "0"
        self.mc_grads = int(self.h_grads.multicast_ptr or 0) if use_multimem else 0
        self.mc_params = int(self.h_params.multicast_ptr or 0) if use_multimem else 0
        if world <= 2:
            # with a single peer a multicast store also rewrites the local copy: plain peer
            # stores move half the bytes
            self.mc_params = 0
        VP = ctypes.c_void_p * world
        self.p_grads = VP(*[int(p) for p in self.h_grads.buffer_ptrs])
        self.p_params = VP(*[int(p) for p in self.h_params.buffer_ptrs])
        self.p_flags = VP(*[int(p) for p in self.h_flags.buffer_ptrs])
        self.p_scratch = VP(*[int(p) for p in self.h_scratch.buffer_ptrs])
        self.done_ctr = torch.zeros(4, dtype=torch.int32, device=device)
        self.epoch = [0] * NUM_FLAG_SLOTS
        # Device-side epoch base (see begin_capture): zero in eager mode, where the host passes
        # absolute epochs; registered once so that every launch on these flags adds it.
        self.epoch_base = torch.zeros(NUM_FLAG_SLOTS, dtype=torch.int32, device=device)
        self._capturing = False
        self._graph_mode = False
        self._used = [0] * NUM_FLAG_SLOTS
        _lib.lib().ft_comm_set_epoch_base(ctypes.c_void_p(int(self.h_flags.buffer_ptrs[rank])),
                                          _lib.ptr(self.epoch_base))
        dist.barrier(group=group)

    def next_epoch(self, slot: int) -> int:
        if self._capturing:
            # relative numbering inside a captured step: the device base supplies the rest
            self._used[slot] += 1
            return self._used[slot]
        if self._graph_mode:
            raise RuntimeError("peer-memory collectives were captured in a CUDA graph; call "
                               "resync_epochs() before launching them eagerly again")
        self.epoch[slot] = bump_epoch(self.epoch[slot])
        return self.epoch[slot]

    def set_epoch(self, slot: int, value: int) -> None:
        """Mirror ``value`` (the epoch another slot just took) into ``slot``."""
        if self._capturing:
            self._used[slot] = value
        else:
            self.epoch[slot] = value

    # -- CUDA-graph support ---------------------------------------------------------------
    def begin_capture(self) -> None:
        """Call right before capturing a step that launches these collectives. From here on the
        launch arguments are epochs relative to the device-side base, which is set to the epochs
        used so far; :meth:`end_capture` (inside the capture) appends the kernel that advances
        the base by what one replay consumes. Every rank must capture the same sequence."""
        if self._graph_mode:
            self.resync_epochs()
        self.epoch_base.copy_(torch.tensor([_as_i32(e) for e in self.epoch], dtype=torch.int32))
        self._used = [0] * NUM_FLAG_SLOTS
        self._capturing = True

    def end_capture(self) -> None:
        add = (ctypes.c_uint * NUM_FLAG_SLOTS)(*self._used)
        rc = _lib.lib().ft_comm_epoch_advance(_lib.ptr(self.epoch_base), add, _lib.stream())
        _lib.check_rc(rc, "ft_comm_epoch_advance")
        self._capturing = False
        self._graph_mode = True

    def resync_epochs(self) -> None:
        """Back to eager launches after graph replays: read the base back (synchronises)."""
        base = self.epoch_base.cpu().tolist()
        self.epoch = [int(b) & 0xFFFFFFFF for b in base]
        self.epoch_base.zero_()
        self._graph_mode = False


class FusedDPComm:
    def __init__(self, symm: SymmetricBuffers, timeout_ms: int | None = None, ctas: int = 0):
        self.s = symm
        if timeout_ms is None:
            timeout_ms = int(os.environ.get("FT_COMM_TIMEOUT_MS", "30000"))
        self.limit_ns = int(timeout_ms) * 1_000_000
        self.ctas = ctas or int(os.environ.get("FT_COMM_CTAS", "96"))
        self.status = _lib.status_word(symm.grads.device)
        self.comm_stream = None
        self.ag_events: list = []

    # -- gradient reduce-scatter ---------------------------------------------------------
    def reduce_scatter_bucket(self, b, sumsq: torch.Tensor, scale: float | None = None) -> None:
        s = self.s
        ep = s.next_epoch(0)
        s.set_epoch(1, ep)
        rc = _lib.lib().ft_bucket_reduce_scatter(
            s.p_grads, s.p_flags, ctypes.c_void_p(s.mc_grads), ctypes.c_int(s.rank),
            ctypes.c_int(s.world), ctypes.c_long(b.start), ctypes.c_long(b.size // s.world),
            ctypes.c_float(1.0 / s.world if scale is None else scale), _lib.ptr(sumsq),
            ctypes.c_uint(ep), ctypes.c_ulonglong(self.limit_ns), _lib.ptr(s.done_ctr),
            ctypes.c_int(self.ctas), _lib.ptr(self.status), _lib.stream())
        _lib.check_rc(rc, "ft_bucket_reduce_scatter")

    # -- parameter all-gather ------------------------------------------------------------
    def all_gather_bucket(self, b) -> None:
        s = self.s
        ep = s.next_epoch(2)
        rc = _lib.lib().ft_bucket_all_gather(
            s.p_params, s.p_flags, ctypes.c_void_p(s.mc_params), ctypes.c_int(s.rank),
            ctypes.c_int(s.world), ctypes.c_long(b.start), ctypes.c_long(b.size // s.world),
            ctypes.c_uint(ep), ctypes.c_ulonglong(self.limit_ns),
            _lib.c_void_p(s.done_ctr.data_ptr() + 4), ctypes.c_int(self.ctas),
            _lib.ptr(self.status), _lib.stream())
        _lib.check_rc(rc, "ft_bucket_all_gather")

    def adamw_all_gather(self, b, p32, m, v, g, hyper, seg_end, seg_wd, seg_lr_mult) -> None:
        """AdamW on this rank's shard of bucket ``b`` with the bf16 results stored straight
        into every rank's parameter buffer (one kernel instead of update + all-gather)."""
        s = self.s
        ep = s.next_epoch(2)
        rc = _lib.lib().ft_adamw_all_gather(
            s.p_params, s.p_flags, ctypes.c_void_p(s.mc_params), ctypes.c_int(s.rank),
            ctypes.c_int(s.world), ctypes.c_long(b.start), ctypes.c_long(b.size // s.world),
            _lib.ptr(p32), _lib.ptr(m), _lib.ptr(v), _lib.ptr(g), _lib.ptr(hyper),
            _lib.ptr(seg_end), _lib.ptr(seg_wd), _lib.ptr(seg_lr_mult),
            ctypes.c_int(seg_end.numel()), ctypes.c_uint(ep), ctypes.c_ulonglong(self.limit_ns),
            _lib.c_void_p(s.done_ctr.data_ptr() + 4), ctypes.c_int(0), _lib.ptr(self.status),
            _lib.stream())
        _lib.check_rc(rc, "ft_adamw_all_gather")

    def wait_all_gathers(self) -> None:
        return  # the kernels run on the caller's stream; stream order is the dependency

    # -- a few floats ----------------------------------------------------------------------
    def all_reduce_small(self, vals: torch.Tensor) -> None:
        """In-place sum over the group of up to 64 fp32 values."""
        s = self.s
        assert vals.dtype == torch.float32 and vals.numel() <= 64
        ep = s.next_epoch(3)
        s.set_epoch(4, ep)
        rc = _lib.lib().ft_small_all_reduce(
            s.p_scratch, s.p_flags, ctypes.c_int(s.rank), ctypes.c_int(s.world), ctypes.c_long(0),
            _lib.ptr(vals), ctypes.c_int(vals.numel()), ctypes.c_uint(ep),
            ctypes.c_ulonglong(self.limit_ns), _lib.ptr(self.status), _lib.stream())
        _lib.check_rc(rc, "ft_small_all_reduce")

    def barrier(self, slot: int = 5, signal: bool = True, timeout_ms: int | None = None) -> None:
        s = self.s
        ep = s.next_epoch(slot)
        limit = self.limit_ns if timeout_ms is None else int(timeout_ms) * 1_000_000
        rc = _lib.lib().ft_peer_barrier(s.p_flags, ctypes.c_int(s.rank), ctypes.c_int(s.world),
                                        ctypes.c_int(slot), ctypes.c_uint(ep),
                                        ctypes.c_ulonglong(limit), ctypes.c_int(int(signal)),
                                        _lib.ptr(self.status), _lib.stream())
        _lib.check_rc(rc, "ft_peer_barrier")
