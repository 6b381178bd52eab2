"""Tensor-parallel context whose GEMM + collective pairs run as ONE kernel over NVLink peer
memory (``csrc/gemm_tp_sm100.cu``): all-gather -> GEMM for column-parallel layers and
GEMM -> reduce-scatter for row-parallel layers, forward and backward.

Symmetric memory owned here (one allocation per kind, shared by all layers):

* a pool of gather buffers ``[n_slots][T][H]`` bf16: the producer's token shard is written into
  this rank's row slot, the fused kernel pulls the peers' slots while it computes; the filled
  buffer doubles as the saved activation for the weight-gradient GEMM;
* two alternating partial-sum areas ``[tp][T/tp][H]`` bf16 for GEMM -> reduce-scatter: every
  rank stores its partial output tiles straight into the owner's plane, the owner sums the
  planes in fp32 afterwards (deterministic, no atomics);
* the flag arrays used to order the ranks; all device-side waits are bounded.

Falls back to the base class (separate collective + GEMM) for shapes the fused kernel does
not take (row slot not a multiple of 128 tokens, weight narrower than one tile).
"""
from __future__ import annotations

import ctypes
import os

import torch
import torch.distributed as dist

from ..ops import _lib
from .tp import TPContext
from .fused_dp import bump_epoch

c_int, c_float, c_uint, c_ull = ctypes.c_int, ctypes.c_float, ctypes.c_uint, ctypes.c_ulonglong


class FusedTPContext(TPContext):
    def __init__(self, group, size: int, rank: int, device: torch.device, tokens: int, hidden: int,
                 n_gather_slots: int, replica_group=None, replica_size: int = 1,
                 timeout_ms: int | None = None):
        super().__init__(group, size, rank, True, replica_group, replica_size)
        import torch.distributed._symmetric_memory as symm_mem
        assert tokens % size == 0
        self.T, self.H = tokens, hidden
        self.device = device
        gname = group.group_name
        self.pool = symm_mem.empty(n_gather_slots * tokens * hidden, dtype=torch.bfloat16, device=device)
        self.partials = symm_mem.empty(2 * tokens * hidden, dtype=torch.bfloat16, device=device)
        self.flags = symm_mem.empty(8 * 16, dtype=torch.int32, device=device)
        self.ce_stats = symm_mem.empty(3 * tokens, dtype=torch.float32, device=device)
        self.pool.zero_()
        self.partials.zero_()
        self.flags.zero_()
        self.ce_stats.zero_()
        torch.cuda.synchronize(device)
        self.h_pool = symm_mem.rendezvous(self.pool, gname)
        self.h_part = symm_mem.rendezvous(self.partials, gname)
        self.h_flags = symm_mem.rendezvous(self.flags, gname)
        self.h_ce = symm_mem.rendezvous(self.ce_stats, gname)
        self.p_ce = (ctypes.c_void_p * size)(*[int(p) for p in self.h_ce.buffer_ptrs])
        self.epoch_ce = 0
        self.pool_ptrs = [int(p) for p in self.h_pool.buffer_ptrs]
        self.part_ptrs = [int(p) for p in self.h_part.buffer_ptrs]
        VP = ctypes.c_void_p * size
        self.p_flags = VP(*[int(p) for p in self.h_flags.buffer_ptrs])
        self.n_slots = n_gather_slots
        self.slot_of: dict[str, int] = {}
        self.chunk_ready = torch.zeros(4096, dtype=torch.int32, device=device)
        self.done_ctr = torch.zeros(4, dtype=torch.int32, device=device)
        self.status = _lib.status_word(device)
        if timeout_ms is None:
            timeout_ms = int(os.environ.get("FT_COMM_TIMEOUT_MS", "30000"))
        self.limit_ns = int(timeout_ms) * 1_000_000
        self.epoch_ag = 0
        self.epoch_rs = 0
        self.rs_toggle = 0
        dist.barrier(group=group)

    # ------------------------------------------------------------------ buffers
    def _slot(self, key: str) -> int:
        s = self.slot_of.get(key)
        if s is None:
            s = len(self.slot_of)
            if s >= self.n_slots:
                raise RuntimeError(f"gather pool exhausted ({self.n_slots} slots) at key {key!r}")
            self.slot_of[key] = s
        return s

    def _gather_view(self, slot: int, rows: int, cols: int) -> torch.Tensor:
        o = slot * self.T * self.H
        return self.pool[o:o + rows * cols].view(rows, cols)

    def _fusable(self, rows_full: int, n_out: int, k: int) -> bool:
        return (rows_full % self.size == 0 and (rows_full // self.size) % 128 == 0 and n_out >= 64
                and k % 8 == 0 and rows_full * max(k, n_out) <= self.T * self.H * 4)

    def gather_dest(self, key: str, rows_local: int, cols: int):
        M = rows_local * self.size
        if cols != self.H or M > self.T or not self._fusable(M, 64, cols):
            return None
        xg = self._gather_view(self._slot(key), M, cols)
        return xg[self.rank * rows_local:(self.rank + 1) * rows_local]

    # ------------------------------------------------------------------ all-gather -> GEMM
    def _ag_gemm(self, x_local, w, alpha, key, b_mn: bool):
        rows_local, K = x_local.shape
        M = rows_local * self.size
        N = w.shape[1] if b_mn else w.shape[0]
        if key is None or K != self.H or not self._fusable(M, N, K) or M > self.T:
            return None
        slot = self._slot(key)
        xg = self._gather_view(slot, M, K)
        mine = xg[self.rank * rows_local:(self.rank + 1) * rows_local]
        if mine.data_ptr() != x_local.data_ptr():
            mine.copy_(x_local)
        out = torch.empty(M, N, dtype=torch.bfloat16, device=x_local.device)
        base = slot * self.T * self.H * 2
        VP = ctypes.c_void_p * self.size
        a_peers = VP(*[p + base for p in self.pool_ptrs])
        self.epoch_ag = bump_epoch(self.epoch_ag)
        rc = _lib.lib().ft_gemm_ag(a_peers, _lib.ptr(w), _lib.ptr(out), c_int(M), c_int(N), c_int(K),
                                   c_int(w.stride(0)), c_int(out.stride(0)), c_int(int(b_mn)),
                                   c_float(alpha), c_int(self.size), c_int(self.rank), self.p_flags,
                                   c_uint(self.epoch_ag), c_ull(self.limit_ns),
                                   _lib.ptr(self.chunk_ready), _lib.ptr(self.done_ctr),
                                   _lib.ptr(self.status), _lib.stream())
        _lib.check_rc(rc, "ft_gemm_ag")
        return out, xg

    def linear_gather(self, x, w, alpha: float = 1.0, key: str | None = None):
        r = self._ag_gemm(x, w, alpha, key, b_mn=False) if x.is_cuda else None
        return r if r is not None else super().linear_gather(x, w, alpha, key)

    def dgrad_gather(self, dy, w, alpha: float = 1.0, key: str | None = None):
        r = self._ag_gemm(dy, w, alpha, key, b_mn=True) if dy.is_cuda else None
        return r if r is not None else super().dgrad_gather(dy, w, alpha, key)

    # ------------------------------------------------------------------ GEMM -> reduce-scatter
    def dgrad_gather_swiglu_bwd(self, dy, w2, y1, alpha: float = 1.0, key: str | None = None):
        # the all-gather -> GEMM kernel has the plain epilogue: activation backward as a second kernel
        from .. import ops
        dact, df = self.dgrad_gather(dy, w2, alpha, key)
        return ops.swiglu_bwd(dact, y1), df

    def _gemm_rs(self, x, w, alpha, b_mn: bool):
        M, K = x.shape
        N = w.shape[1] if b_mn else w.shape[0]
        if not self._fusable(M, N, K) or M * N > self.T * self.H or x.stride(1) != 1:
            return None
        rows_local = M // self.size
        half = self.rs_toggle
        self.rs_toggle ^= 1
        base = half * self.T * self.H * 2
        VP = ctypes.c_void_p * self.size
        d_peers = VP(*[p + base for p in self.part_ptrs])
        self.epoch_rs = bump_epoch(self.epoch_rs)
        rc = _lib.lib().ft_gemm_rs(_lib.ptr(x), _lib.ptr(w), d_peers, c_int(M), c_int(N), c_int(K),
                                   c_int(x.stride(0)), c_int(w.stride(0)), c_int(int(b_mn)),
                                   c_float(alpha), c_int(self.size), c_int(self.rank), self.p_flags,
                                   c_uint(self.epoch_rs), c_ull(self.limit_ns),
                                   _lib.c_void_p(self.done_ctr.data_ptr() + 4),
                                   _lib.ptr(self.status), _lib.stream())
        _lib.check_rc(rc, "ft_gemm_rs")
        plane = rows_local * N
        part = self.partials[half * self.T * self.H:half * self.T * self.H + self.size * plane]
        out = torch.empty(rows_local, N, dtype=torch.bfloat16, device=x.device)
        rc = _lib.lib().ft_tp_sum_partials(_lib.ptr(part), _lib.ptr(out), ctypes.c_long(plane),
                                           c_int(self.size), _lib.stream())
        _lib.check_rc(rc, "ft_tp_sum_partials")
        return out

    def linear_scatter(self, x, w, alpha: float = 1.0):
        r = self._gemm_rs(x, w, alpha, b_mn=False) if x.is_cuda else None
        return r if r is not None else super().linear_scatter(x, w, alpha)

    def dgrad_scatter(self, dy, w, alpha: float = 1.0):
        r = self._gemm_rs(dy, w, alpha, b_mn=True) if dy.is_cuda else None
        return r if r is not None else super().dgrad_scatter(dy, w, alpha)

    # ------------------------------------------------------------------ vocab-parallel CE
    def ce_stats_buffer(self, T: int):
        """[3][T] fp32 view in symmetric memory that the local statistics kernel writes."""
        if T > self.T:
            return None
        return self.ce_stats[:3 * T].view(3, T)

    def ce_exchange(self, T: int, mask, combined: torch.Tensor, row_loss: torch.Tensor) -> None:
        """One kernel: entry barrier, peer loads of every rank's statistics, combination,
        masked row loss, exit barrier."""
        self.epoch_ce = bump_epoch(self.epoch_ce)
        rc = _lib.lib().ft_ce_stats_exchange(
            self.p_ce, self.p_flags, c_int(self.rank), c_int(self.size), ctypes.c_long(0), c_int(T),
            _lib.ptr(mask), _lib.ptr(combined), _lib.ptr(row_loss), c_uint(self.epoch_ce),
            c_ull(self.limit_ns), _lib.c_void_p(self.done_ctr.data_ptr() + 8),
            _lib.ptr(self.status), _lib.stream())
        _lib.check_rc(rc, "ft_ce_stats_exchange")
