"""Tensor-parallel context: the collectives the model calls between tensor-parallel regions.

With sequence parallelism the residual stream is sharded over tokens: ``gather`` is an
all-gather along the token dimension (before a column-parallel GEMM) and ``scatter_reduce`` a
reduce-scatter (after a row-parallel GEMM). Without it the residual stream is replicated:
``gather`` is the identity and ``scatter_reduce`` an all-reduce, which is the reference's
pattern (exports/train_engine_8b/src/training_engine_tensor/forward.py:127,246,267 and
backward.py:454,580,725). The backward of ``gather`` is ``scatter_reduce`` and vice versa.

The collectives themselves come from a *backend*: ``torch.distributed`` (NCCL on GPUs, gloo on
CPU) or the fused peer-memory kernels of :mod:`forgetrain_b200.parallel.fused_tp`, which
overlap the transfer with the neighbouring GEMM.
"""
from __future__ import annotations

import torch
import torch.distributed as dist


class TPContext:
    def __init__(self, group=None, size: int = 1, rank: int = 0, sequence_parallel: bool = True,
                 replica_group=None, replica_size: int = 1):
        self.group = group
        self.size = size
        self.rank = rank
        self.sequence_parallel = sequence_parallel and size > 1
        # ranks that hold replicas of the same KV head (tp > num_query_groups)
        self.replica_group = replica_group
        self.replica_size = replica_size

    @property
    def enabled(self) -> bool:
        return self.size > 1

    def local_tokens(self, T: int) -> int:
        return T // self.size if self.sequence_parallel else T

    # -- activations ---------------------------------------------------------------------
    def gather(self, x: torch.Tensor) -> torch.Tensor:
        if not self.sequence_parallel:
            return x
        out = torch.empty(x.shape[0] * self.size, *x.shape[1:], dtype=x.dtype, device=x.device)
        dist.all_gather_into_tensor(out, x.contiguous(), group=self.group)
        return out

    def scatter_reduce(self, y: torch.Tensor) -> torch.Tensor:
        if self.size == 1:
            return y
        if not self.sequence_parallel:
            dist.all_reduce(y, group=self.group)
            return y
        out = torch.empty(y.shape[0] // self.size, *y.shape[1:], dtype=y.dtype, device=y.device)
        if y.is_cuda:
            dist.reduce_scatter_tensor(out, y.contiguous(), group=self.group)
        else:  # gloo has no reduce_scatter_tensor for every dtype: all-reduce then slice
            tmp = y.float()
            dist.all_reduce(tmp, group=self.group)
            n = out.shape[0]
            out.copy_(tmp[self.rank * n:(self.rank + 1) * n].to(y.dtype))
        return out

    def slice_tokens(self, x: torch.Tensor) -> torch.Tensor:
        """This rank's token shard of a replicated tensor (no communication)."""
        if not self.sequence_parallel:
            return x
        n = x.shape[0] // self.size
        return x[self.rank * n:(self.rank + 1) * n]

    def gather_dest(self, key: str, rows_local: int, cols: int):
        """Where the producer of a to-be-gathered activation should write its token shard so
        that ``linear_gather(key=...)`` needs no staging copy (None: anywhere)."""
        return None

    # -- GEMM + collective pairs (overridden by the fused peer-memory implementation) --------
    def linear_gather(self, x, w, alpha: float = 1.0, key: str | None = None):
        """``(alpha * gather(x) @ w.T, gather(x))`` for a column-parallel weight."""
        from .. import ops
        xf = self.gather(x)
        return ops.linear_fwd(xf, w, alpha), xf

    def linear_scatter(self, x, w, alpha: float = 1.0):
        """``scatter_reduce(alpha * x @ w.T)`` for a row-parallel weight."""
        from .. import ops
        return self.scatter_reduce(ops.linear_fwd(x, w, alpha))

    def dgrad_gather(self, dy, w, alpha: float = 1.0, key: str | None = None):
        """``(alpha * gather(dy) @ w, gather(dy))``: backward of ``linear_scatter``."""
        from .. import ops
        df = self.gather(dy)
        return ops.linear_dgrad(df, w, alpha), df

    def dgrad_gather_swiglu_bwd(self, dy, w2, y1, alpha: float = 1.0, key: str | None = None):
        """``(swiglu_bwd(alpha * gather(dy) @ w2, y1), gather(dy))``: FC2 dgrad with the
        activation backward in the GEMM epilogue (one kernel on CUDA)."""
        from .. import ops
        df = self.gather(dy)
        return ops.linear_dgrad_swiglu_bwd(df, w2, y1, alpha), df

    def dgrad_scatter(self, dy, w, alpha: float = 1.0):
        """``scatter_reduce(alpha * dy @ w)``: backward of ``linear_gather``."""
        from .. import ops
        return self.scatter_reduce(ops.linear_dgrad(dy, w, alpha))

    # -- small statistics (vocab-parallel cross-entropy) -----------------------------------
    def stats_reduce(self, x: torch.Tensor, op: str) -> torch.Tensor:
        if self.size == 1:
            return x
        dist.all_reduce(x, op=dist.ReduceOp.MAX if op == "max" else dist.ReduceOp.SUM,
                        group=self.group)
        return x

    def all_reduce_(self, x: torch.Tensor) -> torch.Tensor:
        if self.size > 1:
            dist.all_reduce(x, group=self.group)
        return x

    def replica_all_reduce_(self, x: torch.Tensor) -> torch.Tensor:
        if self.replica_size > 1:
            dist.all_reduce(x, group=self.replica_group)
        return x


NO_TP = TPContext()
