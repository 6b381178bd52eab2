"""Process topology: DP x TP mesh on one node, process groups, device binding.

Tensor-parallel groups are consecutive ranks, data-parallel groups are strided by the TP
degree (reference: exports/train_engine_8b/src/training_engine_tensor/nccl.py:36-67). One
process drives one GPU; on CPU (gloo) the same code runs for plumbing tests.
"""
from __future__ import annotations

import datetime
import os
from dataclasses import dataclass

import torch
import torch.distributed as dist


@dataclass
class Topology:
    rank: int = 0
    world: int = 1
    local_rank: int = 0
    tp_size: int = 1
    dp_size: int = 1
    tp_rank: int = 0
    dp_rank: int = 0
    tp_group: object = None
    dp_group: object = None
    replica_group: object = None
    replica_size: int = 1
    device: torch.device = torch.device("cpu")
    backend: str = "none"

    @property
    def distributed(self) -> bool:
        return self.world > 1


def node_layout(world: int, ranks_per_node: int | None, tp_size: int) -> tuple[bool, bool]:
    """``(multi_node, tp_groups_inside_a_node)`` for ``world`` ranks launched ``ranks_per_node`` to
    a node. Tensor-parallel groups are runs of consecutive ranks, so they stay inside a node iff
    the TP degree divides the ranks per node; data-parallel groups are strided and span nodes as
    soon as there is more than one. Peer-memory kernels are only used inside a node."""
    per = ranks_per_node or world
    multi = per < world
    return multi, (not multi) or (tp_size <= per and per % tp_size == 0)


def resolve_env() -> tuple[int, int, int]:
    return (int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1")),
            int(os.environ.get("LOCAL_RANK", "0")))


def init_topology(tp_size: int = 1, device: str | None = None, backend: str | None = None,
                  timeout_s: int = 600, num_kv_groups: int | None = None) -> Topology:
    """Bring up ``torch.distributed`` (when WORLD_SIZE > 1) and the DP / TP groups."""
    rank, world, local_rank = resolve_env()
    use_cuda = torch.cuda.is_available() and (device is None or str(device).startswith("cuda"))
    if use_cuda:
        torch.cuda.set_device(local_rank % torch.cuda.device_count())
        dev = torch.device("cuda", torch.cuda.current_device())
    else:
        dev = torch.device("cpu")
    backend = backend or ("nccl" if use_cuda else "gloo")
    if world % tp_size:
        raise ValueError(f"world size {world} is not a multiple of the TP degree {tp_size}")
    topo = Topology(rank=rank, world=world, local_rank=local_rank, tp_size=tp_size,
                    dp_size=world // tp_size, tp_rank=rank % tp_size, dp_rank=rank // tp_size,
                    device=dev, backend=backend if world > 1 else "none")
    global _current
    _current = topo
    if world == 1:
        return topo
    if not dist.is_initialized():
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29500")
        kw = dict(backend=backend, rank=rank, world_size=world,
                  timeout=datetime.timedelta(seconds=timeout_s))
        if use_cuda:
            kw["device_id"] = dev
        dist.init_process_group(**kw)
    # every rank must create every group, in the same order
    for d in range(topo.dp_size):
        ranks = list(range(d * tp_size, (d + 1) * tp_size))
        g = dist.new_group(ranks) if tp_size > 1 else None
        if d == topo.dp_rank:
            topo.tp_group = g
    for t in range(tp_size):
        ranks = list(range(t, world, tp_size))
        g = dist.new_group(ranks) if topo.dp_size > 1 else None
        if t == topo.tp_rank:
            topo.dp_group = g
    if num_kv_groups and tp_size > num_kv_groups:
        rep = tp_size // num_kv_groups
        topo.replica_size = rep
        for d in range(topo.dp_size):
            for kg in range(num_kv_groups):
                ranks = [d * tp_size + kg * rep + i for i in range(rep)]
                g = dist.new_group(ranks)
                if rank in ranks:
                    topo.replica_group = g
    return topo


def shutdown() -> None:
    global _current
    _current = None
    if dist.is_available() and dist.is_initialized():
        dist.destroy_process_group()


# -----------------------------------------------------------------------------------------
# The process's topology as module-level accessors, for code that does not carry the object
# around (the reference's nccl modules offer the same: 0.5B nccl.py:61-76, 8B nccl.py:77-104).
# Before ``init_topology`` they describe a single process.
# -----------------------------------------------------------------------------------------
_current: Topology | None = None


def current() -> Topology:
    return _current if _current is not None else Topology()


def is_distributed() -> bool:
    return current().world > 1


def get_rank() -> int:
    return current().rank


def get_world_size() -> int:
    return current().world


def get_dp_group():
    return current().dp_group


def get_dp_rank() -> int:
    return current().dp_rank


def get_dp_size() -> int:
    return current().dp_size


def get_tp_group():
    return current().tp_group


def get_tp_rank() -> int:
    return current().tp_rank


def get_tp_size() -> int:
    return current().tp_size


def barrier() -> None:
    if dist.is_available() and dist.is_initialized():
        dist.barrier()


def allreduce_loss(local_loss: torch.Tensor, dp_group=None, dp_size: int | None = None) -> float:
    """Mean of a scalar loss over the data-parallel ranks, in place; returns it as a float (a
    host synchronisation). Defaults to the current topology's data-parallel group."""
    topo = current()
    n = topo.dp_size if dp_size is None else dp_size
    if n > 1:
        dist.all_reduce(local_loss, op=dist.ReduceOp.SUM,
                        group=topo.dp_group if dp_group is None else dp_group)
        local_loss.div_(n)
    return float(local_loss)
