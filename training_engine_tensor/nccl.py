"""``training_engine_tensor.nccl``: process groups, bucket layout and the gradient reducer under the
reference's module name (0.5B nccl.py:39-76, 8B nccl.py:17-104,268-280)."""
from forgetrain_b200.parallel.buckets import Bucket, compute_grad_buckets  # noqa: F401
from forgetrain_b200.parallel.dp import BucketedGradReducer  # noqa: F401
from forgetrain_b200.parallel.topology import (  # noqa: F401
    Topology, allreduce_loss, barrier, get_dp_group, get_dp_rank, get_dp_size, get_rank, get_tp_group,
    get_tp_rank, get_tp_size, get_world_size, init_topology, is_distributed, node_layout, shutdown)

__all__ = ["Bucket", "compute_grad_buckets", "BucketedGradReducer", "Topology", "init_topology",
           "node_layout", "shutdown", "is_distributed", "get_rank", "get_world_size", "barrier",
           "get_dp_group", "get_dp_rank", "get_dp_size", "get_tp_group", "get_tp_rank", "get_tp_size",
           "allreduce_loss"]
