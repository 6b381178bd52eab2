"""``training_engine_tensor.nccl``: process groups, bucket layout and the gradient reducer under the
reference's module name (0.5B nccl.py:39-55, 8B nccl.py:17-22)."""
from forgetrain_b200.parallel.buckets import Bucket, compute_grad_buckets  # noqa: F401
from forgetrain_b200.parallel.dp import BucketedGradReducer  # noqa: F401
from forgetrain_b200.parallel.topology import Topology, init_topology, node_layout, shutdown  # noqa: F401

__all__ = ["Bucket", "compute_grad_buckets", "BucketedGradReducer", "Topology", "init_topology",
           "node_layout", "shutdown"]
