"""``training_engine_tensor.data``: host-to-device prefetcher and the synthetic / fixed sources under
the reference's module name (its data.py:37-185)."""
from forgetrain_b200.data.prefetch import DataPrefetcher  # noqa: F401
from forgetrain_b200.data.synthetic import SyntheticTokenSource  # noqa: F401
from forgetrain_b200.data.tokenized import FixedBatchSource  # noqa: F401

__all__ = ["DataPrefetcher", "SyntheticTokenSource", "FixedBatchSource"]
