"""``training_engine_tensor.profiling``: the event-segment step profiler under the reference's module
name (its profiling.py:207-662)."""
from forgetrain_b200.utils.profiler import (  # noqa: F401
    StepProfiler, parse_profile_range, profiler_from_config)

from_config = profiler_from_config

__all__ = ["StepProfiler", "from_config", "profiler_from_config", "parse_profile_range"]
