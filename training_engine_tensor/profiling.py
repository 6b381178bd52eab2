"""``training_engine_tensor.profiling``: the event-segment step profiler under the reference's module
name (its profiling.py:180-662)."""
from forgetrain_b200.utils.profiler import (  # noqa: F401
    DEEP_PHASE_ACCUM, DEEP_PHASE_BWD, DEEP_PHASE_CE, DEEP_PHASE_DATA, DEEP_PHASE_FWD, DEEP_PHASE_ORDER,
    SEG_ALLGATHER, SEG_GRAD_NORM, SEG_LOSS_ALLREDUCE, SEG_MICROBATCHES, SEG_OPTIMIZER,
    SEG_REDUCE_SCATTER, SEG_STEP_START, StepProfiler, parse_profile_range, profiler_from_config,
    summarize_host_phases, summarize_segments)

from_config = profiler_from_config

__all__ = ["StepProfiler", "from_config", "profiler_from_config", "parse_profile_range",
           "summarize_segments", "summarize_host_phases",
           "SEG_STEP_START", "SEG_MICROBATCHES", "SEG_REDUCE_SCATTER", "SEG_GRAD_NORM", "SEG_OPTIMIZER",
           "SEG_LOSS_ALLREDUCE", "SEG_ALLGATHER", "DEEP_PHASE_DATA", "DEEP_PHASE_FWD", "DEEP_PHASE_CE",
           "DEEP_PHASE_BWD", "DEEP_PHASE_ACCUM", "DEEP_PHASE_ORDER"]
