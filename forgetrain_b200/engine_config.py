"""Run-time configuration: one frozen :class:`EngineConfig` installed once per process.

Third tier of the configuration plane (model spec -> constants -> engine switches). Keeps the
field names of the reference's ``EngineConfig``
(exports/train_engine_0.5B/src/training_engine_tensor/engine_config.py:132-277 and
exports/train_engine_8b/src/training_engine_tensor/engine_config.py:107-192) for everything
that is a hyper-parameter, a communication knob, a graph switch or a logging/profiling
switch. The reference's per-fusion on/off flags have no counterpart: the fused sm_100a
kernels are the only GPU path.
"""
from __future__ import annotations

import dataclasses
import os
from dataclasses import dataclass
from typing import Any, Callable

# Environment variables that come from the launcher / libraries, not from this package.
EXTERNAL_ENV_WHITELIST = frozenset({
    "RANK", "LOCAL_RANK", "WORLD_SIZE", "MASTER_ADDR", "MASTER_PORT", "LOCAL_WORLD_SIZE",
    "CUDA_VISIBLE_DEVICES", "CUDA_DEVICE_MAX_CONNECTIONS", "NCCL_DEBUG", "NCCL_ALGO",
    "NCCL_PROTO", "NCCL_MIN_NCHANNELS", "NCCL_NVLS_ENABLE", "NCCL_IB_QPS",
    "TORCH_NCCL_HEARTBEAT_TIMEOUT_SEC", "OUTPUT_DIR", "HF_HOME", "TOKENIZERS_PARALLELISM",
    "FT_PEAK_TFLOPS", "FT_B200_NO_AUTOBUILD", "FT_COMM_MULTIMEM", "FT_COMM_TIMEOUT_MS",
    "FT_COMM_CTAS", "FT_B200_LIB", "FT_FUSE_ADAM_AG", "FT_FUSE_FC1_SWIGLU", "FT_INJECT_FAILURE",
})


@dataclass(frozen=True)
class EngineConfig:
    # ---- precision / debug ----
    dtype: str = "bf16"                  # compute dtype: bf16 (GPU) or fp32 (CPU plumbing runs)
    no_grad_clip: bool = False
    grad_diag: bool = False              # accepted; the reference declares it and never reads it either
    grad_norm_diag: bool = False
    emit_loss_lines: bool = False
    serial_streams: bool = False         # force every side stream onto the main stream
    # ---- communication ----
    comm: str = "fused"                  # "fused": peer-memory kernels; "nccl": library baseline
    wgrad_overlap: bool = True           # reduce buckets while backward is still running
    wgrad_side_stream: bool = True       # decoder weight-gradient GEMMs on a stream of their own
    wgrad_bucket_target_elems: int = 100 * 1024 * 1024
    opt_allgather_overlap: bool = True
    async_loss_ar: bool = True           # accepted; the loss all-reduce never blocks the host here
    sharded_optimizer: bool = True       # ZeRO-1; False: all-reduced grads, full Adam state per rank
    data_prefetch_depth: int = 2
    rs_buckets: int = 32                 # 8B-style: number of layer-aligned buckets (0 = by size)
    tensor_parallel_size: int = 1
    sequence_parallel: bool = True
    # ---- activation recomputation (memory for time) ----
    recompute_attn: bool = False         # attention output / log-sum-exp rebuilt in backward
    recompute_mlp: bool = False          # FC1 output and SwiGLU activation rebuilt in backward
    mask_vocab_padding: bool = False     # TP: keep the vocabulary's pad columns out of the softmax
    # ---- CUDA graphs ----
    forward_cuda_graph: bool = False
    step_cuda_graph: bool = False
    full_step_cuda_graph: bool = False   # micro-batches + norm + clip + AdamW in ONE graph
    step_cuda_graph_warmup: int = 3
    step_cuda_graph_tol: float = 1e-3
    step_cuda_graph_sanity: bool = False
    # ---- muP ----
    mup_emb_scale: float = 12.0
    mup_depth_scale: float = 1.4
    # ---- MTP ----
    mtp_num_layers: int = 0
    mtp_loss_scaling_factor: float = 0.1
    # ---- LR schedule (WSD) ----
    max_lr: float = 3e-4
    min_lr: float = 0.0
    warmup_iters: int = 2000
    lr_decay_iters: int = 240000
    wsd_decay_iters: int = 3000
    # ---- AdamW ----
    adam_beta1: float = 0.9
    adam_beta2: float = 0.95
    adam_eps: float = 1e-8
    weight_decay: float = 0.1
    max_grad_norm: float = 1.0
    mup_lr_scaling: bool = True          # hidden matrices use lr / (hidden / base width)
    # ---- init ----
    random_init: bool = True
    # "spec": muP-aware std from the model spec; "normal": N(0, init_std); "mcore": N(0, init_std)
    # with the residual-stream projections at init_std / sqrt(2 * layers) (the 8B engine's)
    init_scheme: str = "spec"
    init_std: float = 0.02
    # ---- profiling ----
    profile_range: str = ""              # "start,end" (step indices, end exclusive)
    profile_output: str = ""
    profile_deep: bool = False
    host_timer: bool = False

    def replace(self, **kw: Any) -> "EngineConfig":
        return dataclasses.replace(self, **kw)


_BOOL_TRUE = {"1", "true", "yes", "on"}


def _env_bool(env: dict, key: str, default: bool) -> bool:
    v = env.get(key)
    return default if v is None else v.strip().lower() in _BOOL_TRUE


# env name -> (field, parser)
_ENV_MAP: dict[str, tuple[str, Callable[[str], Any]]] = {
    "FT_DTYPE": ("dtype", str),
    "NO_GRAD_CLIP": ("no_grad_clip", lambda v: v.lower() in _BOOL_TRUE),
    "GRAD_DIAG": ("grad_diag", lambda v: v.lower() in _BOOL_TRUE),
    "GRAD_NORM_DIAG": ("grad_norm_diag", lambda v: v.lower() in _BOOL_TRUE),
    "EMIT_LOSS_LINES": ("emit_loss_lines", lambda v: v.lower() in _BOOL_TRUE),
    "SERIAL_STREAMS": ("serial_streams", lambda v: v.lower() in _BOOL_TRUE),
    "FT_COMM": ("comm", str),
    "WGRAD_OVERLAP": ("wgrad_overlap", lambda v: v.lower() in _BOOL_TRUE),
    "WGRAD_SIDE_STREAM": ("wgrad_side_stream", lambda v: v.lower() in _BOOL_TRUE),
    "WGRAD_BUCKET_TARGET_ELEMS": ("wgrad_bucket_target_elems", int),
    "OPT_ALLGATHER_OVERLAP": ("opt_allgather_overlap", lambda v: v.lower() in _BOOL_TRUE),
    "ASYNC_LOSS_AR": ("async_loss_ar", lambda v: v.lower() in _BOOL_TRUE),
    "SHARDED_OPTIMIZER": ("sharded_optimizer", lambda v: v.lower() in _BOOL_TRUE),
    "DATA_PREFETCH_DEPTH": ("data_prefetch_depth", int),
    "RS_BUCKETS": ("rs_buckets", int),
    "TENSOR_PARALLEL_SIZE": ("tensor_parallel_size", int),
    "SEQUENCE_PARALLEL": ("sequence_parallel", lambda v: v.lower() in _BOOL_TRUE),
    "RECOMPUTE_ATTN": ("recompute_attn", lambda v: v.lower() in _BOOL_TRUE),
    "RECOMPUTE_MLP": ("recompute_mlp", lambda v: v.lower() in _BOOL_TRUE),
    "MASK_VOCAB_PADDING": ("mask_vocab_padding", lambda v: v.lower() in _BOOL_TRUE),
    "FORWARD_CUDA_GRAPH": ("forward_cuda_graph", lambda v: v.lower() in _BOOL_TRUE),
    "STEP_CUDA_GRAPH": ("step_cuda_graph", lambda v: v.lower() in _BOOL_TRUE),
    "FULL_STEP_CUDA_GRAPH": ("full_step_cuda_graph", lambda v: v.lower() in _BOOL_TRUE),
    "STEP_CUDA_GRAPH_FULL": ("full_step_cuda_graph", lambda v: v.lower() in _BOOL_TRUE),
    "FP32_MODE": ("dtype", lambda v: "fp32" if v.lower() in _BOOL_TRUE else "bf16"),
    "LR_WARMUP_ITERS": ("warmup_iters", int),
    "LR_WSD_DECAY_ITERS": ("wsd_decay_iters", int),
    "CLIP_GRAD": ("max_grad_norm", float),
    # the reference's whole-step graph has settings of its own; here both graphs share one set
    # (listed before the native names, so those win when both are given)
    "STEP_CUDA_GRAPH_FULL_WARMUP": ("step_cuda_graph_warmup", int),
    "STEP_CUDA_GRAPH_FULL_TOL": ("step_cuda_graph_tol", float),
    "STEP_CUDA_GRAPH_FULL_SANITY": ("step_cuda_graph_sanity", lambda v: v.lower() in _BOOL_TRUE),
    "STEP_CUDA_GRAPH_WARMUP": ("step_cuda_graph_warmup", int),
    "STEP_CUDA_GRAPH_TOL": ("step_cuda_graph_tol", float),
    "STEP_CUDA_GRAPH_SANITY": ("step_cuda_graph_sanity", lambda v: v.lower() in _BOOL_TRUE),
    "MUP_EMB_SCALE": ("mup_emb_scale", float),
    "MUP_DEPTH_SCALE": ("mup_depth_scale", float),
    "MTP_NUM_LAYERS": ("mtp_num_layers", int),
    "MTP_LOSS_SCALING_FACTOR": ("mtp_loss_scaling_factor", float),
    "MAX_LR": ("max_lr", float),
    "MIN_LR": ("min_lr", float),
    "WARMUP_ITERS": ("warmup_iters", int),
    "LR_DECAY_ITERS": ("lr_decay_iters", int),
    "WSD_DECAY_ITERS": ("wsd_decay_iters", int),
    "ADAM_BETA1": ("adam_beta1", float),
    "ADAM_BETA2": ("adam_beta2", float),
    "ADAM_EPS": ("adam_eps", float),
    "WEIGHT_DECAY": ("weight_decay", float),
    "MAX_GRAD_NORM": ("max_grad_norm", float),
    "RANDOM_INIT": ("random_init", lambda v: v.lower() in _BOOL_TRUE),
    "PROFILE_RANGE": ("profile_range", str),
    "PROFILE_OUTPUT": ("profile_output", str),
    "PROFILE_DEEP": ("profile_deep", lambda v: v.lower() in _BOOL_TRUE),
    "HOST_TIMER": ("host_timer", lambda v: v.lower() in _BOOL_TRUE),
}

DECLARED_ENV_VARS = frozenset(_ENV_MAP) | EXTERNAL_ENV_WHITELIST


def from_env(env: dict | None = None, **overrides: Any) -> EngineConfig:
    """Build a config from environment variables (legacy bridge) plus keyword overrides."""
    env = dict(os.environ if env is None else env)
    kw: dict[str, Any] = {}
    for name, (fld, parse) in _ENV_MAP.items():
        if name in env and env[name] != "":
            kw[fld] = parse(env[name])
    kw.update({k: v for k, v in overrides.items() if v is not None})
    cfg = EngineConfig(**kw)
    validate_config(cfg)
    return cfg


# Field names of the reference's two engines that differ from the names here
# (0.5B engine_config.py:141-277, 8B engine_config.py:117-192): old name -> (field, converter).
LEGACY_FIELD_ALIASES: dict[str, tuple[str, Callable[[Any], Any]]] = {
    "lr_warmup_iters": ("warmup_iters", int),
    "lr_wsd_decay_iters": ("wsd_decay_iters", int),
    "clip_grad": ("max_grad_norm", float),
    "step_cuda_graph_full": ("full_step_cuda_graph", bool),
    # the whole-step graph shares the compute-step graph's warm-up / sanity settings here
    "step_cuda_graph_full_warmup": ("step_cuda_graph_warmup", int),
    "step_cuda_graph_full_tol": ("step_cuda_graph_tol", float),
    "step_cuda_graph_full_sanity": ("step_cuda_graph_sanity", bool),
    "fp32_mode": ("dtype", lambda on: "fp32" if on else "bf16"),
}

# Switches of the reference that select between a fused and an unfused code path, a library
# and a custom kernel, or a stream layout. Here the fused kernels are the only path, so the
# names are accepted (a config file written for the reference loads) and have no effect.
LEGACY_NOOP_FIELDS = frozenset({
    "fused_ops", "fuse_ce", "fuse_swiglu", "fuse_rmsnorm_residual", "fuse_rope",
    "fuse_rope_doc_aware", "fuse_adam_sync", "fuse_gemm_pad", "fuse_direct_attn",
    "fuse_inplace_residual", "fuse_index_add_emb_bwd", "use_span_based_attn", "unfused_mode",
    "te_rope", "fp32_allreduce", "fp32_grad_accum", "accum_stream_overlap", "multi_tensor_adam",
    "custom_gemm", "use_fused_norm_bwd", "norm_bwd_nan_diag", "step_cuda_graph_accum",
    "step_cuda_graph_reducer", "step_cuda_graph_nccl_opt", "step_cuda_graph_optimizer",
    "step_cuda_graph_nccl_opt_warmup", "step_cuda_graph_optimizer_warmup",
    "forward_cuda_graph_warmup", "forward_cuda_graph_tol", "forward_cuda_graph_sanity",
    "forward_cuda_graph_sample_stride",
    "fused_rope", "fused_rope_pack", "fused_residual_rmsnorm", "fused_rope_qkv",
    "fused_attn_rmsnorm_bwd", "fused_mlp_residual_rmsnorm", "fused_dw_reduce",
    "fused_rope_fp32cos", "ag_fwd_overlap", "adam_ag_pipeline", "gpu_norm_clip", "fused_ce",
    "defer_wgrad_sync", "fused_swiglu", "dw_reduce_rows_per_block", "direct_attn",
    "dsl_attn_fwd", "rope_bhsd", "padded_vocab_size", "vocab_size",
})


def from_legacy(fields: dict, **overrides: Any) -> tuple[EngineConfig, list[str]]:
    """Build a config from a dict keyed by the reference engines' field names.

    Names that exist here pass through, renamed ones are translated, path selectors that
    have no counterpart are dropped. Returns the config and the list of dropped names so
    the caller can tell the user; an unknown name raises.
    """
    own = {f.name for f in dataclasses.fields(EngineConfig)}
    kw: dict[str, Any] = {}
    dropped: list[str] = []
    for name, value in fields.items():
        if name in own:
            kw[name] = value
        elif name in LEGACY_FIELD_ALIASES:
            fld, conv = LEGACY_FIELD_ALIASES[name]
            kw[fld] = conv(value)
        elif name in LEGACY_NOOP_FIELDS:
            dropped.append(name)
        else:
            raise KeyError(f"unknown engine config field {name!r}")
    kw.update({k: v for k, v in overrides.items() if v is not None})
    cfg = EngineConfig(**kw)
    validate_config(cfg)
    return cfg, sorted(dropped)


def from_spec(spec, **overrides: Any) -> EngineConfig:
    """Defaults taken from a :class:`~forgetrain_b200.config.ModelSpec`'s training section."""
    kw = dict(
        mup_emb_scale=spec.mup_emb_scale if spec.mup_enabled else 0.0,
        mup_depth_scale=spec.mup_depth_scale if spec.mup_enabled else 0.0,
        max_lr=spec.lr, min_lr=spec.min_lr, warmup_iters=spec.lr_warmup_iters,
        lr_decay_iters=spec.lr_decay_iters, wsd_decay_iters=spec.lr_wsd_decay_iters,
        adam_beta1=spec.adam_beta1, adam_beta2=spec.adam_beta2, adam_eps=spec.adam_eps,
        weight_decay=spec.weight_decay, max_grad_norm=spec.clip_grad,
        tensor_parallel_size=spec.tensor_model_parallel_size,
        sequence_parallel=spec.sequence_parallel,
        sharded_optimizer=spec.use_distributed_optimizer,
        init_std=spec.init_method_std,
    )
    kw.update({k: v for k, v in overrides.items() if v is not None})
    cfg = EngineConfig(**kw)
    validate_config(cfg)
    return cfg


def validate_config(cfg: EngineConfig) -> None:
    if cfg.dtype not in ("bf16", "fp32"):
        raise ValueError(f"dtype must be bf16 or fp32, got {cfg.dtype!r}")
    if cfg.comm not in ("fused", "nccl"):
        raise ValueError(f"comm must be 'fused' or 'nccl', got {cfg.comm!r}")
    if cfg.wgrad_bucket_target_elems <= 0:
        raise ValueError("wgrad_bucket_target_elems must be positive")
    if bool(cfg.profile_range) != bool(cfg.profile_output):
        raise ValueError("PROFILE_RANGE and PROFILE_OUTPUT must be given together")
    if cfg.tensor_parallel_size < 1:
        raise ValueError("tensor_parallel_size must be >= 1")
    if not 1 <= cfg.data_prefetch_depth <= 4:
        raise ValueError("data_prefetch_depth must be in 1..4")


# -----------------------------------------------------------------------------------------
# process-wide singleton
# -----------------------------------------------------------------------------------------
_GLOBAL: EngineConfig | None = None
_RESET_HOOKS: list[Callable[[], None]] = []


def set_global_config(cfg: EngineConfig) -> None:
    """Install the process-wide config. Installing twice is an error (reset first)."""
    global _GLOBAL
    if _GLOBAL is not None:
        raise RuntimeError("EngineConfig already installed; call reset_global_config() first")
    _GLOBAL = cfg


def get_config() -> EngineConfig:
    """The installed config, or the defaults when none was installed."""
    return _GLOBAL if _GLOBAL is not None else EngineConfig()


def has_global_config() -> bool:
    return _GLOBAL is not None


def register_reset_hook(fn: Callable[[], None]) -> None:
    """Register a callable run by :func:`reset_global_config` (caches keyed on the config)."""
    _RESET_HOOKS.append(fn)


def reset_global_config() -> None:
    global _GLOBAL
    _GLOBAL = None
    for fn in list(_RESET_HOOKS):
        fn()


def print_config_summary(cfg: EngineConfig, prefix: str = "[CONFIG]") -> str:
    parts = [f"{f.name}={getattr(cfg, f.name)}" for f in dataclasses.fields(cfg)]
    line = f"{prefix} " + " ".join(parts)
    print(line, flush=True)
    return line


# What the package's own switches outside EngineConfig do (kept next to the whitelist so that the
# generated table cannot drift from the code that reads them).
_SWITCH_NOTES = {
    "FT_PEAK_TFLOPS": "peak used for the MFU lines instead of the measured / nominal one",
    "FT_B200_NO_AUTOBUILD": "1: never build the native library on import",
    "FT_B200_LIB": "path of the native library to load instead of the in-tree one",
    "FT_COMM_MULTIMEM": "0: peer loads instead of multimem (NVSwitch) in the fused collectives",
    "FT_COMM_TIMEOUT_MS": "limit (ms, default 30000) of every wait on a peer flag in the fused collectives",
    "FT_COMM_CTAS": "CTAs per fused data-parallel collective launch (default 96)",
    "FT_FUSE_ADAM_AG": "0: AdamW and the parameter all-gather as two kernels instead of one",
    "FT_FUSE_FC1_SWIGLU": "0: FC1 and SwiGLU as two kernels instead of one",
    "FT_INJECT_FAILURE": "recovery tests: `step=K[,rank=R][,once=PATH][,exit=CODE]` makes rank R fail on "
                         "the host right before step K (utils/fault_injection.py)",
}


def env_table_markdown() -> str:
    """The declared environment variables as a markdown document (the counterpart of the
    reference's ENV_WHITELIST.md; ``python -m forgetrain_b200.engine_config`` prints it and
    ``forgetrain_b200/ENV_VARS.md`` is its committed output)."""
    d = EngineConfig()
    lines = ["# Environment variables", "",
             "Generated by `python -m forgetrain_b200.engine_config`; a test keeps this file in step",
             "with the code. Anything else read from the environment fails the whitelist test.", "",
             "## EngineConfig bridge (`engine_config.from_env`; the CLI flag of the same field wins)", "",
             "| variable | field | default |", "|---|---|---|"]
    for name, (fld, _) in _ENV_MAP.items():
        lines.append(f"| `{name}` | `{fld}` | `{getattr(d, fld)!r}` |")
    lines += ["", "## Switches read where they are used", "", "| variable | effect |", "|---|---|"]
    for name in sorted(_SWITCH_NOTES):
        lines.append(f"| `{name}` | {_SWITCH_NOTES[name]} |")
    lines += ["", "## From the launcher and the libraries (read, never set)", "",
              ", ".join(f"`{n}`" for n in sorted(EXTERNAL_ENV_WHITELIST - set(_SWITCH_NOTES))), ""]
    return "\n".join(lines)


if __name__ == "__main__":
    print(env_table_markdown(), end="")
