"""Model specification (geometry + default hyper-parameters) and FLOP accounting.

First two tiers of the configuration plane: a ``model_spec.toml`` file is parsed into an
immutable :class:`ModelSpec`; the third tier (:mod:`forgetrain_b200.engine_config`) holds the
run-time switches. Mirrors the role of the reference's ``model_spec.toml`` -> ``config.py``
constants (exports/train_engine_0.5B/src/training_engine_tensor/config.py:53-202) but as a
value object rather than module globals, so several model shapes can coexist in one process.
"""
from __future__ import annotations

import dataclasses
import json
import math
import os
import tomllib
from dataclasses import dataclass
from pathlib import Path

SPEC_DIR = Path(__file__).resolve().parent / "specs"

BUILTIN_SPECS = {
    "tiny": "tiny.toml",
    "0.5b": "minicpm4_0p5b.toml",
    "minicpm4-0.5b": "minicpm4_0p5b.toml",
    "8b": "minicpm4_8b.toml",
    "minicpm4-8b": "minicpm4_8b.toml",
}


@dataclass(frozen=True)
class ModelSpec:
    name: str = "tiny"
    vocab_size: int = 4096
    hidden_size: int = 256
    num_layers: int = 4
    num_attention_heads: int = 4
    num_query_groups: int = 2
    head_dim: int = 64
    ffn_hidden_size: int = 1024
    seq_length: int = 256
    max_position_embeddings: int = 256
    norm_epsilon: float = 1e-6
    rotary_base: float = 10000.0
    init_method_std: float = 0.02
    tie_embeddings: bool = False
    # muP
    mup_enabled: bool = True
    mup_emb_scale: float = 12.0
    mup_depth_scale: float = 1.4
    mup_base_hidden_size: int = 256
    # training defaults
    micro_batch_size: int = 2
    global_batch_size: int = 4
    grad_accum_steps: int = 0
    lr: float = 1e-3
    min_lr: float = 0.0
    lr_warmup_iters: int = 0
    lr_decay_iters: int = 1_000_000
    lr_wsd_decay_iters: int = 0
    train_iters: int = 1000
    weight_decay: float = 0.1
    adam_beta1: float = 0.9
    adam_beta2: float = 0.95
    adam_eps: float = 1e-8
    clip_grad: float = 1.0
    # parallel defaults
    tensor_model_parallel_size: int = 1
    sequence_parallel: bool = False
    use_distributed_optimizer: bool = True

    # ---- derived geometry -------------------------------------------------------------
    @property
    def q_dim(self) -> int:
        return self.num_attention_heads * self.head_dim

    @property
    def kv_dim(self) -> int:
        return self.num_query_groups * self.head_dim

    @property
    def qkv_dim(self) -> int:
        return self.q_dim + 2 * self.kv_dim

    @property
    def heads_per_group(self) -> int:
        return self.num_attention_heads // self.num_query_groups

    # ---- muP helpers (reference: config.py:69-86) ---------------------------------------
    @property
    def mup_width_scale(self) -> float:
        """Logit divisor and hidden-matrix LR divisor: hidden / base width."""
        return self.hidden_size / self.mup_base_hidden_size if self.mup_enabled else 1.0

    @property
    def mup_residual_scale(self) -> float:
        """Multiplier of every residual branch: depth_scale / sqrt(num_layers)."""
        if not self.mup_enabled:
            return 1.0
        return self.mup_depth_scale / math.sqrt(self.num_layers)

    @property
    def emb_scale(self) -> float:
        return self.mup_emb_scale if self.mup_enabled else 1.0

    def replace(self, **kw) -> "ModelSpec":
        return dataclasses.replace(self, **kw)

    def num_parameters(self, include_mtp_layers: int = 0) -> int:
        h = self.hidden_size
        per_layer = 2 * h + self.qkv_dim * h + h * self.q_dim + 3 * self.ffn_hidden_size * h
        n = self.vocab_size * h * (1 if self.tie_embeddings else 2) + self.num_layers * per_layer + h
        n += include_mtp_layers * (per_layer + 2 * h + 2 * h * h)   # + enorm, hnorm, eh_proj
        return n

    def to_json(self) -> str:
        return json.dumps(dataclasses.asdict(self), sort_keys=True)


def _flatten_spec_toml(doc: dict) -> dict:
    out: dict = {}
    m = doc.get("model", {})
    out.update(m)
    mup = doc.get("mup", {})
    if mup:
        out["mup_enabled"] = bool(mup.get("enabled", True))
        for k_src, k_dst in (("emb_scale", "mup_emb_scale"), ("depth_scale", "mup_depth_scale"),
                             ("base_hidden_size", "mup_base_hidden_size")):
            if k_src in mup:
                out[k_dst] = mup[k_src]
    out.update(doc.get("training", {}))
    out.update(doc.get("parallel", {}))
    return out


def load_model_spec(name_or_path: str | os.PathLike = "tiny", **overrides) -> ModelSpec:
    """Load a built-in spec by name (``tiny``, ``0.5b``, ``8b``) or a ``model_spec.toml`` path."""
    key = str(name_or_path).lower()
    path = SPEC_DIR / BUILTIN_SPECS[key] if key in BUILTIN_SPECS else Path(name_or_path)
    if not path.is_file():
        raise FileNotFoundError(f"model {str(name_or_path)!r} is neither a built-in spec "
                                f"({', '.join(sorted(BUILTIN_SPECS))}) nor a model_spec.toml file")
    with open(path, "rb") as f:
        doc = tomllib.load(f)
    fields = {f.name for f in dataclasses.fields(ModelSpec)}
    flat = {k: v for k, v in _flatten_spec_toml(doc).items() if k in fields}
    flat.update({k: v for k, v in overrides.items() if v is not None})
    spec = ModelSpec(**flat)
    validate_spec(spec)
    return spec


def validate_spec(spec: ModelSpec) -> None:
    if spec.num_attention_heads % spec.num_query_groups:
        raise ValueError("num_attention_heads must be a multiple of num_query_groups")
    if spec.head_dim not in (64, 128) and spec.head_dim % 8:
        raise ValueError("head_dim must be a multiple of 8")
    if spec.hidden_size % 8 or spec.ffn_hidden_size % 8:
        raise ValueError("hidden and ffn sizes must be multiples of 8")


# -----------------------------------------------------------------------------------------
# FLOP accounting (reference: config.py:127-202). Forward FLOPs per token = sum of the GEMMs
# + the attention core; x3 for forward + backward.
# -----------------------------------------------------------------------------------------
def forward_flops_per_token(spec: ModelSpec, seq_len: int, causal: bool, mtp_layers: int = 0) -> float:
    h = spec.hidden_size
    per_layer = 2 * h * spec.qkv_dim + 2 * spec.q_dim * h + 2 * h * 2 * spec.ffn_hidden_size \
        + 2 * spec.ffn_hidden_size * h
    attn = (2 if causal else 4) * seq_len * spec.q_dim
    layer = per_layer + attn
    head = 2 * h * spec.vocab_size
    total = spec.num_layers * layer + head
    total += mtp_layers * (layer + 2 * (2 * h) * h + head)
    return float(total)


def compute_training_flops(spec: ModelSpec, tokens: int, seq_len: int, mtp_layers: int = 0) -> float:
    """'Hardware' FLOPs of one fwd+bwd over ``tokens`` tokens (no causal halving)."""
    return 3.0 * tokens * forward_flops_per_token(spec, seq_len, causal=False, mtp_layers=mtp_layers)


def compute_training_flops_standard(spec: ModelSpec, tokens: int, seq_len: int,
                                    mtp_layers: int = 0) -> float:
    """'Standard' FLOPs: the attention core counted causal-halved."""
    return 3.0 * tokens * forward_flops_per_token(spec, seq_len, causal=True, mtp_layers=mtp_layers)


def peak_tflops(default: float = 2250.0) -> float:
    """bf16 dense peak used as the MFU denominator.

    Order: ``FT_PEAK_TFLOPS`` env, the sustained figure of a ``MEASURED_PEAKS.json`` found in
    the working directory, else the nominal B200 figure.
    """
    env = os.environ.get("FT_PEAK_TFLOPS")
    if env:
        return float(env)
    for cand in (Path.cwd() / "MEASURED_PEAKS.json",
                 Path(__file__).resolve().parent.parent / "MEASURED_PEAKS.json"):
        if cand.exists():
            try:
                doc = json.loads(cand.read_text())
                return float(doc.get("bf16_tflops_sustained") or doc.get("bf16_tflops") or default)
            except Exception:
                pass
    return default
