"""Import of Megatron-exported state: ``canonical_state_fp32.pt`` (parameters) and
``canonical_optimizer_state_fp32.pt`` (fp32 master weights and Adam moments).

A checkpoint root that holds ``canonical_state_fp32.pt`` is what the ``train`` sub-command's
``--checkpoint-root`` points at. The file is a flat ``{megatron_key: fp32 tensor}`` dict; both
key layouts in circulation are accepted:

* unfused: the two RMSNorm gains of a block are their own entries
  (``decoder.layers.N.input_layernorm.weight``, ``...pre_mlp_layernorm.weight``);
* fused mcore: they are attributes of the linear that follows
  (``...self_attention.linear_qkv.layer_norm_weight``, ``...mlp.linear_fc1.layer_norm_weight``).

The MTP head (one EAGLE-style layer, keys ``mtp.*`` without a layer index) is mapped when
present; when the run has MTP layers and the checkpoint has none, they are cold-started (norms
one, matrices N(0, 0.02)) and the fact is reported, never silent. The vocabulary size of the
checkpoint must match the model's.

Behavioural counterpart of the reference's ``load_megatron_checkpoint`` /
``load_megatron_optimizer_state`` (exports/train_engine_0.5B/src/training_engine_tensor/
parameters.py:35-50, 121-170, 265-421) and of the fused key names of the 8B engine
(exports/train_engine_8b/src/training_engine_tensor/parameters.py:1-24, 88-95).
"""
from __future__ import annotations

import os
from pathlib import Path

import torch

from ..config import ModelSpec
from ..models.params import all_param_specs, mtp_layer_prefix

PARAMS_FILE = "canonical_state_fp32.pt"
OPTIM_FILE = "canonical_optimizer_state_fp32.pt"


def is_megatron_root(path: str | os.PathLike) -> bool:
    return (Path(path) / PARAMS_FILE).is_file()


def megatron_name_map(num_layers: int, mtp_num_layers: int = 0) -> dict[str, str]:
    """Megatron key -> name used here. Several Megatron keys may map to one name (the two norm
    layouts); a checkpoint contains one of them."""
    m = {
        "embedding.word_embeddings.weight": "tok_embeddings.weight",
        "output_layer.weight": "output.weight",
        "decoder.final_layernorm.weight": "norm.weight",
    }
    for i in range(num_layers):
        mg, ours = f"decoder.layers.{i}", f"layers.{i}"
        m.update({
            f"{mg}.input_layernorm.weight": f"{ours}.attention_norm.weight",
            f"{mg}.self_attention.linear_qkv.layer_norm_weight": f"{ours}.attention_norm.weight",
            f"{mg}.self_attention.linear_qkv.weight": f"{ours}.attention.wqkv.weight",
            f"{mg}.self_attention.linear_proj.weight": f"{ours}.attention.wo.weight",
            f"{mg}.pre_mlp_layernorm.weight": f"{ours}.ffn_norm.weight",
            f"{mg}.mlp.linear_fc1.layer_norm_weight": f"{ours}.ffn_norm.weight",
            f"{mg}.mlp.linear_fc1.weight": f"{ours}.feed_forward.wfc1.weight",
            f"{mg}.mlp.linear_fc2.weight": f"{ours}.feed_forward.w2.weight",
        })
    if mtp_num_layers > 0:        # the exported head has exactly one layer, without an index
        ours = mtp_layer_prefix(0)
        m.update({
            "mtp.emb_input_layernorm.weight": f"{ours}.enorm.weight",
            "mtp.hidden_input_layernorm.weight": f"{ours}.hnorm.weight",
            "mtp.eagle_fc.weight": f"{ours}.eh_proj.weight",
            "mtp.layers.self_attention.linear_qkv.layer_norm_weight": f"{ours}.attention_norm.weight",
            "mtp.layers.self_attention.linear_qkv.weight": f"{ours}.attention.wqkv.weight",
            "mtp.layers.self_attention.linear_proj.weight": f"{ours}.attention.wo.weight",
            "mtp.layers.mlp.linear_fc1.layer_norm_weight": f"{ours}.ffn_norm.weight",
            "mtp.layers.mlp.linear_fc1.weight": f"{ours}.feed_forward.wfc1.weight",
            "mtp.layers.mlp.linear_fc2.weight": f"{ours}.feed_forward.w2.weight",
        })
    return m


def load_megatron_checkpoint(root: str | os.PathLike, spec: ModelSpec, mtp_num_layers: int = 0,
                             dtype: torch.dtype = torch.float32, seed: int = 1234,
                             log=print) -> dict[str, torch.Tensor]:
    """Full (unsharded) parameter tensors by our names, in ``dtype``, on the CPU."""
    path = Path(root) / PARAMS_FILE
    if not path.is_file():
        raise FileNotFoundError(f"no checkpoint at {path}")
    ckpt = torch.load(path, map_location="cpu", weights_only=False)
    if not isinstance(ckpt, dict):
        raise ValueError(f"{path} is not a dict (got {type(ckpt).__name__})")
    specs = {ps.name: ps for ps in all_param_specs(spec, mtp_num_layers)}
    out: dict[str, torch.Tensor] = {}
    for key, ours in megatron_name_map(spec.num_layers, mtp_num_layers).items():
        w = ckpt.get(key)
        if not isinstance(w, torch.Tensor) or ours not in specs:
            continue
        if tuple(w.shape) != tuple(specs[ours].shape):
            if ours in ("tok_embeddings.weight", "output.weight") and w.dim() == 2:
                raise ValueError(f"checkpoint vocab_size ({w.shape[0]}) != model vocab_size "
                                 f"({spec.vocab_size})")
            raise ValueError(f"{key}: shape {tuple(w.shape)} != expected {tuple(specs[ours].shape)}")
        out[ours] = w.to(dtype)
    if spec.tie_embeddings:
        out.pop("output.weight", None)
    missing = [n for n in specs if n not in out]
    cold = [n for n in missing if n.startswith("mtp.")]
    if cold:
        g = torch.Generator().manual_seed(seed)
        for n in cold:
            ps = specs[n]
            out[n] = (torch.ones(ps.shape) if ps.is_norm
                      else torch.randn(ps.shape, generator=g) * 0.02).to(dtype)
        log(f"  [megatron import] MTP weights NOT in checkpoint: cold-initialised {len(cold)} "
            f"tensors (first {cold[0]!r})")
    hard = [n for n in missing if not n.startswith("mtp.")]
    if hard:
        raise KeyError(f"{path}: {len(hard)} parameters missing, first {hard[0]!r}")
    log(f"  [megatron import] loaded {len(out)} parameters from {path}")
    return out


def load_megatron_optimizer_state(root: str | os.PathLike, log=print) -> dict | None:
    """``{"master_weights", "exp_avg", "exp_avg_sq"}`` (dicts of fp32 tensors by OUR names when
    the file uses them, else by Megatron keys mapped through :func:`megatron_name_map` by the
    caller), ``step_count`` and ``num_samples`` (0 when the file says unknown). ``None`` when
    the file is absent: the caller starts a fresh optimizer."""
    path = Path(root) / OPTIM_FILE
    if not path.is_file():
        return None
    payload = torch.load(path, map_location="cpu", weights_only=False)
    if not isinstance(payload, dict):
        raise ValueError(f"{path} is not a dict (got {type(payload).__name__})")
    need = {"master_weights", "exp_avg", "exp_avg_sq", "step_count"}
    lack = need - set(payload)
    if lack:
        raise ValueError(f"{path} misses required keys {sorted(lack)}")
    out = {k: {n: t.to(torch.float32).contiguous() for n, t in payload[k].items()}
           for k in ("master_weights", "exp_avg", "exp_avg_sq")}
    out["step_count"] = int(payload["step_count"])
    out["num_samples"] = max(0, int(payload.get("num_samples", -1)))
    log(f"  [megatron import] optimizer state step_count={out['step_count']} "
        f"num_samples={out['num_samples']} tensors={len(out['master_weights'])} <- {path}")
    return out


def rename_state(state: dict[str, torch.Tensor], num_layers: int, mtp_num_layers: int = 0
                 ) -> dict[str, torch.Tensor]:
    """Keys of an optimizer-state dict translated to our names (already-ours keys pass)."""
    m = megatron_name_map(num_layers, mtp_num_layers)
    return {m.get(k, k): v for k, v in state.items()}
