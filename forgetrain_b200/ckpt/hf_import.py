"""Start a run from a HuggingFace ``MiniCPMForCausalLM`` folder (``model.safetensors`` +
``config.json``): the inverse of :mod:`forgetrain_b200.ckpt.convert_to_hf`. ``q_proj / k_proj /
v_proj`` are interleaved back into the fused per-KV-group rows ``[q_0..q_{g-1} | k | v]``,
``gate_proj / up_proj`` stacked into ``[gate ; up]``, names mapped back. There is no optimizer
state in such a folder: the moments start at zero and the master weights are the loaded
parameters. The reference has the export direction only (scripts/convert_to_hf.py:58-227); the way
back is what lets a published checkpoint be trained further with this engine."""
from __future__ import annotations

import json
from pathlib import Path

import torch

from ..config import ModelSpec
from .convert_to_hf import merge_qkv_interleaved


def is_hf_folder(path) -> bool:
    p = Path(path)
    return p.is_dir() and (p / "model.safetensors").exists() and (p / "config.json").exists()


def check_config(cfg: dict, spec: ModelSpec) -> None:
    """The folder must describe the architecture the run was configured for."""
    want = {"hidden_size": spec.hidden_size, "intermediate_size": spec.ffn_hidden_size,
            "num_hidden_layers": spec.num_layers, "num_attention_heads": spec.num_attention_heads,
            "num_key_value_heads": spec.num_query_groups, "vocab_size": spec.vocab_size}
    bad = {k: (cfg.get(k), v) for k, v in want.items() if k in cfg and cfg[k] != v}
    if "head_dim" in cfg and cfg["head_dim"] != spec.head_dim:
        bad["head_dim"] = (cfg["head_dim"], spec.head_dim)
    if bad:
        raise ValueError("HuggingFace config does not match the model spec (found, expected): "
                         + ", ".join(f"{k}={a}!={b}" for k, (a, b) in sorted(bad.items())))


def from_hf_state_dict(sd: dict[str, torch.Tensor], spec: ModelSpec) -> dict[str, torch.Tensor]:
    """Engine parameter names -> full tensors. ``output.weight`` is produced only for a spec with
    untied tables (from ``lm_head.weight``, else from the embedding)."""
    out: dict[str, torch.Tensor] = {"tok_embeddings.weight": sd["model.embed_tokens.weight"]}
    for i in range(spec.num_layers):
        p, hp = f"layers.{i}", f"model.layers.{i}"
        out[f"{p}.attention_norm.weight"] = sd[f"{hp}.input_layernorm.weight"]
        out[f"{p}.ffn_norm.weight"] = sd[f"{hp}.post_attention_layernorm.weight"]
        out[f"{p}.attention.wqkv.weight"] = merge_qkv_interleaved(
            sd[f"{hp}.self_attn.q_proj.weight"], sd[f"{hp}.self_attn.k_proj.weight"],
            sd[f"{hp}.self_attn.v_proj.weight"], spec)
        out[f"{p}.attention.wo.weight"] = sd[f"{hp}.self_attn.o_proj.weight"]
        out[f"{p}.feed_forward.wfc1.weight"] = torch.cat(
            [sd[f"{hp}.mlp.gate_proj.weight"], sd[f"{hp}.mlp.up_proj.weight"]], dim=0)
        out[f"{p}.feed_forward.w2.weight"] = sd[f"{hp}.mlp.down_proj.weight"]
    out["norm.weight"] = sd["model.norm.weight"]
    if not spec.tie_embeddings:
        out["output.weight"] = sd.get("lm_head.weight", sd["model.embed_tokens.weight"])
    elif "lm_head.weight" in sd and not torch.equal(sd["lm_head.weight"], sd["model.embed_tokens.weight"]):
        raise ValueError("the folder has an output table of its own but the run ties the two tables; "
                         "use --no-tie-embeddings")
    return out


def load_hf_folder(path, spec: ModelSpec) -> dict[str, torch.Tensor]:
    from safetensors.torch import load_file
    p = Path(path)
    check_config(json.loads((p / "config.json").read_text()), spec)
    return from_hf_state_dict(load_file(str(p / "model.safetensors")), spec)
