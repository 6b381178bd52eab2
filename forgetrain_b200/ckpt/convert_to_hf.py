#!/usr/bin/env python
"""Export a ``training_state.pt`` checkpoint to a HuggingFace ``MiniCPMForCausalLM`` folder.

    python -m forgetrain_b200.ckpt.convert_to_hf --checkpoint <step dir | training_state.pt> \\
        --output <dir> [--model 0.5b] [--dtype bfloat16]

``--checkpoint`` may also be a step directory of a tensor-parallel run (``rank_<R>.pt`` files):
the shards are merged back into full tensors first. Writes ``model.safetensors`` and ``config.json``. The fused projection weights are taken apart:
``attention.wqkv`` is interleaved per KV group as ``[q_0..q_{g-1} | k | v]`` and becomes
``q_proj / k_proj / v_proj``; ``feed_forward.wfc1`` is ``[gate ; up]``. ``tie_word_embeddings``
is decided by comparing the two tables. Same mapping as the reference's export script
(exports/train_engine_0.5B/scripts/convert_to_hf.py:58-227).
"""
from __future__ import annotations

import argparse
import json
from pathlib import Path

import torch

from ..config import ModelSpec, load_model_spec
from .checkpoint import load_resume_checkpoint


def split_qkv_interleaved(wqkv: torch.Tensor, spec: ModelSpec):
    G, g, D, H = spec.num_query_groups, spec.heads_per_group, spec.head_dim, spec.hidden_size
    grouped = wqkv.view(G, (g + 2) * D, H)
    q = grouped[:, :g * D].reshape(G * g * D, H)
    k = grouped[:, g * D:(g + 1) * D].reshape(G * D, H)
    v = grouped[:, (g + 1) * D:].reshape(G * D, H)
    return q.contiguous(), k.contiguous(), v.contiguous()


def merge_qkv_interleaved(q, k, v, spec: ModelSpec) -> torch.Tensor:
    """Inverse of :func:`split_qkv_interleaved` (used to import HF weights and by the tests)."""
    G, g, D, H = spec.num_query_groups, spec.heads_per_group, spec.head_dim, spec.hidden_size
    return torch.cat([q.view(G, g * D, H), k.view(G, D, H), v.view(G, D, H)], dim=1).reshape(-1, H)


def to_hf_state_dict(params: dict[str, torch.Tensor], spec: ModelSpec, dtype=torch.bfloat16):
    out: dict[str, torch.Tensor] = {}
    cast = lambda t: t.to(dtype).contiguous()
    out["model.embed_tokens.weight"] = cast(params["tok_embeddings.weight"])
    for i in range(spec.num_layers):
        p, hp = f"layers.{i}", f"model.layers.{i}"
        out[f"{hp}.input_layernorm.weight"] = cast(params[f"{p}.attention_norm.weight"])
        out[f"{hp}.post_attention_layernorm.weight"] = cast(params[f"{p}.ffn_norm.weight"])
        q, k, v = split_qkv_interleaved(params[f"{p}.attention.wqkv.weight"], spec)
        out[f"{hp}.self_attn.q_proj.weight"] = cast(q)
        out[f"{hp}.self_attn.k_proj.weight"] = cast(k)
        out[f"{hp}.self_attn.v_proj.weight"] = cast(v)
        out[f"{hp}.self_attn.o_proj.weight"] = cast(params[f"{p}.attention.wo.weight"])
        gate, up = params[f"{p}.feed_forward.wfc1.weight"].chunk(2, dim=0)
        out[f"{hp}.mlp.gate_proj.weight"] = cast(gate)
        out[f"{hp}.mlp.up_proj.weight"] = cast(up)
        out[f"{hp}.mlp.down_proj.weight"] = cast(params[f"{p}.feed_forward.w2.weight"])
    out["model.norm.weight"] = cast(params["norm.weight"])
    head = params.get("output.weight", params["tok_embeddings.weight"])
    tied = head.shape == params["tok_embeddings.weight"].shape and \
        torch.equal(head, params["tok_embeddings.weight"])
    # always written, from the trained head, so that any drift between the two tables during
    # training is kept (the reference script does the same, scripts/convert_to_hf.py:114-117)
    out["lm_head.weight"] = cast(head).clone() if tied else cast(head)   # own storage in the file
    return out, tied


def hf_config(spec: ModelSpec, tied: bool, dtype: str = "bfloat16") -> dict:
    return {
        "architectures": ["MiniCPMForCausalLM"],
        # resolved by from_pretrained(trust_remote_code=True) against the MiniCPM modeling files
        "auto_map": {
            "AutoConfig": "configuration_minicpm.MiniCPMConfig",
            "AutoModel": "modeling_minicpm.MiniCPMModel",
            "AutoModelForCausalLM": "modeling_minicpm.MiniCPMForCausalLM",
        },
        "model_type": "minicpm",
        "initializer_range": 0.1,
        "vocab_size": spec.vocab_size,
        "hidden_size": spec.hidden_size,
        "intermediate_size": spec.ffn_hidden_size,
        "num_hidden_layers": spec.num_layers,
        "num_attention_heads": spec.num_attention_heads,
        "num_key_value_heads": spec.num_query_groups,
        "head_dim": spec.head_dim,
        "hidden_act": "silu",
        "max_position_embeddings": spec.max_position_embeddings,
        "rms_norm_eps": spec.norm_epsilon,
        "rope_theta": spec.rotary_base,
        "scale_emb": spec.mup_emb_scale if spec.mup_enabled else 1.0,
        "dim_model_base": spec.mup_base_hidden_size if spec.mup_enabled else spec.hidden_size,
        "scale_depth": spec.mup_depth_scale if spec.mup_enabled else (spec.num_layers ** 0.5),
        "tie_word_embeddings": bool(tied),
        "torch_dtype": dtype,
        "use_cache": True,
        "bos_token_id": 1,
        "eos_token_id": [2, 73440] if spec.vocab_size > 73440 else 2,
    }


def convert(checkpoint: str, output: str, model: str = "0.5b", dtype: str = "bfloat16") -> Path:
    from safetensors.torch import save_file
    ranks = sorted(Path(checkpoint).glob("rank_*.pt"), key=lambda q: int(q.stem.split("_")[1])) \
        if Path(checkpoint).is_dir() else []
    if ranks:
        # tensor-parallel run: one parameter shard per TP rank, merged back into full tensors
        from ..models.params import merge_tp_shards
        shards = [torch.load(q, map_location="cpu", weights_only=False) for q in ranks]
        if len(shards) != int(shards[0].get("tp_size", len(shards))):
            raise ValueError(f"{checkpoint}: found {len(shards)} rank files for tp_size "
                             f"{shards[0].get('tp_size')}")
        tied = "output.weight" not in shards[0]["params"]
        # the full vocabulary size: stored with the shards, else the sum of the shard rows
        # (which includes the padding of the vocabulary split, cut off again by the merge)
        vocab = int(shards[0].get("vocab_size") or 0) or None
        kw = {"vocab_size": vocab} if vocab else {}
        spec = load_model_spec(model, tie_embeddings=tied, **kw)
        params = merge_tp_shards(spec, [sh["params"] for sh in shards])
    else:
        state = load_resume_checkpoint(checkpoint)
        params = state["params"]
        spec = load_model_spec(model, vocab_size=params["tok_embeddings.weight"].shape[0],
                               tie_embeddings="output.weight" not in params)
    sd, tied = to_hf_state_dict(params, spec, getattr(torch, dtype))
    out = Path(output)
    out.mkdir(parents=True, exist_ok=True)
    save_file(sd, str(out / "model.safetensors"), metadata={"format": "pt"})
    (out / "config.json").write_text(json.dumps(hf_config(spec, tied, dtype), indent=2))
    return out


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawTextHelpFormatter)
    ap.add_argument("--checkpoint", "--input", dest="checkpoint", required=True,
                    help="step directory, training_state.pt, or a directory of rank_<R>.pt shards")
    ap.add_argument("--output", required=True)
    ap.add_argument("--model", default="0.5b")
    ap.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float16", "float32"])
    a = ap.parse_args(argv)
    out = convert(a.checkpoint, a.output, a.model, a.dtype)
    print(f"wrote {out / 'model.safetensors'} and {out / 'config.json'}")
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
