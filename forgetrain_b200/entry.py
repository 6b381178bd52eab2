"""Gate entry points: one forward, or one forward + backward, from a checkpoint on a given batch.

The reference exposes these so that an outside harness can compare the engine tensor by tensor with
another implementation fed the same weights and the same batch (8B entry.py:47-123):

* :func:`run_forward` returns the scalar loss and the per-token losses;
* :func:`run_forward_backward` returns the loss and the clipped fp32 gradients keyed by the
  Megatron parameter names;
* the full loop is :func:`forgetrain_b200.trainer.run_training_loop`.

``checkpoint_root`` is a Megatron export (``canonical_state_fp32.pt``) or a checkpoint of this engine.
Single process; ``device`` chooses the native CUDA path (bf16) or the CPU statement (fp32).
"""
from __future__ import annotations

import torch

from .ckpt import checkpoint as ckpt
from .ckpt import megatron_import as mg
from .config import ModelSpec, load_model_spec
from .models.minicpm4 import MiniCPM4
from .models.params import ParamStore


def _build(checkpoint_root, device, model, spec: ModelSpec | None, seq_len: int):
    dev = torch.device(device)
    dtype = torch.bfloat16 if dev.type == "cuda" else torch.float32
    quiet = lambda *_: None
    if mg.is_megatron_root(checkpoint_root):
        spec = spec or load_model_spec(model)
        tensors = mg.load_megatron_checkpoint(checkpoint_root, spec, 0, log=quiet)
    else:
        state = ckpt.load_resume_checkpoint(checkpoint_root)
        tensors = state["params"]
        spec = spec or load_model_spec(model, vocab_size=tensors["tok_embeddings.weight"].shape[0],
                                       tie_embeddings="output.weight" not in tensors)
    store = ParamStore(spec, dev, dtype)
    store.load_named(tensors, full_tensors=True)
    return spec, store, MiniCPM4(spec, store, max_seq_len=max(seq_len, spec.seq_length))


def _batch_on(batch: dict, dev: torch.device):
    tok = batch["tokens"].to(dev).long()
    lab = batch["labels"].to(dev).long()
    mask = batch.get("loss_mask")
    mask = torch.ones(tok.shape, device=dev) if mask is None else mask.to(dev).float()
    pos = batch.get("position_ids")
    return tok, lab, mask, (None if pos is None else pos.to(dev).to(torch.int32))


def run_forward(checkpoint_root, batch: dict, device: str = "cpu", model: str = "8b",
                spec: ModelSpec | None = None) -> tuple[float, torch.Tensor]:
    """``(loss, per_token_losses[B, S])``: masked mean of the per-token cross-entropy (fp32)."""
    spec, store, m = _build(checkpoint_root, device, model, spec, batch["tokens"].shape[1])
    tok, lab, mask, pos = _batch_on(batch, store.device)
    with torch.no_grad():
        logits = m.forward(tok, pos)
        per_tok = torch.nn.functional.cross_entropy(logits.float(), lab.reshape(-1),
                                                    reduction="none").view(tok.shape)
    m._saved = []
    loss = float((per_tok * mask).sum() / mask.sum().clamp_min(1.0))
    return loss, per_tok.float().cpu()


def megatron_grad_names(num_layers: int, fused_norm_keys: bool = True) -> dict[str, str]:
    """Name used here -> Megatron key, for one of the two norm-key layouts (``fused_norm_keys``:
    ``linear_qkv.layer_norm_weight`` / ``linear_fc1.layer_norm_weight`` as Megatron-core's fused
    layers name them, else ``input_layernorm`` / ``pre_mlp_layernorm``)."""
    out: dict[str, str] = {}
    for key, ours in mg.megatron_name_map(num_layers, 0).items():
        fused_key = key.endswith("layer_norm_weight")
        unfused_key = key.endswith("input_layernorm.weight") or key.endswith("pre_mlp_layernorm.weight")
        if (fused_key and not fused_norm_keys) or (unfused_key and fused_norm_keys):
            continue
        out[ours] = key
    return out


def run_forward_backward(checkpoint_root, batch: dict, device: str = "cpu", model: str = "8b",
                         spec: ModelSpec | None = None, clip_grad: float = 1.0,
                         fused_norm_keys: bool = True) -> tuple[float, dict[str, torch.Tensor]]:
    """``(loss, {megatron parameter name: fp32 gradient})`` after global-norm clipping with
    ``clip = min(1, clip_grad / (norm + 1e-6))`` (``clip_grad <= 0``: no clipping)."""
    spec, store, m = _build(checkpoint_root, device, model, spec, batch["tokens"].shape[1])
    tok, lab, mask, pos = _batch_on(batch, store.device)
    loss = m.forward_backward(tok, lab, mask, 1.0, False, None, pos)
    grads = {ps.name: store.grads[ps.name].detach().float() for ps in store.specs}
    norm = torch.sqrt(sum(g.double().pow(2).sum() for g in grads.values()))
    clip = 1.0 if clip_grad <= 0 else min(1.0, clip_grad / (float(norm) + 1e-6))
    names = megatron_grad_names(spec.num_layers, fused_norm_keys)
    out = {names[n]: (g * clip).cpu() for n, g in grads.items() if n in names}
    return float(loss), out
