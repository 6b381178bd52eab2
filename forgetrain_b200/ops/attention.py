"""Causal GQA FlashAttention on the tcgen05 kernels (``csrc/attn_fwd_sm100.cu``,
``csrc/attn_bwd_sm100.cu``), operating directly on the interleaved QKV projection buffer.

Counterpart of the reference's ``attention_fwd`` / ``attention_bwd`` entry points
(exports/train_engine_0.5B/src/training_engine_tensor/ops/attention/kernel.py:298-470).
"""
from __future__ import annotations

import math

import torch

from . import _lib

c_int, c_float = _lib.c_int, _lib.c_float
P = _lib.ptr


def attention_fwd(qkv: torch.Tensor, batch: int, n_groups: int, heads_per_group: int,
                  head_dim: int, scale: float | None = None):
    """Returns ``(out[T, Hq*D] bf16, lse[B, Hq, S] fp32)``."""
    T = qkv.shape[0]
    S = T // batch
    Hq = n_groups * heads_per_group
    scale = 1.0 / math.sqrt(head_dim) if scale is None else scale
    if qkv.dtype != torch.bfloat16 or qkv.stride(1) != 1:
        raise ValueError("attention_fwd: qkv must be bf16 with a contiguous last dimension")
    if S % 256 or head_dim not in (64, 128):
        raise ValueError(f"attention_fwd: needs seq % 256 == 0 and head_dim in (64, 128); got "
                         f"seq={S} head_dim={head_dim}")
    out = torch.empty(T, Hq * head_dim, dtype=torch.bfloat16, device=qkv.device)
    lse = torch.empty(batch, Hq, S, dtype=torch.float32, device=qkv.device)
    rc = _lib.lib().ft_attn_fwd(P(qkv), P(out), P(lse), c_int(batch), c_int(S), c_int(n_groups),
                                c_int(heads_per_group), c_int(head_dim), c_int(qkv.stride(0)),
                                c_int(out.stride(0)), c_float(scale),
                                P(_lib.status_word(qkv.device)), _lib.stream())
    _lib.check_rc(rc, "ft_attn_fwd")
    return out, lse


def attention_bwd(dout: torch.Tensor, qkv: torch.Tensor, out: torch.Tensor, lse: torch.Tensor,
                  batch: int, n_groups: int, heads_per_group: int, head_dim: int,
                  scale: float | None = None, heads_per_cta: int = 0,
                  rope: tuple | None = None) -> torch.Tensor:
    """Gradient wrt the interleaved qkv buffer (bf16, same layout as ``qkv``). ``rope`` =
    ``(cos, sin, position_ids or None)``: the gradient of the q and k heads comes back with the
    backward of the rotary embedding applied (fused into the kernel that converts the fp32
    accumulator), i.e. it is the gradient wrt the UNROTATED projection output."""
    T = qkv.shape[0]
    S = T // batch
    scale = 1.0 / math.sqrt(head_dim) if scale is None else scale
    L = _lib.lib()
    cos = sin = pos = None
    if rope is not None:
        cos, sin, pos = rope
        if cos.dtype != torch.float32 or cos.shape[1] != head_dim // 2 or cos.shape[0] < S:
            raise ValueError("attention_bwd: rope tables must be fp32 [>= seq][head_dim / 2]")
        if pos is not None:
            pos = pos.reshape(-1).to(torch.int32)
    dqkv = torch.empty_like(qkv)
    Hq = n_groups * heads_per_group
    # fp32 scratch: accumulator laid out like qkv, and [delta | lse*log2(e)] per (b, head, s)
    acc = torch.empty(T, qkv.shape[1], dtype=torch.float32, device=qkv.device)
    delta = torch.empty(2, batch, Hq, S, dtype=torch.float32, device=qkv.device)
    rc = L.ft_attn_bwd(P(dout), P(qkv), P(out), P(lse), P(dqkv), P(acc), P(delta),
                       c_int(batch), c_int(S), c_int(n_groups), c_int(heads_per_group),
                       c_int(head_dim), c_int(qkv.stride(0)), c_int(out.stride(0)),
                       c_int(dout.stride(0)), c_float(scale), c_int(heads_per_cta),
                       P(cos), P(sin), P(pos),
                       P(_lib.status_word(qkv.device)), _lib.stream())
    _lib.check_rc(rc, "ft_attn_bwd")
    return dqkv
