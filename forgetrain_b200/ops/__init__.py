"""Op layer: one function per op, routed by device.

CUDA tensors always run the hand-written sm_100a kernels of the native library
(:mod:`forgetrain_b200.ops.cuda_ops`); CPU tensors run the plain PyTorch statement of the same
op (:mod:`forgetrain_b200.ops.reference`), which is also the oracle of the kernel tests. There
is no library fallback for CUDA tensors: if the native library cannot be loaded the call
raises.
"""
from __future__ import annotations

import torch

from . import reference as _ref


def _cuda():
    from . import cuda_ops
    return cuda_ops


def _pick(t: torch.Tensor):
    return _cuda() if t.is_cuda else _ref


def embedding_fwd(ids, w, scale, vocab_start: int = 0):
    if w.is_cuda:
        return _cuda().embedding_fwd(ids, w, scale, vocab_start)
    if vocab_start == 0 and int(ids.max()) < w.shape[0]:
        return _ref.embedding_fwd(ids, w, scale)
    flat = ids.reshape(-1) - vocab_start
    ok = (flat >= 0) & (flat < w.shape[0])
    out = torch.zeros(flat.numel(), w.shape[1], dtype=w.dtype)
    out[ok] = (w[flat[ok]].float() * scale).to(w.dtype)
    return out


def embedding_bwd(ids, dy, scale, dw, vocab_start: int = 0):
    return _pick(dy).embedding_bwd(ids, dy, scale, dw, vocab_start)


def add_rmsnorm_fwd(res, x, w, eps, y_out=None):
    return _pick(x).add_rmsnorm_fwd(res, x, w, eps, y_out)


def rmsnorm_bwd(dy, h, w, rstd, dres, dw, accumulate):
    return _pick(dy).rmsnorm_bwd(dy, h, w, rstd, dres, dw, accumulate)


def rope_(qkv, cos, sin, batch, n_groups, heads_per_group, head_dim, inverse=False,
          position_ids=None):
    return _pick(qkv).rope_(qkv, cos, sin, batch, n_groups, heads_per_group, head_dim,
                            inverse=inverse, position_ids=position_ids)


def attention_fwd(qkv, batch, n_groups, heads_per_group, head_dim, scale=None):
    return _pick(qkv).attention_fwd(qkv, batch, n_groups, heads_per_group, head_dim, scale)


def attention_bwd(dout, qkv, out, lse, batch, n_groups, heads_per_group, head_dim, scale=None,
                  rope=None):
    """``rope = (cos, sin, position_ids)``: also apply the backward of the rotary embedding to
    the q / k gradients (fused into the CUDA kernel; a second step on the reference path)."""
    mod = _pick(qkv)
    if rope is None:
        return mod.attention_bwd(dout, qkv, out, lse, batch, n_groups, heads_per_group, head_dim,
                                 scale)
    if mod is _ref:
        d = mod.attention_bwd(dout, qkv, out, lse, batch, n_groups, heads_per_group, head_dim, scale)
        return mod.rope_(d, rope[0], rope[1], batch, n_groups, heads_per_group, head_dim,
                         inverse=True, position_ids=rope[2])
    return mod.attention_bwd(dout, qkv, out, lse, batch, n_groups, heads_per_group, head_dim, scale,
                             rope=rope)


def swiglu_fwd(y1):
    return _pick(y1).swiglu_fwd(y1)


def swiglu_bwd(dact, y1):
    return _pick(y1).swiglu_bwd(dact, y1)


def linear_fwd(x, w, alpha: float = 1.0):
    return _pick(x).linear_fwd(x, w, alpha)


def linear_swiglu_fwd(x, w, alpha: float = 1.0):
    """``(y, act)``: FC1 output and ``silu(gate) * up`` of it, fused into one kernel on CUDA."""
    return _pick(x).linear_swiglu_fwd(x, w, alpha)


def linear_dgrad(dy, w, alpha: float = 1.0):
    return _pick(dy).linear_dgrad(dy, w, alpha)


def linear_dgrad_swiglu_bwd(dy, w2, y1, alpha: float = 1.0):
    """``swiglu_bwd(alpha * dy @ w2, y1)``: FC2 dgrad and the activation backward, one kernel on CUDA."""
    return _pick(dy).linear_dgrad_swiglu_bwd(dy, w2, y1, alpha)


def linear_wgrad(dy, x, out, accumulate: bool, alpha: float = 1.0):
    return _pick(dy).linear_wgrad(dy, x, out, accumulate, alpha)


def cross_entropy_fwd_bwd(logits, labels, mask, loss_scale, valid=None, vocab_start=0,
                          stats_reduce=None, tp_exchange=None):
    if logits.is_cuda:
        return _cuda().cross_entropy_fwd_bwd(logits, labels, mask, loss_scale, valid, vocab_start,
                                             stats_reduce, tp_exchange)
    return _ref.cross_entropy_fwd_bwd(logits, labels, mask, loss_scale, valid, vocab_start,
                                      stats_reduce)


def rope_tables(seq_len, head_dim, base, device=None):
    return _ref.rope_tables(seq_len, head_dim, base, device=device)
