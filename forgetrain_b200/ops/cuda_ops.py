"""CUDA implementations of the ops in :mod:`forgetrain_b200.ops.reference`, same signatures.

Every function launches hand-written sm_100a kernels from the in-tree native library
(``csrc/elementwise.cu``, ``csrc/gemm_sm100.cu``, ``csrc/attn_sm100.cu``) on the current
stream. Tensors must be bf16 (activations / weights) or fp32 (statistics, weight gradients,
optimizer state), contiguous in the last dimension and 16-byte aligned.
"""
from __future__ import annotations

import torch

from . import _lib, gemm

c_int, c_long, c_float = _lib.c_int, _lib.c_long, _lib.c_float
P = _lib.ptr


def _L():
    return _lib.lib()


def _bf16(t: torch.Tensor, name: str) -> None:
    if t.dtype != torch.bfloat16 or not t.is_cuda or t.stride(-1) != 1 or t.data_ptr() % 16:
        raise ValueError(f"{name}: expected an aligned CUDA bf16 tensor contiguous in its last "
                         f"dimension, got {t.dtype} {tuple(t.shape)} strides {t.stride()}")


# ------------------------------------------------------------------------------ embedding
def embedding_fwd(ids, w, scale, vocab_start: int = 0):
    ids = ids.reshape(-1)
    T, H = ids.numel(), w.shape[1]
    out = torch.empty(T, H, dtype=w.dtype, device=w.device)
    rc = _L().ft_embedding_fwd(P(ids), P(w), P(out), c_int(T), c_int(H), c_float(scale),
                               c_int(vocab_start), c_int(w.shape[0]), _lib.stream())
    _lib.check_rc(rc, "ft_embedding_fwd")
    return out


def embedding_bwd(ids, dy, scale, dw, vocab_start: int = 0):
    ids = ids.reshape(-1)
    _bf16(dy, "dy")
    assert dw.dtype == torch.float32 and dw.is_contiguous()
    rc = _L().ft_embedding_bwd(P(ids), P(dy), P(dw), c_int(ids.numel()), c_int(dy.shape[1]),
                               c_float(scale), c_int(vocab_start), c_int(dw.shape[0]),
                               _lib.stream())
    _lib.check_rc(rc, "ft_embedding_bwd")


# ------------------------------------------------------------------------------- RMSNorm
def add_rmsnorm_fwd(res, x, w, eps, y_out=None):
    _bf16(x, "x")
    assert x.is_contiguous() and (res is None or res.is_contiguous())
    T, H = x.shape
    y = torch.empty_like(x) if y_out is None else y_out
    assert y.is_contiguous() and y.shape == x.shape
    h = torch.empty_like(x) if res is not None else x
    rstd = torch.empty(T, dtype=torch.float32, device=x.device)
    rc = _L().ft_add_rmsnorm_fwd(P(res), P(x), P(w), P(h if res is not None else None), P(y),
                                 P(rstd), c_int(T), c_int(H), c_float(eps), _lib.stream())
    _lib.check_rc(rc, "ft_add_rmsnorm_fwd")
    return h, y, rstd


def rmsnorm_bwd(dy, h, w, rstd, dres, dw, accumulate):
    _bf16(dy, "dy")
    assert dy.is_contiguous() and h.is_contiguous()
    T, H = dy.shape
    nparts = _L().ft_rmsnorm_bwd_partials(c_int(T), c_int(H))
    if nparts <= 0:
        raise ValueError(f"rmsnorm_bwd: unsupported hidden size {H}")
    partial = torch.empty(nparts, H, dtype=torch.float32, device=dy.device)
    out = dres if dres is not None else torch.empty_like(dy)
    rc = _L().ft_rmsnorm_bwd(P(dy), P(h), P(w), P(rstd), P(dres), P(out), P(partial), P(dw),
                             c_int(int(accumulate)), c_int(T), c_int(H), _lib.stream())
    _lib.check_rc(rc, "ft_rmsnorm_bwd")
    return out


# ---------------------------------------------------------------------------------- RoPE
def rope_(qkv, cos, sin, batch, n_groups, heads_per_group, head_dim, inverse=False,
          position_ids=None):
    _bf16(qkv, "qkv")
    T = qkv.shape[0]
    S = T // batch
    assert cos.dtype == torch.float32 and cos.is_contiguous() and cos.shape[1] == head_dim // 2
    if position_ids is not None:
        position_ids = position_ids.reshape(-1).to(torch.int32)
    rc = _L().ft_rope(P(qkv), P(cos), P(sin), P(position_ids), c_long(T), c_int(S),
                      c_int(n_groups), c_int(heads_per_group), c_int(head_dim),
                      c_int(qkv.stride(0)), c_int(int(inverse)), _lib.stream())
    _lib.check_rc(rc, "ft_rope")
    return qkv


# -------------------------------------------------------------------------------- SwiGLU
def swiglu_fwd(y1):
    _bf16(y1, "y1")
    T, F2 = y1.shape
    F = F2 // 2
    act = torch.empty(T, F, dtype=y1.dtype, device=y1.device)
    rc = _L().ft_swiglu_fwd(P(y1), P(act), c_long(T), c_int(F), c_int(y1.stride(0)),
                            c_int(act.stride(0)), _lib.stream())
    _lib.check_rc(rc, "ft_swiglu_fwd")
    return act


def swiglu_bwd(dact, y1):
    _bf16(dact, "dact")
    T, F2 = y1.shape
    F = F2 // 2
    dy1 = torch.empty_like(y1)
    rc = _L().ft_swiglu_bwd(P(dact), P(y1), P(dy1), c_long(T), c_int(F), c_int(dact.stride(0)),
                            c_int(y1.stride(0)), _lib.stream())
    _lib.check_rc(rc, "ft_swiglu_bwd")
    return dy1


# -------------------------------------------------------------------------------- linear
def linear_fwd(x, w, alpha=1.0):
    return gemm.linear_fwd(x, w, alpha=alpha)


def linear_swiglu_fwd(x, w, alpha=1.0):
    if (w.shape[0] // 2) % 128:
        y = gemm.linear_fwd(x, w, alpha=alpha)
        return y, swiglu_fwd(y)
    return gemm.linear_swiglu_fwd(x, w, alpha=alpha)


def linear_dgrad(dy, w, alpha=1.0):
    return gemm.linear_dgrad(dy, w, alpha=alpha)


def linear_dgrad_swiglu_bwd(dy, w2, y1, alpha=1.0):
    if w2.shape[1] % 64:
        return swiglu_bwd(gemm.linear_dgrad(dy, w2, alpha=alpha), y1)
    return gemm.linear_dgrad_swiglu_bwd(dy, w2, y1, alpha=alpha)


def linear_wgrad(dy, x, out, accumulate, alpha=1.0):
    return gemm.linear_wgrad(dy, x, out=out, accumulate=accumulate, alpha=alpha)


# ------------------------------------------------------------------------- cross-entropy
def cross_entropy_fwd_bwd(logits, labels, mask, loss_scale, valid=None, vocab_start=0,
                          stats_reduce=None, tp_exchange=None):
    """In place: ``logits`` is overwritten by its gradient (returned as ``dlogits``).
    ``tp_exchange`` (an object with ``ce_stats_buffer`` / ``ce_exchange``) combines the
    vocabulary-shard statistics in one peer-memory kernel instead of two all-reduces."""
    _bf16(logits, "logits")
    T, V = logits.shape
    dev = logits.device
    labels = labels.reshape(-1)
    if mask is not None:
        mask = mask.reshape(-1).to(torch.float32)
    if valid is None:
        valid_t = (mask.sum().reshape(1) if mask is not None
                   else torch.full((1,), float(T), dtype=torch.float32, device=dev))
    elif torch.is_tensor(valid):
        valid_t = valid.reshape(1).to(torch.float32)
    else:
        valid_t = torch.full((1,), float(valid), dtype=torch.float32, device=dev)
    stats = torch.empty(3, T, dtype=torch.float32, device=dev)
    row_loss = torch.empty(T, dtype=torch.float32, device=dev)
    loss = torch.empty(1, dtype=torch.float32, device=dev)
    L = _L()
    st = _lib.stream()
    sym = tp_exchange.ce_stats_buffer(T) if tp_exchange is not None else None
    if stats_reduce is None and sym is None:
        rc = L.ft_cross_entropy(P(logits), P(labels), P(mask), P(valid_t), P(stats), P(row_loss),
                                c_int(T), c_int(V), c_long(logits.stride(0)), c_int(vocab_start),
                                c_float(loss_scale), c_int(3), st)
        _lib.check_rc(rc, "ft_cross_entropy")
    elif sym is not None:
        rc = L.ft_cross_entropy(P(logits), P(labels), P(mask), P(valid_t), P(sym), P(row_loss),
                                c_int(T), c_int(V), c_long(logits.stride(0)), c_int(vocab_start),
                                c_float(loss_scale), c_int(1), st)
        _lib.check_rc(rc, "ft_cross_entropy(stats)")
        tp_exchange.ce_exchange(T, mask, stats, row_loss)
        rc = L.ft_cross_entropy(P(logits), P(labels), P(mask), P(valid_t), P(stats), P(row_loss),
                                c_int(T), c_int(V), c_long(logits.stride(0)), c_int(vocab_start),
                                c_float(loss_scale), c_int(2), st)
        _lib.check_rc(rc, "ft_cross_entropy(grad)")
    else:
        rc = L.ft_cross_entropy(P(logits), P(labels), P(mask), P(valid_t), P(stats), P(row_loss),
                                c_int(T), c_int(V), c_long(logits.stride(0)), c_int(vocab_start),
                                c_float(loss_scale), c_int(1), st)
        _lib.check_rc(rc, "ft_cross_entropy(stats)")
        gmax = stats_reduce(stats[0].clone(), "max")
        # rebase the local sum-exp onto the global maximum before summing over ranks
        stats[1].mul_(torch.exp(stats[0] - gmax))
        stats[0].copy_(gmax)
        red = stats_reduce(stats[1:3].clone(), "sum")
        stats[1:3].copy_(red)
        rc = L.ft_ce_row_loss(P(stats), P(mask), P(row_loss), c_int(T), st)
        _lib.check_rc(rc, "ft_ce_row_loss")
        rc = L.ft_cross_entropy(P(logits), P(labels), P(mask), P(valid_t), P(stats), P(row_loss),
                                c_int(T), c_int(V), c_long(logits.stride(0)), c_int(vocab_start),
                                c_float(loss_scale), c_int(2), st)
        _lib.check_rc(rc, "ft_cross_entropy(grad)")
    rc = L.ft_reduce_sum(P(row_loss), c_long(T), P(valid_t), c_float(1.0), P(loss), c_int(0), st)
    _lib.check_rc(rc, "ft_reduce_sum")
    return loss[0], logits


# --------------------------------------------------------------------------------- AdamW
def adamw_flat(p32, m, v, g, p_out, hyper, seg_end, seg_wd, seg_lr_mult):
    """Fused AdamW over a flat fp32 shard; ``hyper`` is the 8-float device vector
    ``[lr, beta1, beta2, eps, bias_corr1, bias_corr2, clip, _]``."""
    n = p32.numel()
    rc = _L().ft_adamw(P(p32), P(m), P(v), P(g), P(p_out), c_long(n), P(hyper), P(seg_end),
                       P(seg_wd), P(seg_lr_mult), c_int(seg_end.numel()), _lib.stream())
    _lib.check_rc(rc, "ft_adamw")


def sumsq_into(x, out) -> None:
    """``out[0] += sum(x^2)`` for a flat fp32 tensor."""
    assert x.dtype == torch.float32 and x.is_contiguous()
    rc = _L().ft_sumsq(P(x), c_long(x.numel()), P(out), _lib.stream())
    _lib.check_rc(rc, "ft_sumsq")


def clip_coef(sumsq_t, max_norm, hyper, norm_out) -> None:
    """``hyper[6] = min(1, max_norm/(sqrt(sumsq)+1e-6))``, ``norm_out[0] = sqrt(sumsq)``."""
    rc = _L().ft_clip_coef(P(sumsq_t), c_float(max_norm), c_void_off(hyper, 6), P(norm_out),
                           _lib.stream())
    _lib.check_rc(rc, "ft_clip_coef")


def adam_hyper_step(step_dev, sched, hyper) -> None:
    """Device-side schedule: ``step_dev[0] += 1`` and ``hyper[0:6]`` = this step's learning
    rate (warmup - stable - decay), betas, eps and bias corrections."""
    assert step_dev.dtype == torch.int32 and sched.dtype == torch.float32 and sched.numel() >= 8
    rc = _L().ft_adam_hyper(P(step_dev), P(sched), P(hyper), _lib.stream())
    _lib.check_rc(rc, "ft_adam_hyper")


def c_void_off(t: torch.Tensor, elem_off: int):
    return _lib.c_void_p(t.data_ptr() + elem_off * t.element_size())


# ----------------------------------------------------------------------------- attention
def attention_fwd(qkv, batch, n_groups, heads_per_group, head_dim, scale=None):
    from . import attention
    return attention.attention_fwd(qkv, batch, n_groups, heads_per_group, head_dim, scale)


def attention_bwd(dout, qkv, out, lse, batch, n_groups, heads_per_group, head_dim, scale=None,
                  rope=None):
    from . import attention
    return attention.attention_bwd(dout, qkv, out, lse, batch, n_groups, heads_per_group,
                                   head_dim, scale, rope=rope)
