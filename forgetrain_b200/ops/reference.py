"""Plain PyTorch statement of every op of the model, optimizer and loss.

These functions are (a) the implementation used on CPU (gloo plumbing runs, unit tests) and
(b) the oracle the CUDA kernels are compared against. They work in the dtype of their inputs
with fp32 internal math, and follow the rounding points of the numerical contract:
residual sums are rounded to the storage dtype before the variance is taken, weight gradients
and the loss are fp32, activation gradients are in the storage dtype.

Semantics follow the reference's baseline ops
(exports/train_engine_0.5B/src/training_engine_tensor/kernels.py:39-56,265-335 for RoPE and the
QKV layout, triton_kernels.py:39-178 for cross-entropy, :302-406 / :645-791 for RMSNorm,
:186-294 for SwiGLU, :414-607 for AdamW).
"""
from __future__ import annotations

import math

import torch


# ------------------------------------------------------------------------------ embedding
def embedding_fwd(ids: torch.Tensor, w: torch.Tensor, scale: float) -> torch.Tensor:
    out = w[ids.reshape(-1)]
    return (out.float() * scale).to(w.dtype) if scale != 1.0 else out.clone()


def embedding_bwd(ids: torch.Tensor, dy: torch.Tensor, scale: float, dw: torch.Tensor,
                  vocab_start: int = 0) -> None:
    """``dw[ids - vocab_start] += scale * dy`` (fp32 accumulate); ids outside the local vocab
    range are skipped (vocab-parallel)."""
    flat = ids.reshape(-1) - vocab_start
    ok = (flat >= 0) & (flat < dw.shape[0])
    dw.index_add_(0, flat[ok], dy[ok].float() * scale)


# ------------------------------------------------------------------------------- RMSNorm
def add_rmsnorm_fwd(res: torch.Tensor | None, x: torch.Tensor, w: torch.Tensor, eps: float,
                    y_out: torch.Tensor | None = None):
    """``h = round(res + x)``; ``y = h * rsqrt(mean(h^2) + eps) * w``. Returns (h, y, rstd)."""
    h = x if res is None else (res.float() + x.float()).to(x.dtype)
    hf = h.float()
    rstd = torch.rsqrt(hf.pow(2).mean(dim=-1) + eps)
    y = (hf * rstd[:, None] * w.float()).to(x.dtype)
    if y_out is not None:
        y_out.copy_(y)
        y = y_out
    return h, y, rstd


def rmsnorm_bwd(dy: torch.Tensor, h: torch.Tensor, w: torch.Tensor, rstd: torch.Tensor,
                dres: torch.Tensor | None, dw: torch.Tensor, accumulate: bool):
    """``dx = rstd * (dy*w - xhat * mean(dy*w*xhat))`` added to ``dres`` (storage dtype);
    ``dw (+)= sum_rows dy * xhat`` in fp32. Returns dx (+ dres)."""
    xhat = h.float() * rstd[:, None]
    g = dy.float() * w.float()
    c = (g * xhat).mean(dim=-1, keepdim=True)
    dx = rstd[:, None] * (g - xhat * c)
    if dres is not None:
        dx = dx + dres.float()
    dwn = (dy.float() * xhat).sum(dim=0)
    if accumulate:
        dw.add_(dwn)
    else:
        dw.copy_(dwn)
    return dx.to(h.dtype)


# ---------------------------------------------------------------------------------- RoPE
def rope_tables(seq_len: int, head_dim: int, base: float, device=None,
                positions: torch.Tensor | None = None):
    """cos / sin tables [S, D/2] in fp32 (rotate-half convention: emb = cat(freqs, freqs))."""
    inv = 1.0 / (base ** (torch.arange(0, head_dim, 2, dtype=torch.float32, device=device) / head_dim))
    pos = torch.arange(seq_len, dtype=torch.float32, device=device) if positions is None \
        else positions.to(torch.float32)
    freqs = torch.outer(pos, inv)
    return freqs.cos(), freqs.sin()


def _qk_column_slices(n_groups: int, heads_per_group: int, head_dim: int):
    """Column ranges of the rotary-encoded heads (all q heads and the k head of every group)
    in the interleaved layout ``[q_0..q_{g-1} | k | v]`` per KV group."""
    gw = (heads_per_group + 2) * head_dim
    out = []
    for j in range(n_groups):
        for i in range(heads_per_group + 1):  # q heads then k
            out.append(j * gw + i * head_dim)
    return out


def rope_(qkv: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, batch: int, n_groups: int,
          heads_per_group: int, head_dim: int, inverse: bool = False,
          position_ids: torch.Tensor | None = None) -> torch.Tensor:
    """In-place rotary embedding of the q and k heads of ``qkv[T, n_groups*(g+2)*D]``.
    Token t of a batch-major [B, S] layout has position ``t % S`` unless ``position_ids[T]``
    is given (packed documents). ``inverse=True`` applies the transposed rotation (backward).
    """
    T = qkv.shape[0]
    S = T // batch
    half = head_dim // 2
    if position_ids is None:
        c = cos[:S].repeat(batch, 1)
        s = sin[:S].repeat(batch, 1)
    else:
        c = cos[position_ids.reshape(-1).long()]
        s = sin[position_ids.reshape(-1).long()]
    if inverse:
        s = -s
    for col in _qk_column_slices(n_groups, heads_per_group, head_dim):
        x1 = qkv[:, col:col + half].float().clone()
        x2 = qkv[:, col + half:col + head_dim].float().clone()
        qkv[:, col:col + half] = (x1 * c - x2 * s).to(qkv.dtype)
        qkv[:, col + half:col + head_dim] = (x2 * c + x1 * s).to(qkv.dtype)
    return qkv


# ----------------------------------------------------------------------------- attention
def split_qkv(qkv: torch.Tensor, batch: int, n_groups: int, heads_per_group: int, head_dim: int):
    """Views q[B,G,g,S,D], k[B,G,S,D], v[B,G,S,D] of the interleaved qkv[T, ...] buffer."""
    T = qkv.shape[0]
    S = T // batch
    x = qkv.view(batch, S, n_groups, heads_per_group + 2, head_dim)
    q = x[:, :, :, :heads_per_group].permute(0, 2, 3, 1, 4)
    k = x[:, :, :, heads_per_group].permute(0, 2, 1, 3)
    v = x[:, :, :, heads_per_group + 1].permute(0, 2, 1, 3)
    return q, k, v


def attention_fwd(qkv: torch.Tensor, batch: int, n_groups: int, heads_per_group: int,
                  head_dim: int, scale: float | None = None):
    """Causal GQA attention over the interleaved qkv buffer. Returns (out[T, Hq*D] in the
    storage dtype, lse[B, Hq, S] fp32, natural log)."""
    T = qkv.shape[0]
    S = T // batch
    scale = 1.0 / math.sqrt(head_dim) if scale is None else scale
    q, k, v = split_qkv(qkv, batch, n_groups, heads_per_group, head_dim)
    s = torch.einsum("bgqsd,bgtd->bgqst", q.float(), k.float()) * scale
    mask = torch.ones(S, S, dtype=torch.bool, device=qkv.device).tril()
    s = s.masked_fill(~mask, float("-inf"))
    lse = torch.logsumexp(s, dim=-1)
    p = torch.exp(s - lse[..., None])
    o = torch.einsum("bgqst,bgtd->bgqsd", p, v.float())
    out = o.permute(0, 3, 1, 2, 4).reshape(T, n_groups * heads_per_group * head_dim).to(qkv.dtype)
    return out, lse.reshape(batch, n_groups * heads_per_group, S)


def attention_bwd(dout: torch.Tensor, qkv: torch.Tensor, out: torch.Tensor, lse: torch.Tensor,
                  batch: int, n_groups: int, heads_per_group: int, head_dim: int,
                  scale: float | None = None) -> torch.Tensor:
    """Gradient wrt the interleaved qkv buffer (same layout and dtype as ``qkv``)."""
    T = qkv.shape[0]
    S = T // batch
    g = heads_per_group
    scale = 1.0 / math.sqrt(head_dim) if scale is None else scale
    q, k, v = split_qkv(qkv, batch, n_groups, g, head_dim)
    q, k, v = q.float(), k.float(), v.float()
    do = dout.view(batch, S, n_groups, g, head_dim).permute(0, 2, 3, 1, 4).float()
    o = out.view(batch, S, n_groups, g, head_dim).permute(0, 2, 3, 1, 4).float()
    s = torch.einsum("bgqsd,bgtd->bgqst", q, k) * scale
    mask = torch.ones(S, S, dtype=torch.bool, device=qkv.device).tril()
    p = torch.exp(s - lse.view(batch, n_groups, g, S)[..., None]).masked_fill(~mask, 0.0)
    dv = torch.einsum("bgqst,bgqsd->bgtd", p, do)
    dp = torch.einsum("bgqsd,bgtd->bgqst", do, v)
    delta = (o * do).sum(-1, keepdim=True)
    ds = p * (dp - delta) * scale
    dq = torch.einsum("bgqst,bgtd->bgqsd", ds, k)
    dk = torch.einsum("bgqst,bgqsd->bgtd", ds, q)
    dqkv = torch.empty_like(qkv)
    x = dqkv.view(batch, S, n_groups, g + 2, head_dim)
    x[:, :, :, :g] = dq.permute(0, 3, 1, 2, 4).to(qkv.dtype)
    x[:, :, :, g] = dk.permute(0, 2, 1, 3).to(qkv.dtype)
    x[:, :, :, g + 1] = dv.permute(0, 2, 1, 3).to(qkv.dtype)
    return dqkv


# -------------------------------------------------------------------------------- SwiGLU
def swiglu_fwd(y1: torch.Tensor) -> torch.Tensor:
    """``silu(gate) * up`` with ``y1 = [gate | up]`` along the last dimension."""
    gate, up = y1.float().chunk(2, dim=-1)
    return (torch.nn.functional.silu(gate) * up).to(y1.dtype)


def swiglu_bwd(dact: torch.Tensor, y1: torch.Tensor) -> torch.Tensor:
    gate, up = y1.float().chunk(2, dim=-1)
    sig = torch.sigmoid(gate)
    g = dact.float()
    dgate = g * sig * (1.0 + gate * (1.0 - sig)) * up
    dup = g * gate * sig
    return torch.cat([dgate, dup], dim=-1).to(y1.dtype)


# -------------------------------------------------------------------------------- linear
def linear_fwd(x: torch.Tensor, w: torch.Tensor, alpha: float = 1.0) -> torch.Tensor:
    y = x.float() @ w.float().t()
    return (y * alpha).to(x.dtype) if alpha != 1.0 else y.to(x.dtype)


def linear_swiglu_fwd(x: torch.Tensor, w: torch.Tensor, alpha: float = 1.0):
    y = linear_fwd(x, w, alpha)
    return y, swiglu_fwd(y)


def linear_dgrad_swiglu_bwd(dy: torch.Tensor, w2: torch.Tensor, y1: torch.Tensor,
                            alpha: float = 1.0) -> torch.Tensor:
    return swiglu_bwd(linear_dgrad(dy, w2, alpha), y1)


def linear_dgrad(dy: torch.Tensor, w: torch.Tensor, alpha: float = 1.0) -> torch.Tensor:
    dx = dy.float() @ w.float()
    return (dx * alpha).to(dy.dtype) if alpha != 1.0 else dx.to(dy.dtype)


def linear_wgrad(dy: torch.Tensor, x: torch.Tensor, out: torch.Tensor, accumulate: bool,
                 alpha: float = 1.0) -> torch.Tensor:
    dw = dy.float().t() @ x.float()
    if alpha != 1.0:
        dw = dw * alpha
    if accumulate:
        out.add_(dw)
    else:
        out.copy_(dw)
    return out


# ------------------------------------------------------------------------- cross-entropy
def cross_entropy_fwd_bwd(logits: torch.Tensor, labels: torch.Tensor, mask: torch.Tensor | None,
                          loss_scale: float, valid: torch.Tensor | float | None = None,
                          vocab_start: int = 0, stats_reduce=None):
    """Masked mean cross-entropy and its gradient.

    Returns ``(loss, dlogits)`` with ``loss = sum(mask * ce) / valid`` (fp32 scalar, not
    multiplied by ``loss_scale``) and ``dlogits = (softmax - onehot) * mask / valid *
    loss_scale`` in the dtype of ``logits``. With ``stats_reduce`` (vocab-parallel) the row
    maximum is max-reduced and (sum-exp, target logit) are sum-reduced across the
    tensor-parallel group; ``vocab_start`` is the first vocabulary id of the local shard.
    """
    lf = logits.float()
    T, V = lf.shape
    lab = labels.reshape(-1).long() - vocab_start
    m = torch.ones(T, dtype=torch.float32, device=lf.device) if mask is None else mask.reshape(-1).float()
    if valid is None:
        valid = m.sum().clamp_min(1.0)
    row_max = lf.max(dim=-1).values
    if stats_reduce is not None:
        row_max = stats_reduce(row_max, "max")
    ex = torch.exp(lf - row_max[:, None])
    sum_exp = ex.sum(dim=-1)
    in_shard = (lab >= 0) & (lab < V)
    tgt = torch.where(in_shard, lf.gather(1, lab.clamp(0, V - 1)[:, None])[:, 0],
                      torch.zeros_like(row_max))
    if stats_reduce is not None:
        st = stats_reduce(torch.stack([sum_exp, tgt]), "sum")
        sum_exp, tgt = st[0], st[1]
    ce = torch.log(sum_exp) + row_max - tgt
    loss = (ce * m).sum() / valid
    p = ex / sum_exp[:, None]
    onehot = torch.zeros_like(p)
    rows = torch.nonzero(in_shard)[:, 0]
    onehot[rows, lab[rows]] = 1.0
    coef = (m / valid * loss_scale)[:, None]
    dlogits = ((p - onehot) * coef).to(logits.dtype)
    return loss, dlogits


# --------------------------------------------------------------------------------- AdamW
def adamw_step(p32: torch.Tensor, m: torch.Tensor, v: torch.Tensor, g: torch.Tensor,
               p_out: torch.Tensor | None, lr: float, beta1: float, beta2: float, eps: float,
               weight_decay: float, step: int, clip: float = 1.0) -> None:
    """In-place AdamW with decoupled weight decay and bias correction on fp32 master weights;
    the updated value is also written to ``p_out`` in its (lower) dtype."""
    gg = g.float() * clip
    m.mul_(beta1).add_(gg, alpha=1.0 - beta1)
    v.mul_(beta2).addcmul_(gg, gg, value=1.0 - beta2)
    bc1 = 1.0 - beta1 ** step
    bc2 = 1.0 - beta2 ** step
    upd = (m / bc1) / ((v / bc2).sqrt() + eps) + weight_decay * p32
    p32.add_(upd, alpha=-lr)
    if p_out is not None:
        p_out.copy_(p32.to(p_out.dtype))


def sumsq(x: torch.Tensor) -> torch.Tensor:
    return x.float().pow(2).sum()
