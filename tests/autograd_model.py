"""Autograd statement of the decoder used as the oracle of the hand-written backward."""
import math

import torch
import torch.nn.functional as F


def rmsnorm(x, w, eps):
    return x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + eps) * w


def rope(x, cos, sin):
    # x: [B, S, heads, D]
    half = x.shape[-1] // 2
    x1, x2 = x[..., :half], x[..., half:]
    c, s = cos[None, :, None, :], sin[None, :, None, :]
    return torch.cat([x1 * c - x2 * s, x2 * c + x1 * s], dim=-1)


def forward_loss(spec, params, tokens, labels, mask, cos, sin):
    B, S = tokens.shape
    G, g, D = spec.num_query_groups, spec.heads_per_group, spec.head_dim
    r = spec.mup_residual_scale
    h = params["tok_embeddings.weight"][tokens.reshape(-1)] * spec.emb_scale
    for i in range(spec.num_layers):
        p = f"layers.{i}"
        n1 = rmsnorm(h, params[f"{p}.attention_norm.weight"], spec.norm_epsilon)
        qkv = (n1 @ params[f"{p}.attention.wqkv.weight"].t()).view(B, S, G, g + 2, D)
        q = rope(qkv[:, :, :, :g].reshape(B, S, G * g, D), cos[:S], sin[:S])
        k = rope(qkv[:, :, :, g], cos[:S], sin[:S])
        v = qkv[:, :, :, g + 1]
        k = k.repeat_interleave(g, dim=2)
        v = v.repeat_interleave(g, dim=2)
        a = F.scaled_dot_product_attention(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2),
                                           is_causal=True, scale=1.0 / math.sqrt(D))
        a = a.transpose(1, 2).reshape(B * S, G * g * D)
        h = h + r * (a @ params[f"{p}.attention.wo.weight"].t())
        n2 = rmsnorm(h, params[f"{p}.ffn_norm.weight"], spec.norm_epsilon)
        y1 = n2 @ params[f"{p}.feed_forward.wfc1.weight"].t()
        gate, up = y1.chunk(2, dim=-1)
        h = h + r * ((F.silu(gate) * up) @ params[f"{p}.feed_forward.w2.weight"].t())
    nf = rmsnorm(h, params["norm.weight"], spec.norm_epsilon) / spec.mup_width_scale
    wout = params["tok_embeddings.weight"] if spec.tie_embeddings else params["output.weight"]
    logits = nf @ wout.t()
    ce = F.cross_entropy(logits, labels.reshape(-1), reduction="none")
    m = mask.reshape(-1)
    return (ce * m).sum() / m.sum().clamp_min(1.0)
