"""MTP head: hand-written backward vs autograd (fp32, CPU)."""
import math

import torch
import torch.nn.functional as F

from forgetrain_b200.config import load_model_spec
from forgetrain_b200.models.minicpm4 import MiniCPM4
from forgetrain_b200.models.mtp import MTPHead, roll_left_one
from forgetrain_b200.models.params import ParamStore, all_param_specs

from autograd_model import rmsnorm, rope


def _block(spec, params, pre, h, B, S, cos, sin):
    G, g, D = spec.num_query_groups, spec.heads_per_group, spec.head_dim
    r = spec.mup_residual_scale
    n1 = rmsnorm(h, params[f"{pre}.attention_norm.weight"], spec.norm_epsilon)
    qkv = (n1 @ params[f"{pre}.attention.wqkv.weight"].t()).view(B, S, G, g + 2, D)
    q = rope(qkv[:, :, :, :g].reshape(B, S, G * g, D), cos[:S], sin[:S])
    k = rope(qkv[:, :, :, g], cos[:S], sin[:S]).repeat_interleave(g, dim=2)
    v = qkv[:, :, :, g + 1].repeat_interleave(g, dim=2)
    a = F.scaled_dot_product_attention(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2),
                                       is_causal=True, scale=1 / math.sqrt(D))
    h = h + r * (a.transpose(1, 2).reshape(B * S, -1) @ params[f"{pre}.attention.wo.weight"].t())
    n2 = rmsnorm(h, params[f"{pre}.ffn_norm.weight"], spec.norm_epsilon)
    gate, up = (n2 @ params[f"{pre}.feed_forward.wfc1.weight"].t()).chunk(2, dim=-1)
    return h + r * ((F.silu(gate) * up) @ params[f"{pre}.feed_forward.w2.weight"].t())


def _ce(logits, labels, mask):
    ce = F.cross_entropy(logits, labels.reshape(-1), reduction="none")
    m = mask.reshape(-1)
    return (ce * m).sum() / m.sum().clamp_min(1.0)


def test_mtp_backward_matches_autograd_and_param_registry():
    torch.manual_seed(0)
    spec = load_model_spec("tiny", num_layers=2, vocab_size=256, hidden_size=128, ffn_hidden_size=256,
                           num_attention_heads=4, num_query_groups=2, head_dim=32, seq_length=32,
                           max_position_embeddings=32, tie_embeddings=False)
    K, factor = 2, 0.3
    names = [s.name for s in all_param_specs(spec, K)]
    assert "mtp.layers.1.eh_proj.weight" in names and names[-1] == "output.weight"
    store = ParamStore(spec, "cpu", torch.float32, mtp_num_layers=K)
    store.init_random(0)
    model = MiniCPM4(spec, store)
    head = MTPHead(model, K, factor)
    B, S = 2, 32
    tok = torch.randint(0, spec.vocab_size, (B, S))
    lab = torch.randint(0, spec.vocab_size, (B, S))
    msk = (torch.rand(B, S) > 0.2).float()
    seen = []
    loss = head.forward_backward(tok, lab, msk, 1.0, grad_ready=seen.append)
    assert sorted(seen) == sorted(names)

    P = {n: store.params[n].clone().requires_grad_(True) for n in names}
    cos, sin = model.cos, model.sin
    h = P["tok_embeddings.weight"][tok.reshape(-1)] * spec.emb_scale
    for i in range(spec.num_layers):
        h = _block(spec, P, f"layers.{i}", h, B, S, cos, sin)
    nf = rmsnorm(h, P["norm.weight"], spec.norm_epsilon)
    total = _ce((nf / spec.mup_width_scale) @ P["output.weight"].t(), lab, msk)
    main = total.detach().clone()
    ids, l2, m2, hid = tok, lab, msk, nf
    for k in range(K):
        pre = f"mtp.layers.{k}"
        ids, l2, m2 = roll_left_one(ids), roll_left_one(l2), roll_left_one(m2)
        e = P["tok_embeddings.weight"][ids.reshape(-1)] * spec.emb_scale
        comb = torch.cat([rmsnorm(e, P[f"{pre}.enorm.weight"], spec.norm_epsilon),
                          rmsnorm(hid, P[f"{pre}.hnorm.weight"], spec.norm_epsilon)], dim=-1)
        hid = _block(spec, P, pre, comb @ P[f"{pre}.eh_proj.weight"].t(), B, S, cos, sin)
        total = total + factor / K * _ce((hid / spec.mup_width_scale) @ P["output.weight"].t(), l2, m2)
    total.backward()
    assert abs(float(loss) - float(main)) < 1e-4
    for n in names:
        a, b = store.grads[n], P[n].grad
        err = float((a - b).abs().max() / (b.abs().max() + 1e-12))
        assert err < 3e-4, (n, err)
