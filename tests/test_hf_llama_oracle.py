"""An oracle that shares no code with this engine: the exported weights, loaded into the
``transformers`` Llama model, must give this engine's logits. MiniCPM is the Llama block with three
muP multipliers (embedding output x ``scale_emb``, every residual branch x ``scale_depth /
sqrt(layers)``, hidden state / (``hidden / dim_model_base``) before the head), which are folded into
the embedding, the two output projections and the head here. The comparison covers the exporter's
de-interleaving of the fused QKV and gate / up rows, the rotary convention (half-split pairs), GQA
head grouping, RMSNorm and the causal mask. Exporter under test: ckpt/convert_to_hf.py (reference:
exports/train_engine_0.5B/scripts/convert_to_hf.py:58-227)."""
import pytest
import torch

transformers = pytest.importorskip("transformers")

from forgetrain_b200.ckpt.convert_to_hf import to_hf_state_dict  # noqa: E402
from forgetrain_b200.config import load_model_spec  # noqa: E402
from forgetrain_b200.models.minicpm4 import MiniCPM4  # noqa: E402
from forgetrain_b200.models.params import ParamStore  # noqa: E402


def _llama_from(spec, params):
    from transformers import LlamaConfig, LlamaForCausalLM
    sd, _ = to_hf_state_dict(params, spec, dtype=torch.float32)
    sd = {k: v.clone() for k, v in sd.items()}
    sd["model.embed_tokens.weight"] *= spec.mup_emb_scale
    for i in range(spec.num_layers):
        sd[f"model.layers.{i}.self_attn.o_proj.weight"] *= spec.mup_residual_scale
        sd[f"model.layers.{i}.mlp.down_proj.weight"] *= spec.mup_residual_scale
    sd["lm_head.weight"] /= spec.mup_width_scale
    cfg = LlamaConfig(vocab_size=spec.vocab_size, hidden_size=spec.hidden_size,
                      intermediate_size=spec.ffn_hidden_size, num_hidden_layers=spec.num_layers,
                      num_attention_heads=spec.num_attention_heads,
                      num_key_value_heads=spec.num_query_groups, head_dim=spec.head_dim,
                      rms_norm_eps=spec.norm_epsilon, rope_theta=spec.rotary_base,
                      max_position_embeddings=spec.max_position_embeddings, tie_word_embeddings=False,
                      attention_bias=False, mlp_bias=False, hidden_act="silu")
    hf = LlamaForCausalLM(cfg).float().eval()
    hf.load_state_dict(sd, strict=True)
    return hf


@pytest.mark.parametrize("heads,groups,head_dim", [(4, 2, 64), (8, 8, 32), (8, 1, 32)])
def test_exported_weights_in_the_transformers_llama_model_give_the_engines_logits_and_loss(heads, groups, head_dim):
    spec = load_model_spec("tiny", tie_embeddings=False, hidden_size=512, num_layers=3,
                           num_attention_heads=heads, num_query_groups=groups, head_dim=head_dim,
                           ffn_hidden_size=768, vocab_size=1000)
    assert spec.mup_enabled and spec.mup_width_scale == 2.0 and spec.mup_emb_scale == 12.0
    st = ParamStore(spec, "cpu", torch.float32)
    st.init_random(0)
    g = torch.Generator().manual_seed(5)
    for ps in st.specs:                       # norm weights away from one, so that they matter
        if ps.is_norm:
            st.params[ps.name].add_(0.1 * torch.randn(st.params[ps.name].shape, generator=g))
    model = MiniCPM4(spec, st)
    B, S = 2, 40
    chunk = torch.randint(0, spec.vocab_size, (B, S + 1), generator=torch.Generator().manual_seed(1))
    tokens, labels = chunk[:, :-1].contiguous(), chunk[:, 1:].contiguous()
    logits = model.forward(tokens)
    ours = logits.float().view(B, S, -1).clone()
    hf = _llama_from(spec, {n: st.params[n] for n in st.offsets})
    with torch.no_grad():
        ref = hf(input_ids=tokens).logits
    assert float(ref.abs().max()) > 0.1
    assert torch.allclose(ours, ref, atol=2e-5, rtol=1e-4), float((ours - ref).abs().max())
    loss, _ = model.loss_and_dlogits(logits, labels, None, 1.0)
    want = torch.nn.functional.cross_entropy(ref.view(B * S, -1), labels.view(-1))
    assert float(loss) == pytest.approx(float(want), rel=1e-5)


def test_gradients_match_autograd_through_the_transformers_model():
    """The hand-derived backward against autograd of the independent model: gradients of the exported
    tensors are mapped back through the same folding and (de-)interleaving."""
    from forgetrain_b200.ckpt.convert_to_hf import merge_qkv_interleaved
    spec = load_model_spec("tiny", tie_embeddings=False, hidden_size=512, num_layers=2,
                           num_attention_heads=4, num_query_groups=2, head_dim=64,
                           ffn_hidden_size=768, vocab_size=1000)
    st = ParamStore(spec, "cpu", torch.float32)
    st.init_random(3)
    model = MiniCPM4(spec, st)
    B, S = 2, 24
    chunk = torch.randint(0, spec.vocab_size, (B, S + 1), generator=torch.Generator().manual_seed(2))
    tokens, labels = chunk[:, :-1].contiguous(), chunk[:, 1:].contiguous()
    loss = model.forward_backward(tokens, labels, None, 1.0, False, None, None)
    hf = _llama_from(spec, {n: st.params[n] for n in st.offsets}).train()
    out = hf(input_ids=tokens).logits
    ref_loss = torch.nn.functional.cross_entropy(out.view(B * S, -1), labels.view(-1))
    ref_loss.backward()
    assert float(loss) == pytest.approx(float(ref_loss.detach()), rel=1e-5)
    g = {k: v.grad for k, v in hf.named_parameters()}
    res, ws, emb = spec.mup_residual_scale, spec.mup_width_scale, spec.mup_emb_scale

    def close(a, b, name):
        assert torch.allclose(a, b, atol=2e-5 * max(1.0, float(b.abs().max())), rtol=2e-4), \
            (name, float((a - b).abs().max()), float(b.abs().max()))

    # folded tensors: d/dw = d/d(w * c) * c
    close(st.grads["tok_embeddings.weight"], g["model.embed_tokens.weight"] * emb, "embedding")
    close(st.grads["output.weight"], g["lm_head.weight"] / ws, "head")
    close(st.grads["norm.weight"], g["model.norm.weight"], "final norm")
    for i in range(spec.num_layers):
        hp, p = f"model.layers.{i}", f"layers.{i}"
        qkv = merge_qkv_interleaved(g[f"{hp}.self_attn.q_proj.weight"], g[f"{hp}.self_attn.k_proj.weight"],
                                    g[f"{hp}.self_attn.v_proj.weight"], spec)
        close(st.grads[f"{p}.attention.wqkv.weight"], qkv, f"{p} qkv")
        close(st.grads[f"{p}.attention.wo.weight"], g[f"{hp}.self_attn.o_proj.weight"] * res, f"{p} wo")
        fc1 = torch.cat([g[f"{hp}.mlp.gate_proj.weight"], g[f"{hp}.mlp.up_proj.weight"]], dim=0)
        close(st.grads[f"{p}.feed_forward.wfc1.weight"], fc1, f"{p} fc1")
        close(st.grads[f"{p}.feed_forward.w2.weight"], g[f"{hp}.mlp.down_proj.weight"] * res, f"{p} w2")
        close(st.grads[f"{p}.attention_norm.weight"], g[f"{hp}.input_layernorm.weight"], f"{p} norm1")
        close(st.grads[f"{p}.ffn_norm.weight"], g[f"{hp}.post_attention_layernorm.weight"], f"{p} norm2")
