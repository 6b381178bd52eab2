"""Hand-written forward/backward vs autograd (fp32, CPU)."""
import pytest
import torch

from forgetrain_b200.config import load_model_spec
from forgetrain_b200.models.minicpm4 import MiniCPM4
from forgetrain_b200.models.params import ParamStore
from forgetrain_b200 import ops

from autograd_model import forward_loss


def _small_spec(tie):
    return load_model_spec("tiny", num_layers=2, vocab_size=512, hidden_size=128, ffn_hidden_size=256,
                           num_attention_heads=4, num_query_groups=2, head_dim=32, seq_length=64,
                           max_position_embeddings=64, tie_embeddings=tie)


@pytest.mark.parametrize("tie", [False, True])
def test_manual_backward_matches_autograd(tie):
    torch.manual_seed(0)
    spec = _small_spec(tie)
    store = ParamStore(spec, "cpu", torch.float32)
    store.init_random(0)
    for ps in store.specs:  # make norm weights non-trivial
        if ps.is_norm:
            store.params[ps.name].add_(0.1 * torch.randn(ps.shape))
    model = MiniCPM4(spec, store)
    B, S = 2, 64
    tokens = torch.randint(0, spec.vocab_size, (B, S))
    labels = torch.randint(0, spec.vocab_size, (B, S))
    mask = (torch.rand(B, S) > 0.2).float()
    loss = model.forward_backward(tokens, labels, mask, loss_scale=1.0)
    ref_params = {ps.name: store.params[ps.name].clone().requires_grad_(True) for ps in store.specs}
    ref_loss = forward_loss(spec, ref_params, tokens, labels, mask, model.cos, model.sin)
    ref_loss.backward()
    assert abs(float(loss) - float(ref_loss.detach())) < 1e-4
    for ps in store.specs:
        a, b = store.grads[ps.name], ref_params[ps.name].grad
        err = (a - b).abs().max() / (b.abs().max() + 1e-12)
        assert err < 2e-4, (ps.name, float(err))


def test_gradient_accumulation_equals_sum():
    torch.manual_seed(1)
    spec = _small_spec(False)
    store = ParamStore(spec, "cpu", torch.float32)
    store.init_random(0)
    model = MiniCPM4(spec, store)
    mk = lambda: (torch.randint(0, spec.vocab_size, (1, 64)), torch.randint(0, spec.vocab_size, (1, 64)))
    (t1, l1), (t2, l2) = mk(), mk()
    model.forward_backward(t1, l1, None, 0.5, accumulate=False)
    model.forward_backward(t2, l2, None, 0.5, accumulate=True)
    acc = store.flat_grads.clone()
    model.forward_backward(t1, l1, None, 0.5, accumulate=False)
    g1 = store.flat_grads.clone()
    model.forward_backward(t2, l2, None, 0.5, accumulate=False)
    g2 = store.flat_grads.clone()
    assert torch.allclose(acc, g1 + g2, atol=1e-6)


def test_grad_ready_reports_every_parameter_once():
    spec = _small_spec(False)
    store = ParamStore(spec, "cpu", torch.float32)
    store.init_random(0)
    model = MiniCPM4(spec, store)
    seen = []
    t = torch.randint(0, spec.vocab_size, (1, 64))
    model.forward_backward(t, t, None, 1.0, grad_ready=seen.append)
    assert sorted(seen) == sorted(ps.name for ps in store.specs)
    # reverse-registration order: the head first, the embedding last
    assert seen[0] == "output.weight" and seen[-1] == "tok_embeddings.weight"


def test_rope_inverse_is_transpose():
    torch.manual_seed(0)
    cos, sin = ops.rope_tables(32, 16, 10000.0)
    x = torch.randn(64, 2 * 4 * 16)
    y = ops.rope_(x.clone(), cos, sin, 2, 2, 2, 16)
    z = ops.rope_(y.clone(), cos, sin, 2, 2, 2, 16, inverse=True)
    assert torch.allclose(z, x, atol=1e-5)
    # v columns untouched
    v = x.view(64, 2, 4, 16)[:, :, 3]
    assert torch.equal(y.view(64, 2, 4, 16)[:, :, 3], v)


def test_init_schemes():
    """muP-aware, plain and depth-scaled initial standard deviations."""
    import math
    from forgetrain_b200.config import load_model_spec
    from forgetrain_b200.models.params import ParamStore
    spec = load_model_spec("tiny")
    stds = {}
    for scheme in ("spec", "normal", "mcore"):
        st = ParamStore(spec, "cpu", torch.float32)
        st.init_random(0, scheme, 0.1)
        stds[scheme] = {n: float(st.params[n].std()) for n in
                        ("tok_embeddings.weight", "layers.0.attention.wqkv.weight",
                         "layers.0.attention.wo.weight", "layers.1.feed_forward.w2.weight")}
        assert torch.all(st.params["layers.0.ffn_norm.weight"] == 1)
    w = math.sqrt(spec.mup_width_scale) if spec.mup_enabled else 1.0
    assert stds["spec"]["tok_embeddings.weight"] == pytest.approx(0.1, rel=0.05)
    assert stds["spec"]["layers.0.attention.wqkv.weight"] == pytest.approx(0.1 / w, rel=0.05)
    assert all(v == pytest.approx(0.1, rel=0.05) for v in stds["normal"].values())
    d = math.sqrt(2 * spec.num_layers)
    assert stds["mcore"]["layers.0.attention.wqkv.weight"] == pytest.approx(0.1, rel=0.05)
    assert stds["mcore"]["layers.0.attention.wo.weight"] == pytest.approx(0.1 / d, rel=0.05)
    assert stds["mcore"]["layers.1.feed_forward.w2.weight"] == pytest.approx(0.1 / d, rel=0.05)


def test_backward_diagnostics_hook():
    """``model.diagnostics = {}`` collects the gradients a cross-engine comparison starts from;
    leaving it None changes nothing."""
    spec = load_model_spec("tiny")
    store = ParamStore(spec, "cpu", torch.float32)
    store.init_random(0, "normal", 0.05)
    model = MiniCPM4(spec, store)
    tok = torch.randint(0, spec.vocab_size, (2, 33), generator=torch.Generator().manual_seed(1))
    x, y = tok[:, :-1].contiguous(), tok[:, 1:].contiguous()
    model.forward_backward(x, y)
    ref = store.flat_grads.clone()
    model.diagnostics = {}
    model.forward_backward(x, y)
    assert torch.equal(store.flat_grads, ref)
    d = model.diagnostics
    T, H, F = 64, spec.hidden_size, spec.ffn_hidden_size
    assert set(d) == {"d_normed_final", "d_hidden_after_norm", "d_hidden_into_last_layer",
                      "d_intermediate_last", "d_fc1_last"}
    assert d["d_normed_final"].shape == (T, H) and d["d_intermediate_last"].shape == (T, F)
    assert d["d_fc1_last"].shape == (T, 2 * F)
    assert torch.equal(d["d_hidden_after_norm"], d["d_hidden_into_last_layer"])
    assert float(d["d_fc1_last"].abs().sum()) > 0


def test_position_ids_reach_the_rotary_embedding():
    """A batch with ``position_ids`` equal to 0..S-1 trains exactly like one without them; with
    document-relative positions the loss differs, and a row whose second document is moved to the
    front of another row sees the same rotary phases there."""
    import torch
    from forgetrain_b200.config import load_model_spec
    from forgetrain_b200.engine_config import from_spec
    from forgetrain_b200.parallel.topology import Topology
    from forgetrain_b200.trainer import Trainer
    spec = load_model_spec("tiny")
    tok = torch.randint(1, spec.vocab_size, (2, 33), generator=torch.Generator().manual_seed(0))
    base = {"tokens": tok[:, :-1].contiguous(), "labels": tok[:, 1:].contiguous()}
    plain = torch.arange(32, dtype=torch.int32).expand(2, 32).contiguous()
    reset = torch.cat([torch.arange(16), torch.arange(16)]).to(torch.int32).expand(2, 32).contiguous()
    losses = {}
    for name, pos in (("none", None), ("plain", plain), ("reset", reset)):
        cfg = from_spec(spec, dtype="fp32", comm="nccl", warmup_iters=0)
        tr = Trainer(spec, cfg, Topology(device=torch.device("cpu")), seq_length=32, micro_batch_size=2,
                     seed=0)
        batch = dict(base) if pos is None else {**base, "position_ids": pos}
        losses[name] = float(tr.train_step([batch])["loss"])
    assert losses["plain"] == losses["none"]
    assert abs(losses["reset"] - losses["none"]) > 1e-6


@pytest.mark.parametrize("attn,mlp", [(True, False), (False, True), (True, True)])
def test_recompute_switches_give_bitwise_the_saved_activation_gradients(attn, mlp):
    """recompute_attn / recompute_mlp rebuild the dropped activations with the forward's own
    ops on the same inputs, so loss and every gradient are bitwise those of the default path;
    what the forward keeps per layer shrinks accordingly."""
    torch.manual_seed(3)
    spec = _small_spec(False)
    tokens = torch.randint(0, spec.vocab_size, (2, 64))
    labels = torch.randint(0, spec.vocab_size, (2, 64))
    out = []
    for kw in ({}, {"recompute_attn": attn, "recompute_mlp": mlp}):
        store = ParamStore(spec, "cpu", torch.float32)
        store.init_random(0)
        model = MiniCPM4(spec, store, **kw)
        logits = model.forward(tokens)
        kept = [(sv.attn is not None, sv.y1 is not None, sv.act is not None) for sv in model._saved]
        loss, dlogits = model.loss_and_dlogits(logits, labels, None, 1.0)
        model.backward(tokens, dlogits, accumulate=False)
        out.append((float(loss), store.flat_grads.clone(), kept))
    (l0, g0, k0), (l1, g1, k1) = out
    assert l0 == l1 and torch.equal(g0, g1)
    assert all(k == (True, True, True) for k in k0)
    assert all(k == (not attn, not mlp, not mlp) for k in k1)


def test_fused_fc2_dgrad_swiglu_backward_front_ends_agree():
    """``ops.linear_dgrad_swiglu_bwd`` and the tensor-parallel context's ``dgrad_gather_swiglu_bwd``
    are the composition of the dgrad GEMM and the SwiGLU backward (on CUDA one kernel computes it;
    the model calls the fused front end for every block but the last, whose intermediate gradient
    the diagnostics keep)."""
    from forgetrain_b200.parallel.tp import NO_TP
    torch.manual_seed(0)
    T, H, F = 24, 16, 32
    dy, w2, y1 = torch.randn(T, H), torch.randn(H, F) * 0.1, torch.randn(T, 2 * F)
    ref = ops.swiglu_bwd(ops.linear_dgrad(dy, w2, 0.7), y1)
    assert torch.equal(ops.linear_dgrad_swiglu_bwd(dy, w2, y1, 0.7), ref)
    got, gathered = NO_TP.dgrad_gather_swiglu_bwd(dy, w2, y1, alpha=0.7, key="bwd.ffn")
    assert torch.equal(got, ref) and gathered is dy
    # the closed form, for the record: d gate = d act * sig * (1 + g (1 - sig)) * u, d up = d act * g * sig
    da = 0.7 * dy @ w2
    g, u = y1[:, :F], y1[:, F:]
    sig = torch.sigmoid(g)
    closed = torch.cat([da * sig * (1 + g * (1 - sig)) * u, da * g * sig], dim=1)
    assert torch.allclose(ref, closed, rtol=1e-5, atol=1e-6)


def test_weight_gradient_stream_switch_is_inert_on_cpu_and_off_for_fused_tensor_parallelism():
    """``wgrad_side_stream`` defaults to on; the trainer only creates the stream on a CUDA device,
    outside graph modes, serial-stream mode and fused tensor parallelism, and without a stream the
    model's weight-gradient helper is the in-line call."""
    from forgetrain_b200.engine_config import from_spec
    from forgetrain_b200.parallel.topology import Topology
    from forgetrain_b200.trainer import Trainer
    spec = load_model_spec("tiny", num_layers=2, vocab_size=256, hidden_size=128, ffn_hidden_size=256,
                           num_attention_heads=4, num_query_groups=2, head_dim=32, seq_length=32,
                           max_position_embeddings=32)
    cfg = from_spec(spec, dtype="fp32", comm="nccl")
    assert cfg.wgrad_side_stream is True
    tr = Trainer(spec, cfg, Topology(device=torch.device("cpu")), seq_length=32, micro_batch_size=2, seed=0)
    assert tr.model.wgrad_stream is None and tr.model._wgrad_done == {}
    g = torch.Generator().manual_seed(0)
    c = torch.randint(0, 256, (2, 33), generator=g)
    batch = {"tokens": c[:, :-1].contiguous(), "labels": c[:, 1:].contiguous(),
             "loss_mask": torch.ones(2, 32)}
    l0 = float(tr.train_step([batch])["loss"])
    l1 = float(tr.train_step([batch])["loss"])
    assert l0 == l0 and l1 == l1 and tr.model._wgrad_done == {}
