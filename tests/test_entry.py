"""Gate entry points: forward / forward + backward from a checkpoint on a given batch."""
import pytest
import torch

from forgetrain_b200 import entry
from forgetrain_b200.ckpt import megatron_import as mg
from forgetrain_b200.config import load_model_spec
from forgetrain_b200.models.minicpm4 import MiniCPM4
from forgetrain_b200.models.params import ParamStore, all_param_specs


def _export(tmp_path, spec):
    g = torch.Generator().manual_seed(0)
    ours = {ps.name: torch.randn(ps.shape, generator=g) * 0.05 for ps in all_param_specs(spec)}
    for n in ours:
        if n.endswith("norm.weight"):
            ours[n] = 1.0 + 0.1 * ours[n]
    names = entry.megatron_grad_names(spec.num_layers, fused_norm_keys=True)
    torch.save({names[n]: t.clone() for n, t in ours.items() if n in names}, tmp_path / mg.PARAMS_FILE)
    return ours


def _batch(spec, B=2, S=32):
    c = torch.randint(0, spec.vocab_size, (B, S + 1), generator=torch.Generator().manual_seed(1))
    mask = torch.ones(B, S)
    mask[0, :5] = 0
    return {"tokens": c[:, :-1].contiguous(), "labels": c[:, 1:].contiguous(), "loss_mask": mask}


def test_run_forward_matches_the_model_and_masks_the_mean(tmp_path):
    spec = load_model_spec("tiny", tie_embeddings=False)
    ours = _export(tmp_path, spec)
    batch = _batch(spec)
    loss, per_tok = entry.run_forward(tmp_path, batch, "cpu", spec=spec)
    assert per_tok.shape == (2, 32) and per_tok.dtype == torch.float32
    assert loss == pytest.approx(float((per_tok * batch["loss_mask"]).sum() / batch["loss_mask"].sum()))
    st = ParamStore(spec, "cpu", torch.float32)
    st.load_named(ours, full_tensors=True)
    want = MiniCPM4(spec, st).forward_backward(batch["tokens"], batch["labels"], batch["loss_mask"])
    assert loss == pytest.approx(float(want), rel=1e-5)


def test_run_forward_backward_returns_clipped_grads_by_megatron_names(tmp_path):
    spec = load_model_spec("tiny", tie_embeddings=False)
    ours = _export(tmp_path, spec)
    batch = _batch(spec)
    loss, grads = entry.run_forward_backward(tmp_path, batch, "cpu", spec=spec, clip_grad=0.5)
    assert "decoder.layers.0.self_attention.linear_qkv.layer_norm_weight" in grads
    assert "decoder.layers.0.input_layernorm.weight" not in grads
    assert "embedding.word_embeddings.weight" in grads and "output_layer.weight" in grads
    assert all(g.dtype == torch.float32 for g in grads.values())
    total = torch.sqrt(sum(g.double().pow(2).sum() for g in grads.values()))
    assert float(total) == pytest.approx(0.5, rel=1e-4)            # the raw norm was above the limit
    _, raw = entry.run_forward_backward(tmp_path, batch, "cpu", spec=spec, clip_grad=0.0,
                                        fused_norm_keys=False)
    assert "decoder.layers.0.input_layernorm.weight" in raw
    st = ParamStore(spec, "cpu", torch.float32)
    st.load_named(ours, full_tensors=True)
    MiniCPM4(spec, st).forward_backward(batch["tokens"], batch["labels"], batch["loss_mask"])
    assert torch.allclose(raw["decoder.layers.1.mlp.linear_fc2.weight"],
                          st.grads["layers.1.feed_forward.w2.weight"])
    k = "decoder.layers.1.mlp.linear_fc2.weight"
    assert torch.allclose(grads[k], raw[k] * (0.5 / (float(torch.sqrt(sum(
        g.double().pow(2).sum() for g in raw.values()))) + 1e-6)), rtol=1e-5)


def test_entry_points_also_take_a_checkpoint_of_this_engine(tmp_path):
    from forgetrain_b200.ckpt import checkpoint as ck
    spec = load_model_spec("tiny")
    st = ParamStore(spec, "cpu", torch.float32)
    st.init_random(0)
    names = [p.name for p in st.specs]
    ck.save_checkpoint(tmp_path, 3, params={n: st.params[n] for n in names}, param_names=names,
                       optimizer_state=None, async_io=False)
    loss, per_tok = entry.run_forward(tmp_path / "step_0000003", _batch(spec), "cpu", model="tiny")
    assert per_tok.shape == (2, 32) and loss > 0
    from training_engine_tensor.entry import run_forward, run_training
    assert run_forward is entry.run_forward and callable(run_training)


def test_loss_readback_handle_returns_the_step_result_on_cpu():
    import torch
    from forgetrain_b200.trainer import LossReadback
    h = LossReadback(torch.tensor([2.5]), torch.tensor([0.75]))
    assert h.value() == (2.5, 0.75) and h.nbytes == 8
