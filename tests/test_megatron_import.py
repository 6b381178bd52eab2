"""Import of Megatron-exported parameters / optimizer state (both key layouts, MTP cold start,
vocabulary check) and ``train --checkpoint-root`` on top of it."""
import pytest
import torch

from forgetrain_b200.ckpt import megatron_import as mg
from forgetrain_b200.config import load_model_spec
from forgetrain_b200.models.params import all_param_specs


def _export(spec, fused, mtp=0, seed=0):
    """A fake Megatron export of ``spec`` with deterministic values."""
    g = torch.Generator().manual_seed(seed)
    ours = {ps.name: torch.randn(ps.shape, generator=g) for ps in all_param_specs(spec, mtp)}
    inv = {}
    for k, v in mg.megatron_name_map(spec.num_layers, mtp).items():
        is_fused_norm = k.endswith("layer_norm_weight")
        is_unfused_norm = k.endswith("input_layernorm.weight") or k.endswith("pre_mlp_layernorm.weight")
        if k.startswith("decoder.layers") and ((is_fused_norm and not fused) or (is_unfused_norm and fused)):
            continue
        inv[k] = v
    return {k: ours[v].clone() for k, v in inv.items() if v in ours}, ours


@pytest.mark.parametrize("fused", [False, True])
def test_both_key_layouts_round_trip(tmp_path, fused):
    spec = load_model_spec("tiny")
    ck, ours = _export(spec, fused)
    torch.save(ck, tmp_path / mg.PARAMS_FILE)
    assert mg.is_megatron_root(tmp_path)
    got = mg.load_megatron_checkpoint(tmp_path, spec, log=lambda *_: None)
    want = {n for n in ours if not (spec.tie_embeddings and n == "output.weight")}
    assert set(got) == want
    for n in want:
        assert torch.equal(got[n], ours[n])


def test_mtp_mapped_or_cold_started_and_vocab_checked(tmp_path):
    spec = load_model_spec("tiny")
    ck, ours = _export(spec, True, mtp=1)
    torch.save(ck, tmp_path / mg.PARAMS_FILE)
    got = mg.load_megatron_checkpoint(tmp_path, spec, 1, log=lambda *_: None)
    assert torch.equal(got["mtp.layers.0.eh_proj.weight"], ours["mtp.layers.0.eh_proj.weight"])
    # a checkpoint without the head: cold start, reported
    ck2 = {k: v for k, v in ck.items() if not k.startswith("mtp.")}
    torch.save(ck2, tmp_path / mg.PARAMS_FILE)
    lines = []
    got = mg.load_megatron_checkpoint(tmp_path, spec, 1, log=lines.append)
    assert torch.all(got["mtp.layers.0.enorm.weight"] == 1)
    assert float(got["mtp.layers.0.eh_proj.weight"].std()) == pytest.approx(0.02, rel=0.2)
    assert any("cold-initialised" in l for l in lines)
    # wrong vocabulary / missing tensor
    ck3 = dict(ck2)
    ck3["embedding.word_embeddings.weight"] = torch.zeros(spec.vocab_size + 8, spec.hidden_size)
    torch.save(ck3, tmp_path / mg.PARAMS_FILE)
    with pytest.raises(ValueError, match="vocab_size"):
        mg.load_megatron_checkpoint(tmp_path, spec, log=lambda *_: None)
    ck4 = {k: v for k, v in ck2.items() if "layers.1.mlp.linear_fc2" not in k}
    torch.save(ck4, tmp_path / mg.PARAMS_FILE)
    with pytest.raises(KeyError):
        mg.load_megatron_checkpoint(tmp_path, spec, log=lambda *_: None)


def test_optimizer_state_rules(tmp_path):
    assert mg.load_megatron_optimizer_state(tmp_path) is None
    t = {"a": torch.ones(3, dtype=torch.float64)}
    torch.save({"master_weights": t, "exp_avg": t, "exp_avg_sq": t, "step_count": 7,
                "num_samples": -1}, tmp_path / mg.OPTIM_FILE)
    st = mg.load_megatron_optimizer_state(tmp_path, log=lambda *_: None)
    assert st["step_count"] == 7 and st["num_samples"] == 0
    assert st["exp_avg"]["a"].dtype == torch.float32
    torch.save({"master_weights": t}, tmp_path / mg.OPTIM_FILE)
    with pytest.raises(ValueError, match="required keys"):
        mg.load_megatron_optimizer_state(tmp_path)


def test_trainer_starts_from_a_megatron_export(tmp_path):
    """``Trainer.load`` of a Megatron root: parameters land in the flat buffer, the Adam state
    (by Megatron keys) is taken over with its step count."""
    from forgetrain_b200.engine_config import from_spec
    from forgetrain_b200.parallel.topology import Topology
    from forgetrain_b200.trainer import Trainer
    spec = load_model_spec("tiny")
    ck, ours = _export(spec, True, seed=3)
    ck = {k: v * 0.02 for k, v in ck.items()}
    torch.save(ck, tmp_path / mg.PARAMS_FILE)
    mom = {k: torch.full_like(v, 1e-3) for k, v in ck.items()}
    torch.save({"master_weights": ck, "exp_avg": mom, "exp_avg_sq": {k: v * v for k, v in mom.items()},
                "step_count": 11, "num_samples": 44}, tmp_path / mg.OPTIM_FILE)
    cfg = from_spec(spec, dtype="fp32", comm="nccl", warmup_iters=0)
    tr = Trainer(spec, cfg, Topology(device=torch.device("cpu")), seq_length=32, micro_batch_size=2, seed=0)
    state = tr.load(tmp_path)
    assert state["step"] == 0 and tr.opt.step_count == 11 and tr.num_samples == 44
    w = tr.store.params["layers.1.attention.wqkv.weight"]
    assert torch.allclose(w, ck["decoder.layers.1.self_attention.linear_qkv.weight"])
    full = tr.opt.gather_full_state()
    assert torch.allclose(full["exp_avg"]["layers.0.feed_forward.w2.weight"],
                          torch.full_like(full["exp_avg"]["layers.0.feed_forward.w2.weight"], 1e-3))
    tok = torch.randint(0, spec.vocab_size, (2, 33))
    out = tr.train_step([{"tokens": tok[:, :-1].contiguous(), "labels": tok[:, 1:].contiguous()}])
    assert torch.isfinite(out["loss"]).all() and tr.opt.step_count == 12
