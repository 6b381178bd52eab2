import os
import threading

import pytest
import torch

from forgetrain_b200.ckpt import checkpoint as ck


def _payload():
    return dict(params={"a": torch.randn(4, 4), "b": torch.ones(3)}, param_names=["a", "b"],
                optimizer_state={"master_weights": {"a": torch.zeros(4, 4)}, "exp_avg": {}, "exp_avg_sq": {},
                                 "step_count": 7, "num_samples": 70}, num_samples=70,
                dataloader_state={"kind": "synthetic", "batches_drawn": 3})


def test_roundtrip_and_layout(tmp_path):
    p = ck.save_checkpoint(tmp_path, 12, async_io=False, **_payload())
    assert p == tmp_path / "step_0000012" / "training_state.pt"
    st = ck.load_resume_checkpoint(tmp_path)
    assert st["format_version"] == 1 and st["step"] == 12 and st["num_samples"] == 70
    assert st["param_names"] == ["a", "b"]
    assert set(st["optimizer_state"]) >= {"master_weights", "exp_avg", "exp_avg_sq", "step_count", "num_samples"}
    assert st["dataloader_state"]["batches_drawn"] == 3
    assert not list(tmp_path.rglob("*.tmp"))


def test_async_write_and_auto_wait(tmp_path):
    ck.save_checkpoint(tmp_path, 1, async_io=True, **_payload())
    ck.save_checkpoint(tmp_path, 2, async_io=True, **_payload())   # waits for the first
    ck.wait_for_async_save()
    assert (tmp_path / "step_0000001" / "training_state.pt").exists()
    assert ck.latest_checkpoint(tmp_path).parent.name == "step_0000002"


def test_nonzero_rank_is_noop(tmp_path):
    assert ck.save_checkpoint(tmp_path, 1, rank=1, async_io=False, **_payload()) is None
    assert not any(tmp_path.iterdir())


def test_async_error_is_reraised_and_tmp_removed(tmp_path, monkeypatch):
    def boom(obj, f, *a, **k):
        open(f, "wb").write(b"partial")
        raise OSError("disk full")
    monkeypatch.setattr(torch, "save", boom)
    ck.save_checkpoint(tmp_path, 3, async_io=True, **_payload())
    with pytest.raises(RuntimeError, match="disk full"):
        ck.wait_for_async_save()
    assert not list(tmp_path.rglob("*.tmp"))
    assert not (tmp_path / "step_0000003" / "training_state.pt").exists()
    ck.wait_for_async_save()   # error slot is cleared


def test_corrupt_or_wrong_version_rejected(tmp_path):
    d = tmp_path / "step_0000001"
    d.mkdir()
    (d / "training_state.pt").write_bytes(b"not a checkpoint")
    with pytest.raises(Exception):
        ck.load_resume_checkpoint(tmp_path)
    torch.save({"format_version": 99, "params": {}}, d / "training_state.pt")
    with pytest.raises(ValueError, match="format_version"):
        ck.load_resume_checkpoint(d)
    torch.save({"format_version": 1, "params": {"tok_embeddings.weight": torch.zeros(10, 4)}},
               d / "training_state.pt")
    with pytest.raises(ValueError, match="vocabulary"):
        ck.load_resume_checkpoint(d, expected_vocab=11)


def test_save_boundary_policy():
    f = ck.should_save_after_step
    assert not f(0, 10, 2)
    assert f(2, 10, 2) and not f(3, 10, 2) and f(10, 10, 0) and f(10, 10, 3)
    assert not f(5, 10, 0)
    assert not f(4, 10, 2, start_step=4)


def test_async_save_snapshots_host_tensors(tmp_path, monkeypatch):
    """The writer thread must own its data: parameters that already live on the host are cloned
    on the caller's thread, so a training step that runs while the file is being written cannot
    leak into the checkpoint."""
    import threading
    import torch
    gate = threading.Event()
    real = ck._write_atomic

    def slow_write(payload, path):
        gate.wait(10)                       # hold the writer until the caller has changed the tensor
        real(payload, path)

    monkeypatch.setattr(ck, "_write_atomic", slow_write)
    w = torch.zeros(8)
    ck.save_checkpoint(tmp_path, 1, params={"w": w}, param_names=["w"], optimizer_state=None,
                       async_io=True)
    w.fill_(7.0)                            # "the next training step"
    gate.set()
    ck.wait_for_async_save()
    st = ck.load_resume_checkpoint(tmp_path / "step_0000001")
    assert float(st["params"]["w"].sum()) == 0.0


# ---------------------------------------------------------------------------------------------
# loading named tensors into a model: what is accepted, what is refused
# ---------------------------------------------------------------------------------------------
def _store(**kw):
    from forgetrain_b200.config import load_model_spec
    from forgetrain_b200.models.params import ParamStore
    base = dict(num_layers=2, vocab_size=128, hidden_size=128, ffn_hidden_size=256, num_attention_heads=4,
                num_query_groups=2, head_dim=32)
    mtp = kw.pop("mtp", 0)
    base.update(kw)
    st = ParamStore(load_model_spec("tiny", **base), "cpu", torch.float32, mtp_num_layers=mtp)
    st.init_random(1)
    return st


def test_a_checkpoint_of_another_architecture_is_refused_by_name():
    big, small = _store(num_layers=3, tie_embeddings=False), _store(tie_embeddings=False)
    tensors = big.named_cpu_params()
    with pytest.raises(ValueError, match=r"6 tensors this model has no parameter for \(layers\.2\."):
        small.load_named(tensors)
    with pytest.raises(KeyError, match=r"lacks 6 parameters of this model \(layers\.2\."):
        big.load_named(small.named_cpu_params())
    wide = _store(ffn_hidden_size=512, tie_embeddings=False).named_cpu_params()
    with pytest.raises(ValueError, match=r"feed_forward\.wfc1\.weight: the checkpoint holds \(1024, 128\), this model needs \(512, 128\)"):
        small.load_named(wide)
    # a refused checkpoint leaves the model as it was, also when the misfit is its last tensor
    before = small.flat_params.clone()
    odd = {n: t * 2 for n, t in _store(tie_embeddings=False).named_cpu_params().items()}
    odd["tok_embeddings.weight"] = torch.zeros(64, 128)
    with pytest.raises(ValueError, match="tok_embeddings.weight"):
        small.load_named(odd)
    assert torch.equal(small.flat_params, before)


def test_tied_checkpoint_into_untied_run_and_plain_checkpoint_into_mtp_run():
    tied, untied = _store(tie_embeddings=True), _store(tie_embeddings=False)
    notes = []
    untied.load_named(tied.named_cpu_params(), log=notes.append)
    assert torch.equal(untied.params["output.weight"], tied.params["tok_embeddings.weight"])
    assert len(notes) == 1 and "output.weight starts as its copy" in notes[0]
    # the other way would throw the trained output table away
    with pytest.raises(ValueError, match="output.weight"):
        tied.load_named(untied.named_cpu_params())
    # an MTP run started from a plain checkpoint keeps its freshly initialised head ...
    mtp = _store(tie_embeddings=False, mtp=1)
    head = mtp.params["mtp.layers.0.eh_proj.weight"].clone()
    mtp.load_named(untied.named_cpu_params(), keep_missing=("mtp.",))
    assert torch.equal(mtp.params["mtp.layers.0.eh_proj.weight"], head)
    assert torch.equal(mtp.params["layers.1.attention.wo.weight"], untied.params["layers.1.attention.wo.weight"])
    # ... and without the permission the missing head is an error
    with pytest.raises(KeyError, match="mtp.layers.0"):
        mtp.load_named(untied.named_cpu_params())
    # a plain run drops the head of an MTP checkpoint, and says so
    notes.clear()
    untied.load_named(mtp.named_cpu_params(), log=notes.append)
    assert notes == ["the checkpoint's MTP head is not used by this run and is dropped"]


def test_optimizer_state_without_a_parameter_starts_that_parameter_fresh():
    from forgetrain_b200.optim.adamw import ShardedAdamW
    from forgetrain_b200.parallel.buckets import compute_grad_buckets
    tied, untied = _store(tie_embeddings=True), _store(tie_embeddings=False)
    a = ShardedAdamW(tied, compute_grad_buckets(tied.entries(), 1, 10 ** 9), 1, 0, None)
    tied.flat_grads.normal_()
    a.compute_clip(tied.flat_grads.pow(2).sum().reshape(1))
    a.step(1e-3)
    state = a.gather_full_state()
    untied.load_named(tied.named_cpu_params())
    b = ShardedAdamW(untied, compute_grad_buckets(untied.entries(), 1, 10 ** 9), 1, 0, None)
    b.load_full_state(state, 1)
    got = b.gather_full_state()
    assert torch.equal(got["exp_avg"]["layers.0.attention.wo.weight"], state["exp_avg"]["layers.0.attention.wo.weight"])
    assert not got["exp_avg"]["output.weight"].any() and not got["exp_avg_sq"]["output.weight"].any()
    assert torch.equal(got["master_weights"]["output.weight"], untied.params["output.weight"])
    assert b.step_count == 1
