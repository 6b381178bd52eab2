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
