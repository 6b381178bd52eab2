"""Failure handling, exercised on the host: a rank that dies, a rank that never joins, a
collective that times out, a checkpoint writer that fails. No GPU is involved."""
import os
import sys
import time

import pytest
import torch

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
from dist_util import run_ranks  # noqa: E402


def _rank_raises(rank, world):
    import datetime
    import torch.distributed as dist
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=5))
    t = torch.ones(4)
    dist.all_reduce(t)                       # healthy step
    if rank == 1:
        raise RuntimeError("injected failure on rank 1")
    try:
        dist.all_reduce(t)                   # the peer is gone: must end with an error, not hang
    except Exception as e:  # noqa: BLE001
        return f"collective failed: {type(e).__name__}"
    return "collective unexpectedly succeeded"


def test_a_failing_rank_surfaces_as_an_error_on_every_rank():
    t0 = time.time()
    with pytest.raises(RuntimeError, match="injected failure on rank 1|collective failed"):
        run_ranks(_rank_raises, 2, timeout=120)
    assert time.time() - t0 < 120


def _late_rank(rank, world):
    """Rank 1 never joins the second collective; rank 0's short timeout ends it."""
    import datetime
    import torch.distributed as dist
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=3))
    t = torch.ones(2)
    dist.all_reduce(t)
    if rank == 1:
        time.sleep(8)
        return "absent"
    try:
        dist.all_reduce(t)
        return "no error"
    except Exception as e:  # noqa: BLE001
        return f"timeout: {type(e).__name__}"


def test_missing_rank_ends_the_collective_with_a_timeout():
    res = run_ranks(_late_rank, 2, timeout=120)
    assert res[0].startswith("timeout") and res[1] == "absent"


def test_reducer_detects_a_gradient_that_never_arrives():
    from forgetrain_b200.config import load_model_spec
    from forgetrain_b200.models.params import ParamStore
    from forgetrain_b200.parallel.dp import BucketedGradReducer
    spec = load_model_spec("tiny", num_layers=1, vocab_size=128, hidden_size=128, ffn_hidden_size=256,
                           num_attention_heads=4, num_query_groups=2, head_dim=32, tie_embeddings=False)
    st = ParamStore(spec, "cpu", torch.float32)
    red = BucketedGradReducer(st.flat_grads, st.entries(), 1, 0, None, 10 ** 9)
    red.start_step()
    for ps in st.order[:-1]:                 # the embedding's gradient is "lost"
        red.on_grad_ready(ps.name)
    with pytest.raises(RuntimeError, match="never became ready"):
        red.wait_all()


def test_truncated_checkpoint_is_rejected(tmp_path):
    from forgetrain_b200.ckpt import checkpoint as ck
    p = ck.save_checkpoint(tmp_path, 1, params={"a": torch.randn(64, 64)}, param_names=["a"],
                           optimizer_state=None, async_io=False)
    data = p.read_bytes()
    p.write_bytes(data[: len(data) // 2])
    with pytest.raises(Exception):
        ck.load_resume_checkpoint(tmp_path)


def test_status_word_codes_have_messages():
    from forgetrain_b200.ops import _lib
    assert set(_lib.STATUS_MESSAGES) == {1, 2, 3, 4, 5, 6}
    assert "peer" in _lib.STATUS_MESSAGES[5]


def test_sigterm_finishes_the_step_writes_a_checkpoint_and_leaves_normally(tmp_path):
    """A pre-emption notice in the middle of a run: the process is sent SIGTERM once it has logged
    a few iterations; it finishes the step it is in, saves, exits with code 0, and the saved step
    resumes into the same losses as a run that was never interrupted."""
    import re
    import signal
    import subprocess
    import sys
    import time
    from pathlib import Path
    root = Path(__file__).resolve().parent.parent
    base = [sys.executable, "-u", "-m", "training_engine_tensor", "pretrain", "--model", "tiny", "--device", "cpu",
            "--dtype", "fp32", "--micro-batch-size", "2", "--global-batch-size", "2", "--seq-length", "64",
            "--seed", "0"]
    p = subprocess.Popen(base + ["--num-steps", "400", "--save-dir", str(tmp_path / "run")], cwd=root,
                         stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    lines = []
    deadline = time.time() + 300
    while time.time() < deadline:
        line = p.stdout.readline()
        if not line:
            break
        lines.append(line)
        if "iteration        3 " in line:
            p.send_signal(signal.SIGTERM)
            break
    rest, _ = p.communicate(timeout=300)
    out = "".join(lines) + rest
    assert p.returncode == 0, out[-2000:]
    m = re.search(r"\[signal\] stop requested: checkpoint written at step (\d+) of 400", out)
    assert m, out[-2000:]
    stopped = int(m.group(1))
    assert 3 <= stopped < 400 and (tmp_path / "run" / f"step_{stopped:07d}" / "training_state.pt").exists()
    assert f"iteration {stopped + 1:8d} " not in out
    losses = {int(a): float(b) for a, b in re.findall(r"iteration +(\d+) \| loss ([0-9.E+-]+)", out)}
    r = subprocess.run(base[:4] + ["train"] + base[5:] + ["--num-steps", "2", "--resume",
                                                          str(tmp_path / "run" / f"step_{stopped:07d}")],
                       cwd=root, capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    resumed = {int(a): float(b) for a, b in re.findall(r"iteration +(\d+) \| loss ([0-9.E+-]+)", r.stdout)}
    whole = subprocess.run(base + ["--num-steps", str(stopped + 2)], cwd=root, capture_output=True, text=True,
                           timeout=300)
    ref = {int(a): float(b) for a, b in re.findall(r"iteration +(\d+) \| loss ([0-9.E+-]+)", whole.stdout)}
    assert {k: ref[k] for k in losses} == losses
    assert resumed == {stopped + 1: ref[stopped + 1], stopped + 2: ref[stopped + 2]}


def test_stop_request_handlers_are_put_back_also_after_a_loop_that_raised():
    import signal
    from forgetrain_b200.trainer import _StopRequest
    before = signal.getsignal(signal.SIGTERM)
    a = _StopRequest()                      # a loop that raises never calls restore() ...
    assert signal.getsignal(signal.SIGTERM) == a._handler
    b = _StopRequest()                      # ... the next one cleans up after it
    assert a._pair is None and signal.getsignal(signal.SIGTERM) == b._handler
    assert not b.requested
    signal.raise_signal(signal.SIGUSR1)
    assert b.requested and not a.requested
    b.restore()
    assert signal.getsignal(signal.SIGTERM) == before and _StopRequest._live is None


def test_a_non_finite_loss_names_the_tensors_that_hold_the_bad_values():
    import torch
    from forgetrain_b200.config import load_model_spec
    from forgetrain_b200.engine_config import from_spec
    from forgetrain_b200.parallel.topology import Topology
    from forgetrain_b200.trainer import Trainer, run_training_loop
    spec = load_model_spec("tiny", num_layers=2, seq_length=32, max_position_embeddings=32)
    cfg = from_spec(spec, dtype="fp32", comm="nccl")
    tr = Trainer(spec, cfg, Topology(), seq_length=32, micro_batch_size=2, seed=0)
    assert tr.nonfinite_report().startswith("parameters and gradients of this rank are finite")
    tr.store.params["layers.1.attention.wo.weight"][0, :3] = float("nan")
    tr.store.grads["norm.weight"][5] = float("inf")
    rep = tr.nonfinite_report()
    assert "parameter layers.1.attention.wo.weight: 3 of" in rep and "gradient norm.weight: 1 of" in rep

    class Poisoned:
        """A source whose very first batch makes the loss NaN through a poisoned label mask."""
        def __iter__(self):
            return self

        def __next__(self):
            c = torch.randint(0, spec.vocab_size, (2, 33))
            return {"tokens": c[:, :-1].contiguous(), "labels": c[:, 1:].contiguous(),
                    "loss_mask": torch.full((2, 32), float("nan"))}

    with pytest.raises(FloatingPointError, match=r"non-finite loss at step 1; .*(finite|non-finite values in)"):
        run_training_loop(spec=spec, cfg=cfg, topo=Topology(), num_steps=2, micro_batch_size=2, seq_length=32,
                          data_source=Poisoned())
