"""The plumbing configuration, launched the way a user launches it: two ranks on CPU (gloo) through
``python -m torch.distributed.run ... -m training_engine_tensor pretrain`` with the tiny
MiniCPM4-style decoder (4 layers, hidden 256, 4 query / 2 KV heads of 64, SwiGLU 1024, vocabulary
4096, tied tables, muP scales), sequence 256, micro-batch 2, global batch 4, fp32, AdamW 1e-3,
uniform token ids from seed 0. Five steps: the loss falls; the checkpoint written after step 5
resumes into exactly the run that was never interrupted."""
import re
import socket
import subprocess
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent


def _port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _run(command: str, steps: int, *extra: str, ranks: int = 2, mesh: str = "world=2 dp=2 tp=1") -> dict[int, float]:
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", str(ranks),
           "--master-addr", "127.0.0.1", "--master-port", str(_port()),
           "-m", "training_engine_tensor", command, "--model", "tiny", "--device", "cpu", "--dtype", "fp32",
           "--num-steps", str(steps), "--global-batch-size", "4", "--micro-batch-size", "2",
           "--seq-length", "256", "--seed", "0", "--max-lr", "1e-3", "--tie-embeddings", *extra]
    r = subprocess.run(cmd, cwd=ROOT, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    assert mesh in r.stdout and "DONE" in r.stdout
    return {int(m.group(1)): float(m.group(2))
            for m in re.finditer(r"iteration +(\d+) \| loss ([0-9.E+-]+)", r.stdout)}


def test_two_cpu_ranks_train_save_and_resume_bit_for_bit(tmp_path):
    run = tmp_path / "run"
    first = _run("pretrain", 5, "--save-dir", str(run), "--save-interval", "5")
    assert sorted(first) == [1, 2, 3, 4, 5]
    # fresh uniform tokens every step: the loss can only fall towards ln(4096) = 8.318
    assert 8.25 < min(first.values()) and (first[4] + first[5]) / 2 < first[1] < 8.6
    assert (run / "step_0000005" / "training_state.pt").exists()
    resumed = _run("train", 2, "--resume", str(run / "step_0000005"), "--save-dir", str(run))
    whole = _run("pretrain", 7)
    assert sorted(resumed) == [6, 7]
    assert {k: whole[k] for k in (1, 2, 3, 4, 5)} == first
    assert resumed == {6: whole[6], 7: whole[7]}
    assert (run / "step_0000007" / "training_state.pt").exists()


def test_four_cpu_ranks_tensor_parallel_match_data_parallel_and_their_checkpoint_moves(tmp_path):
    """The same run as TP=2 x DP=2 (sequence-parallel activations, vocabulary-parallel tables and
    loss) follows the DP=2 losses to fp32 summation order; its per-rank shard files resume on two
    ranks without tensor parallelism into the data-parallel run's next step."""
    run = tmp_path / "tp"
    tp = _run("pretrain", 3, "--tensor-parallel-size", "2", "--sequence-parallel", "--save-dir", str(run),
              "--save-interval", "3", ranks=4, mesh="world=4 dp=2 tp=2")
    dp = _run("pretrain", 4)
    for k in (1, 2, 3):
        assert abs(tp[k] - dp[k]) < 5e-6 * dp[k], (k, tp[k], dp[k])
    assert sorted(p.name for p in (run / "step_0000003").glob("rank_*.pt")) == ["rank_0.pt", "rank_1.pt"]
    moved = _run("train", 1, "--resume", str(run / "step_0000003"))
    assert abs(moved[4] - dp[4]) < 5e-6 * dp[4]
