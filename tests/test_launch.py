"""Job launcher: stage selection, validation, and the command it builds
(behaviour of the reference's scripts/entry_train.sh:274-455 and entry_hf_pretrain.sh)."""
import os
import subprocess
import sys
from pathlib import Path

import pytest

from forgetrain_b200 import launch

ROOT = Path(__file__).resolve().parent.parent


def _plan(env, **kw):
    return launch.plan_from_env(env, nproc_per_node=kw.pop("nproc", 8), repo_root="/job", **kw)


def test_stable_stage_is_random_init_pretrain():
    p = _plan({"STAGE": "stable", "HF_DATASET": "ds", "TOKENIZER_PATH": "tok", "RESUME_DIR": "/stale",
               "CHECKPOINT_ROOT": "/stale2", "NUM_STEPS": "10", "MAX_LR": "1e-2"})
    assert p.subcommand == "pretrain" and p.child_env["RANDOM_INIT"] == "1"
    a = list(p.cli_args)
    assert "--resume" not in a and "--checkpoint-root" not in a
    assert a[a.index("--num-steps") + 1] == "10" and a[a.index("--max-lr") + 1] == "1e-2"
    assert a[a.index("--save-dir") + 1] == "/job/.checkpoints/stable"
    assert a[a.index("--save-interval") + 1] == "5000"


@pytest.mark.parametrize("stage", ["stable_2", "decay_from_ours"])
def test_resume_stages_need_resume_dir(stage):
    with pytest.raises(launch.LaunchError, match="RESUME_DIR"):
        _plan({"STAGE": stage, "HF_DATASET": "ds"})
    p = _plan({"STAGE": stage, "HF_DATASET": "ds", "RESUME_DIR": "/prev/step_0000100"})
    a = list(p.cli_args)
    assert p.subcommand == "train" and a[a.index("--resume") + 1] == "/prev/step_0000100"
    assert "--checkpoint-root" not in a


def test_decay_from_megatron_default_and_alias():
    with pytest.raises(launch.LaunchError, match="CHECKPOINT_ROOT"):
        _plan({"HF_DATASET": "ds"})
    for stage in (None, "decay", "decay_from_megatron"):
        env = {"HF_DATASET": "ds", "CHECKPOINT_ROOT": "/mg", "MTP_NUM_LAYERS": "1"}
        if stage:
            env["STAGE"] = stage
        p = _plan(env)
        a = list(p.cli_args)
        assert p.stage == "decay_from_megatron" and a[a.index("--checkpoint-root") + 1] == "/mg"
        assert a[a.index("--mtp-num-layers") + 1] == "1"
        assert a[a.index("--mtp-loss-scaling-factor") + 1] == "0.1"


def test_validation_errors():
    with pytest.raises(launch.LaunchError, match="unknown STAGE"):
        _plan({"STAGE": "warm", "HF_DATASET": "ds"})
    with pytest.raises(launch.LaunchError, match="HF_DATASET"):
        _plan({"STAGE": "stable"})
    with pytest.raises(launch.LaunchError, match="must differ"):
        _plan({"STAGE": "stable_2", "HF_DATASET": "d", "RESUME_DIR": "/a/b", "SAVE_DIR": "/a/b"})
    with pytest.raises(launch.LaunchError, match="node rank"):
        _plan({"STAGE": "stable", "HF_DATASET": "d", "WORLD_SIZE": "2", "RANK": "2"})
    assert _plan({"STAGE": "stable", "SYNTHETIC_DATA": "1"}).subcommand == "pretrain"


def test_node_topology_and_command():
    p = _plan({"STAGE": "hf_pretrain", "HF_DATASET": "ds", "WORLD_SIZE": "8", "RANK": "3",
               "MASTER_ADDR": "10.0.0.1", "MASTER_PORT": "23456", "HF_TEXT_FIELD": "question answer",
               "MODEL": "8b", "TENSOR_PARALLEL_SIZE": "2", "CUDA_DEVICE_MAX_CONNECTIONS": "4"},
              extra_args=("--no-sequence-parallel",))
    assert (p.nnodes, p.node_rank, p.nproc_per_node) == (8, 3, 8)
    cmd = p.command("py")
    assert cmd[:3] == ["py", "-m", "torch.distributed.run"]
    assert "--nnodes=8" in cmd and "--node-rank=3" in cmd and "--master-addr=10.0.0.1" in cmd
    i = cmd.index("forgetrain_b200")
    assert cmd[i + 1] == "pretrain" and cmd[-1] == "--no-sequence-parallel"
    a = list(p.cli_args)
    assert a[a.index("--hf-text-field") + 1:a.index("--hf-text-field") + 3] == ["question", "answer"]
    assert "--save-dir" not in a and a[a.index("--model") + 1] == "8b"
    assert "CUDA_DEVICE_MAX_CONNECTIONS" not in p.child_env      # the job's own value wins
    # the flags the plan emits are flags the training CLI knows
    from forgetrain_b200.cli import build_parser
    ns = build_parser().parse_args([p.subcommand, *p.cli_args])
    assert ns.hf_text_field == ["question", "answer"] and ns.cfg_tensor_parallel_size == 2


def test_dry_run_exit_codes():
    import os
    env = {k: v for k, v in os.environ.items() if k not in ("STAGE", "HF_DATASET", "RANK", "WORLD_SIZE")}
    r = subprocess.run([sys.executable, "-m", "forgetrain_b200.launch", "--dry-run", "--nproc-per-node", "2"],
                       env={**env, "STAGE": "stable", "SYNTHETIC_DATA": "1"}, capture_output=True, text=True)
    assert r.returncode == 0 and "torch.distributed.run" in r.stdout and "--nproc-per-node=2" in r.stdout
    r = subprocess.run([sys.executable, "-m", "forgetrain_b200.launch", "--dry-run"],
                       env={**env, "STAGE": "stable_2", "HF_DATASET": "x"}, capture_output=True, text=True)
    assert r.returncode == 2 and "RESUME_DIR" in r.stderr


def test_bundled_job_specs_give_valid_plans():
    """Every spec under forgetrain_b200/job_specs launches: its variables pass the stage validation
    and every flag the plan emits is one the training CLI parses (the reference checks its own
    specs in tests/test_job_specs.py)."""
    import json
    from pathlib import Path
    from forgetrain_b200.cli import build_parser
    root = Path(launch.__file__).parent / "job_specs"
    files = sorted(root.glob("*.json"))
    assert len(files) >= 4
    for f in files:
        task = json.loads(f.read_text())["task"]
        assert task["resources"]["gpuCount"] == 8 and task["resources"]["gpuModel"] == "b200"
        assert "replicas" not in task                    # single-node examples
        env = launch.env_from_job_spec(str(f), {"HOME": "/home/u"})
        assert all("${HOME}" not in v for v in env.values())
        plan = launch.plan_from_env(env, repo_root="/job")
        assert plan.nproc_per_node == 8
        ns = build_parser().parse_args([plan.subcommand, *plan.cli_args])
        assert ns.global_batch_size % ns.micro_batch_size == 0
        if "8b" in f.name:
            assert ns.cfg_tensor_parallel_size == 2 and ns.grad_accum_steps == 8
        if "gsm8k" in f.name:
            assert ns.hf_text_template == "Question: {question}\nAnswer: {answer}"
            assert "--save-dir" not in plan.cli_args


# ---------------------------------------------------------------------------------------------
# recovery: AUTO_RESUME / MAX_RESTARTS
# ---------------------------------------------------------------------------------------------
def _finished(save_dir, step, name="training_state.pt"):
    d = save_dir / f"step_{step:07d}"
    d.mkdir(parents=True, exist_ok=True)
    (d / name).write_bytes(b"x")
    return d


def test_auto_resume_continues_from_the_newest_finished_checkpoint(tmp_path):
    from forgetrain_b200.launch import find_restart_point, plan_from_env
    save = tmp_path / "run"
    env = {"STAGE": "stable", "SYNTHETIC_DATA": "1", "SAVE_DIR": str(save), "NUM_STEPS": "10",
           "AUTO_RESUME": "1", "NPROC_PER_NODE": "2"}
    fresh = plan_from_env(env)
    assert fresh.subcommand == "pretrain" and "--resume" not in fresh.cli_args      # nothing to resume yet
    assert find_restart_point(str(save)) is None
    _finished(save, 2)
    _finished(save, 6)
    (save / "step_0000008").mkdir()                                    # the writer never finished this one
    (save / "step_0000008" / "training_state.pt.tmp").write_bytes(b"half")
    assert find_restart_point(str(save)) == (6, str(save / "step_0000006"))
    plan = plan_from_env(env)
    args = list(plan.cli_args)
    assert plan.subcommand == "train"
    assert args[args.index("--resume") + 1] == str(save / "step_0000006")
    assert args[args.index("--num-steps") + 1] == "4"                   # 10 in all, 6 done
    assert args[args.index("--save-dir") + 1] == str(save)
    # tensor-parallel shard files count as a finished checkpoint too, and the newest of both kinds wins
    _finished(save, 7, "rank_0.pt")
    assert find_restart_point(str(save))[0] == 7
    # off by default
    off = plan_from_env({**env, "AUTO_RESUME": "0"})
    assert off.subcommand == "pretrain" and "--resume" not in off.cli_args
    # a Megatron start is replaced as well: the job's own checkpoint has everything
    mg = plan_from_env({**env, "STAGE": "decay_from_megatron", "CHECKPOINT_ROOT": "/ckpt/mg"})
    assert "--checkpoint-root" not in mg.cli_args and "--resume" in mg.cli_args


def test_supervisor_restarts_a_failed_job_with_fewer_steps_and_gives_up_after_the_limit(tmp_path):
    from forgetrain_b200 import launch
    save = tmp_path / "run"
    env = {"STAGE": "stable", "SYNTHETIC_DATA": "1", "SAVE_DIR": str(save), "NUM_STEPS": "6",
           "NPROC_PER_NODE": "2"}
    calls = []

    def run_fails_once(cmd, child_env):
        calls.append(list(cmd))
        if len(calls) == 1:
            _finished(save, 4)                     # got as far as step 4, then died
            return 1
        return 0
    plan = launch.plan_from_env(env)
    rc = launch.supervise(plan, env, None, (), 2, lambda pl: dict(env), run=run_fails_once)
    assert rc == 0 and len(calls) == 2
    assert "pretrain" in calls[0] and "--resume" not in calls[0]
    second = calls[1]
    assert "train" in second and second[second.index("--resume") + 1] == str(save / "step_0000004")
    assert second[second.index("--num-steps") + 1] == "2"

    calls.clear()
    rc = launch.supervise(launch.plan_from_env(env), env, None, (), 2, lambda pl: dict(env),
                          run=lambda cmd, e: calls.append(cmd) or 3)
    assert rc == 3 and len(calls) == 3              # the first attempt and two restarts

    # a job whose newest checkpoint is already the last step has nothing left to run
    _finished(save, 6)
    calls.clear()
    done = launch.plan_from_env({**env, "AUTO_RESUME": "1"})
    assert launch.supervise(done, env, None, (), 2, lambda pl: dict(env),
                            run=lambda cmd, e: calls.append(cmd) or 0) == 0
    assert calls == []


def test_fault_injection_spec_and_once_marker(tmp_path):
    from forgetrain_b200.utils.fault_injection import InjectedFailure, maybe_fail, parse
    assert parse(None) is None and parse("") is None
    assert parse("step=3") == {"step": 3, "rank": 0, "once": None, "exit": None}
    assert parse("step=3, rank=1, once=/x/y")["once"] == "/x/y"
    for bad in ("rank=1", "step", "step=3,when=now"):
        with pytest.raises(ValueError):
            parse(bad)
    marker = tmp_path / "m"
    env = {"FT_INJECT_FAILURE": f"step=3,rank=1,once={marker}"}
    maybe_fail(2, 1, env)                           # another step
    maybe_fail(3, 0, env)                           # another rank
    assert not marker.exists()
    with pytest.raises(InjectedFailure, match="before step 3 on rank 1"):
        maybe_fail(3, 1, env)
    assert marker.exists()
    maybe_fail(3, 1, env)                           # the relaunched job passes the same step
    maybe_fail(3, 1, {})                            # no variable: nothing happens


def test_a_rank_that_fails_mid_run_is_recovered_by_the_launcher_and_the_run_ends_identical(tmp_path):
    """Two CPU ranks, a host-side failure of rank 1 right before step 5 of 6: the launcher sees the
    failed attempt, resumes from the step-4 checkpoint for the two remaining steps, and the final
    checkpoint equals that of a run that was never interrupted."""
    import socket
    import torch

    def port():
        with socket.socket() as s:
            s.bind(("127.0.0.1", 0))
            return s.getsockname()[1]

    def job(save, **more):
        env = dict(os.environ)
        env.update({"STAGE": "stable", "SYNTHETIC_DATA": "1", "MODEL": "tiny", "NUM_STEPS": "6",
                    "GLOBAL_BATCH_SIZE": "4", "MICRO_BATCH_SIZE": "2", "SEQ_LENGTH": "64", "SEED": "0",
                    "SAVE_DIR": str(save), "SAVE_INTERVAL": "2", "NPROC_PER_NODE": "2",
                    "MASTER_ADDR": "127.0.0.1", "MASTER_PORT": str(port())})
        env.pop("RANK", None)
        env.pop("WORLD_SIZE", None)
        env.update(more)
        return subprocess.run([sys.executable, "-m", "forgetrain_b200.launch", "--", "--device", "cpu",
                               "--dtype", "fp32"], cwd=ROOT, env=env, capture_output=True, text=True,
                              timeout=600)

    marker = tmp_path / "failed_once"
    r = job(tmp_path / "a", MAX_RESTARTS="2", FT_INJECT_FAILURE=f"step=5,rank=1,once={marker}")
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    assert marker.exists() and "attempt 1 of 2" in r.stdout and "attempt 2 of 2" not in r.stdout
    assert "injected failure before step 5 on rank 1" in r.stdout + r.stderr
    assert f"resumed from {tmp_path / 'a' / 'step_0000004'} at step 4" in r.stdout
    whole = job(tmp_path / "b")
    assert whole.returncode == 0, whole.stdout[-3000:] + whole.stderr[-3000:]
    a = torch.load(tmp_path / "a" / "step_0000006" / "training_state.pt", weights_only=False)
    b = torch.load(tmp_path / "b" / "step_0000006" / "training_state.pt", weights_only=False)
    assert a["step"] == b["step"] == 6
    for name in b["params"]:
        assert torch.equal(a["params"][name], b["params"][name]), name
    for name in b["optimizer_state"]["exp_avg_sq"]:
        assert torch.equal(a["optimizer_state"]["exp_avg_sq"][name], b["optimizer_state"]["exp_avg_sq"][name])


def test_a_stop_signal_to_the_supervising_launcher_reaches_the_ranks_and_is_not_followed_by_a_restart(tmp_path):
    """SIGTERM to the launcher (what a scheduler sends before it takes the node away): it is passed
    on to ``torch.distributed.run`` and from there to both ranks, which agree on a step, write its
    checkpoint and leave; the launcher does not start the job again although restarts are allowed.
    A relaunch with ``AUTO_RESUME`` then continues from that step."""
    import re
    import signal
    import socket
    import time
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    env = dict(os.environ)
    env.update({"STAGE": "stable", "SYNTHETIC_DATA": "1", "MODEL": "tiny", "NUM_STEPS": "400",
                "GLOBAL_BATCH_SIZE": "4", "MICRO_BATCH_SIZE": "2", "SEQ_LENGTH": "64", "SEED": "0",
                "SAVE_DIR": str(tmp_path / "run"), "SAVE_INTERVAL": "1000", "NPROC_PER_NODE": "2",
                "MASTER_ADDR": "127.0.0.1", "MASTER_PORT": str(port), "MAX_RESTARTS": "3",
                "PYTHONUNBUFFERED": "1"})
    env.pop("RANK", None)
    env.pop("WORLD_SIZE", None)
    p = subprocess.Popen([sys.executable, "-u", "-m", "forgetrain_b200.launch", "--", "--device", "cpu",
                          "--dtype", "fp32"], cwd=ROOT, env=env, stdout=subprocess.PIPE,
                         stderr=subprocess.STDOUT, text=True)
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
    m = re.search(r"\[signal\] stop requested: checkpoint written at step (\d+) of 400", out)
    assert m, out[-3000:]
    stopped = int(m.group(1))
    assert (tmp_path / "run" / f"step_{stopped:07d}" / "training_state.pt").exists()
    assert "attempt 1 of 3" not in out                      # a requested stop is not a failure to retry
    plan = launch.plan_from_env({**env, "AUTO_RESUME": "1"})
    args = list(plan.cli_args)
    assert args[args.index("--resume") + 1] == str(tmp_path / "run" / f"step_{stopped:07d}")
    assert args[args.index("--num-steps") + 1] == str(400 - stopped)
