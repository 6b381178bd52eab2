"""Job launcher: stage selection, validation, and the command it builds
(behaviour of the reference's scripts/entry_train.sh:274-455 and entry_hf_pretrain.sh)."""
import subprocess
import sys

import pytest

from forgetrain_b200 import launch


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
