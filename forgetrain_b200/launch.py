"""Job launcher: environment variables of a cluster job -> one ``torch.distributed.run`` command.

``python -m forgetrain_b200.launch [--dry-run] [--job-spec FILE] [--nproc-per-node N] [-- extra CLI args]``

The reference drives its production runs through shell entry scripts that read the job's
environment, pick a training *stage* and exec ``torchrun -m training_engine_tensor <cmd> ...``
(0.5B ``scripts/entry_train.sh:274-455``, ``scripts/entry_hf_pretrain.sh``). This module keeps that
contract (same variable names, same stage names, same validation and exit code 2 on a bad
combination) as testable Python: :func:`plan_from_env` is a pure function from a dict to a
:class:`LaunchPlan`, and ``main`` either prints the plan (``--dry-run``) or replaces the process
with the launcher.

Stages
------
``stable``               random init, ``pretrain`` (no checkpoint root, no resume).
``stable_2``             continue from a save directory of this engine: ``train --resume``.
``decay_from_ours``      same mechanics as ``stable_2`` (the schedule differs by ``WSD_DECAY_ITERS``).
``decay_from_megatron``  ``train --checkpoint-root <dir with canonical_state_fp32.pt>``; ``RESUME_DIR``
                         optional (restart after a crash). ``decay`` is an alias.
``hf_pretrain``          the short HF-dataset pretrain of ``entry_hf_pretrain.sh``: ``pretrain`` with
                         no periodic saves unless ``SAVE_DIR`` is given.

Recovery
--------
``AUTO_RESUME=1``   when ``SAVE_DIR`` already holds a finished checkpoint (a ``step_<N>`` directory
                    with ``training_state.pt`` or ``rank_<R>.pt`` files), the job continues from
                    the newest one whatever the stage says: ``train --resume SAVE_DIR/step_<N>``
                    with ``NUM_STEPS`` reduced by N, so that a relaunched job ends where the
                    original one would have.
``MAX_RESTARTS=K``  the launcher stays in front of ``torch.distributed.run`` and, when it exits with
                    an error, starts it again (at most K times) with ``AUTO_RESUME`` on. A SIGTERM
                    sent to the launcher is passed on to the job (whose ranks finish their step,
                    write a checkpoint and leave) and is not followed by a restart. On several
                    nodes every node runs its own launcher: when one node's ranks fail, the other
                    nodes' ranks lose their peers, fail too, and all launchers meet again at the
                    rendezvous of the next attempt (``SAVE_DIR`` must be storage every node sees). The
                    reference has no recovery of its own (a failed job is resubmitted by hand with
                    ``RESUME_DIR``); this is that resubmission, automated.

Node topology follows the PyTorchJob convention the reference's scripts rely on: ``WORLD_SIZE`` is
the number of nodes and ``RANK`` the node rank *of the launcher's own environment*; the launcher
then gives every worker its global rank.
"""
from __future__ import annotations

import argparse
import dataclasses
import os
import shlex
import sys

STAGES = ("stable", "stable_2", "decay_from_megatron", "decay_from_ours", "hf_pretrain")
_STAGE_ALIASES = {"decay": "decay_from_megatron"}


class LaunchError(ValueError):
    """A combination of stage and variables that cannot be launched (exit code 2)."""


@dataclasses.dataclass(frozen=True)
class LaunchPlan:
    stage: str
    subcommand: str
    nnodes: int
    node_rank: int
    nproc_per_node: int
    master_addr: str
    master_port: int
    cli_args: tuple[str, ...]
    child_env: dict

    def command(self, python: str = sys.executable) -> list[str]:
        return [python, "-m", "torch.distributed.run",
                f"--nproc-per-node={self.nproc_per_node}", f"--nnodes={self.nnodes}",
                f"--node-rank={self.node_rank}", f"--master-addr={self.master_addr}",
                f"--master-port={self.master_port}",
                "-m", "forgetrain_b200", self.subcommand, *self.cli_args]


# variables forwarded as ``--flag value`` when set: (env name, flag, default or None)
_VALUE_FLAGS = (
    ("NUM_STEPS", "--num-steps", None),
    ("GLOBAL_BATCH_SIZE", "--global-batch-size", None),
    ("MICRO_BATCH_SIZE", "--micro-batch-size", None),
    ("GRAD_ACCUM_STEPS", "--grad-accum-steps", None),
    ("SEQ_LENGTH", "--seq-length", None),
    ("SEED", "--seed", "1234"),
    ("MUP_EMB_SCALE", "--mup-emb-scale", None),
    ("MUP_DEPTH_SCALE", "--mup-depth-scale", None),
    ("MAX_LR", "--max-lr", None),
    ("MIN_LR", "--min-lr", None),
    ("WARMUP_ITERS", "--warmup-iters", None),
    ("LR_DECAY_ITERS", "--lr-decay-iters", None),
    ("WSD_DECAY_ITERS", "--wsd-decay-iters", None),
    ("TENSOR_PARALLEL_SIZE", "--tensor-parallel-size", None),
    ("HF_DATASET", "--hf-dataset", None),
    ("HF_DATASET_CONFIG", "--hf-dataset-config", None),
    ("HF_DATASET_SPLIT", "--hf-dataset-split", None),
    ("HF_TEXT_TEMPLATE", "--hf-text-template", None),
    ("HF_DATA_FORMAT", "--hf-data-format", None),
    ("HF_DATA_FILES", "--hf-data-files", None),
    ("TOKENIZER_PATH", "--tokenizer-path", None),
    ("DUMP_INPUTS_DIR", "--dump-inputs-dir", None),
    ("EXPORT_REPORT", "--export-report", None),
)

# process-environment defaults for the workers (set only where the job left them unset)
_CHILD_ENV_DEFAULTS = {
    "CUDA_DEVICE_MAX_CONNECTIONS": "8",     # side streams must not serialise behind one queue
    "PYTORCH_CUDA_ALLOC_CONF": "expandable_segments:True",
    "TORCH_NCCL_HEARTBEAT_TIMEOUT_SEC": "1800",
}


def _get(env: dict, key: str, default: str | None = None) -> str | None:
    v = env.get(key)
    return default if v is None or v == "" else v


def plan_from_env(env: dict, nproc_per_node: int | None = None,
                  extra_args: tuple[str, ...] = (), repo_root: str | None = None) -> LaunchPlan:
    """Translate a job environment into a launch plan; raises :class:`LaunchError` when invalid."""
    stage = _get(env, "STAGE", "decay_from_megatron")
    stage = _STAGE_ALIASES.get(stage, stage)
    if stage not in STAGES:
        raise LaunchError(f"unknown STAGE={stage} (allowed: {', '.join(STAGES)}, decay)")
    root = repo_root or os.getcwd()
    ckpt_root = _get(env, "CHECKPOINT_ROOT")
    resume = _get(env, "RESUME_DIR")
    save_dir = _get(env, "SAVE_DIR")
    save_interval = _get(env, "SAVE_INTERVAL")
    synthetic = _get(env, "SYNTHETIC_DATA", "0") == "1"

    if stage in ("stable", "hf_pretrain"):
        sub, resume, ckpt_root = "pretrain", None, None
    elif stage in ("stable_2", "decay_from_ours"):
        if resume is None:
            raise LaunchError(f"STAGE={stage} requires RESUME_DIR (a step_<N> directory of the previous phase)")
        sub, ckpt_root = "train", None
    else:  # decay_from_megatron
        if ckpt_root is None:
            raise LaunchError(f"STAGE={stage} requires CHECKPOINT_ROOT (directory holding canonical_state_fp32.pt)")
        sub = "train"
    if _get(env, "HF_DATASET") is None and not synthetic:
        raise LaunchError("HF_DATASET must be set (or SYNTHETIC_DATA=1 for uniform random token ids)")
    if stage != "hf_pretrain":
        save_dir = save_dir or os.path.join(root, ".checkpoints", stage)
        save_interval = save_interval or "5000"
    if resume is not None and save_dir is not None and \
            os.path.abspath(resume) == os.path.abspath(save_dir):
        raise LaunchError("RESUME_DIR and SAVE_DIR must differ (a resumed run never overwrites its source)")
    steps_done = 0
    if _get(env, "AUTO_RESUME", "0") == "1" and save_dir is not None:
        point = find_restart_point(save_dir)
        if point is not None:
            # continue this job's own run: the newest finished checkpoint wins over the stage's
            # starting point (random init, Megatron export or the previous phase's RESUME_DIR)
            sub, resume, ckpt_root = "train", point[1], None
            steps_done = point[0]

    args: list[str] = ["--model", _get(env, "MODEL", "0.5b")]
    if ckpt_root is not None:
        args += ["--checkpoint-root", ckpt_root]
    for name, flag, default in _VALUE_FLAGS:
        v = _get(env, name, default)
        if name == "NUM_STEPS" and v is not None and steps_done:
            v = str(max(0, int(v) - steps_done))     # --num-steps counts the steps of THIS launch
        if v is not None:
            args += [flag, v]
    tf = _get(env, "HF_TEXT_FIELD")
    if tf is not None:
        args += ["--hf-text-field", *tf.split()]     # several columns: space-separated
    if save_dir is not None:
        args += ["--save-dir", save_dir]
        if save_interval is not None:
            args += ["--save-interval", save_interval]
    if resume is not None:
        args += ["--resume", resume]
    mtp = int(_get(env, "MTP_NUM_LAYERS", "0"))
    if mtp > 0:
        args += ["--mtp-num-layers", str(mtp),
                 "--mtp-loss-scaling-factor", _get(env, "MTP_LOSS_SCALING_FACTOR", "0.1")]
    args += list(extra_args)

    child = {k: v for k, v in _CHILD_ENV_DEFAULTS.items() if _get(env, k) is None}
    if stage == "stable":
        child["RANDOM_INIT"] = "1"
    nnodes = int(_get(env, "NNODES", _get(env, "WORLD_SIZE", "1")))
    node_rank = int(_get(env, "NODE_RANK", _get(env, "RANK", "0")))
    if not 0 <= node_rank < nnodes:
        raise LaunchError(f"node rank {node_rank} outside 0..{nnodes - 1}")
    if nproc_per_node is None:
        nproc_per_node = int(_get(env, "NPROC_PER_NODE", "0")) or _visible_gpus()
    return LaunchPlan(stage=stage, subcommand=sub, nnodes=nnodes, node_rank=node_rank,
                      nproc_per_node=nproc_per_node,
                      master_addr=_get(env, "MASTER_ADDR", "127.0.0.1"),
                      master_port=int(_get(env, "MASTER_PORT", "29500")),
                      cli_args=tuple(args), child_env=child)


def find_restart_point(save_dir: str) -> tuple[int, str] | None:
    """``(N, path)`` of the newest ``step_<N>`` directory under ``save_dir`` that holds a finished
    checkpoint (a single-file one or the per-rank shards of a tensor-parallel run), else None."""
    from .ckpt.checkpoint import latest_step_dir
    if not os.path.isdir(save_dir):
        return None
    best = None
    for pattern in ("training_state.pt", "rank_*.pt"):
        d = latest_step_dir(save_dir, pattern)
        if d is not None:
            n = int(d.name[len("step_"):])
            if best is None or n > best[0]:
                best = (n, str(d))
    return best


def env_from_job_spec(path: str, base_env: dict | None = None) -> dict:
    """Environment of a scheduler job spec (``task.envVars`` = list of ``{name, value}``) laid over
    ``base_env``; ``${VAR}`` references in values are expanded from the combined environment.
    Spec files for an 8-GPU node live in ``forgetrain_b200/job_specs/`` (the counterpart of the
    reference's ``job_specs/smoke/*.json``)."""
    import json
    import re
    with open(path) as f:
        task = json.load(f)["task"]
    env = dict(base_env or {})
    for item in task.get("envVars", []):
        env[item["name"]] = str(item["value"])
    expand = lambda v: re.sub(r"\$\{(\w+)\}", lambda m: env.get(m.group(1), m.group(0)), v)
    out = {k: expand(v) for k, v in env.items()}
    gpus = task.get("resources", {}).get("gpuCount")
    if gpus and "NPROC_PER_NODE" not in out:
        out["NPROC_PER_NODE"] = str(gpus)
    return out


def _visible_gpus() -> int:
    import torch
    n = torch.cuda.device_count() if torch.cuda.is_available() else 0
    return n or 1


def describe(plan: LaunchPlan) -> str:
    lines = [f"=== forgetrain_b200 launch: STAGE={plan.stage} -> {plan.subcommand} ===",
             f"  nodes={plan.nnodes} node_rank={plan.node_rank} procs/node={plan.nproc_per_node} "
             f"rendezvous={plan.master_addr}:{plan.master_port}"]
    lines += [f"  env {k}={v}" for k, v in sorted(plan.child_env.items())]
    lines.append("  " + " ".join(shlex.quote(a) for a in plan.command()))
    return "\n".join(lines)


def main(argv: list[str] | None = None) -> int:
    p = argparse.ArgumentParser(prog="forgetrain_b200.launch", description=__doc__.split("\n\n")[0])
    p.add_argument("--dry-run", action="store_true", help="print the plan and exit")
    p.add_argument("--nproc-per-node", type=int, default=None)
    p.add_argument("--max-restarts", type=int, default=None,
                   help="restart a failed job from its newest checkpoint up to this many times (MAX_RESTARTS)")
    p.add_argument("--job-spec", default=None,
                   help="scheduler job spec (JSON) whose task.envVars are laid over the environment")
    p.add_argument("extra", nargs=argparse.REMAINDER, help="after --: flags passed to the training CLI")
    a = p.parse_args(argv)
    extra = tuple(x for x in a.extra if x != "--")
    try:
        job_env = env_from_job_spec(a.job_spec, dict(os.environ)) if a.job_spec else dict(os.environ)
        plan = plan_from_env(job_env, a.nproc_per_node, extra)
    except LaunchError as e:
        print(f"ERROR: {e}", file=sys.stderr)
        return 2
    print(describe(plan), flush=True)
    if a.dry_run:
        return 0
    max_restarts = a.max_restarts if a.max_restarts is not None else int(_get(job_env, "MAX_RESTARTS", "0"))

    def worker_env(pl: LaunchPlan) -> dict:
        env = dict(job_env)
        env.update(pl.child_env)
        # the launcher's own RANK / WORLD_SIZE are node-level; workers get theirs from the launcher
        env.pop("RANK", None)
        env.pop("WORLD_SIZE", None)
        return env

    if max_restarts <= 0:
        cmd = plan.command()
        os.execvpe(cmd[0], cmd, worker_env(plan))
        return 0  # not reached
    return supervise(plan, job_env, a.nproc_per_node, extra, max_restarts, worker_env)


def supervise(plan: LaunchPlan, job_env: dict, nproc_per_node, extra, max_restarts: int, worker_env,
              run=None) -> int:
    """Run the plan as a child process; after a failure plan again with ``AUTO_RESUME`` on (the
    newest finished checkpoint of ``SAVE_DIR``, fewer steps left) and start it again, at most
    ``max_restarts`` times. Returns the exit code of the last attempt. ``run(cmd, env) -> int`` is
    replaceable for tests."""
    import signal
    import subprocess
    stop = {"requested": False, "child": None}

    def forward(signum, frame):           # a pre-emption notice goes to the job and ends the loop
        stop["requested"] = True
        if stop["child"] is not None and stop["child"].poll() is None:
            stop["child"].send_signal(signum)

    def run_child(cmd, env):
        stop["child"] = subprocess.Popen(cmd, env=env)
        return stop["child"].wait()

    if run is None:
        run = run_child
        try:
            signal.signal(signal.SIGTERM, forward)
        except ValueError:                # not the main thread: leave the default behaviour
            pass
    attempt = 0
    while True:
        steps = plan.cli_args[plan.cli_args.index("--num-steps") + 1] if "--num-steps" in plan.cli_args else None
        if steps == "0":
            print("=== nothing left to do: the newest checkpoint is at the last step ===", flush=True)
            return 0
        rc = run(plan.command(), worker_env(plan))
        if rc == 0 or attempt >= max_restarts or stop["requested"]:
            return rc
        attempt += 1
        env = dict(job_env)
        env["AUTO_RESUME"] = "1"
        plan = plan_from_env(env, nproc_per_node, extra)
        print(f"=== attempt {attempt} of {max_restarts} after exit code {rc} ===\n{describe(plan)}", flush=True)


if __name__ == "__main__":
    sys.exit(main())
