import ast
import json
import os
import subprocess
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent


def test_public_api_all_is_importable():
    import forgetrain_b200 as pkg
    tree = ast.parse((ROOT / "forgetrain_b200" / "__init__.py").read_text())
    names = None
    for node in tree.body:
        if isinstance(node, ast.Assign) and getattr(node.targets[0], "id", "") == "__all__":
            names = [e.value for e in node.value.elts]
    assert names
    for n in names:
        assert hasattr(pkg, n), n


def test_cli_flags_cover_reference_surface():
    from forgetrain_b200.cli import build_parser
    p = build_parser()
    opts = {o for a in p._actions for o in a.option_strings}
    for flag in ["--num-steps", "--global-batch-size", "--micro-batch-size", "--seq-length",
                 "--num-local-microbatches", "--save-interval", "--save-dir", "--resume",
                 "--mup-emb-scale", "--mup-depth-scale", "--max-lr", "--min-lr", "--warmup-iters",
                 "--lr-decay-iters", "--wsd-decay-iters", "--mtp-num-layers",
                 "--mtp-loss-scaling-factor", "--dump-inputs-dir", "--seed", "--device",
                 "--export-checkpoint-root", "--checkpoint-root", "--hf-dataset", "--tokenizer-path",
                 "--grad-accum-steps", "--export-report", "--tensor-parallel-size",
                 "--sequence-parallel", "--no-sequence-parallel", "--comm", "--dtype"]:
        assert flag in opts, flag


def test_resume_save_dir_mutex(tmp_path):
    from forgetrain_b200.cli import main
    with pytest.raises(SystemExit):
        main(["pretrain", "--model", "tiny", "--resume", str(tmp_path), "--save-dir", str(tmp_path)])


def test_no_undeclared_environment_reads():
    """Every os.environ access in the package names a declared variable."""
    from forgetrain_b200.engine_config import DECLARED_ENV_VARS
    declared = set(DECLARED_ENV_VARS) | {"FT_BENCH_GRAPH"}
    for path in (ROOT / "forgetrain_b200").rglob("*.py"):
        tree = ast.parse(path.read_text())
        for node in ast.walk(tree):
            key = None
            if isinstance(node, ast.Call) and isinstance(node.func, ast.Attribute) \
                    and node.func.attr in ("get", "setdefault") \
                    and isinstance(node.func.value, ast.Attribute) and node.func.value.attr == "environ" \
                    and node.args and isinstance(node.args[0], ast.Constant):
                key = node.args[0].value
            if isinstance(node, ast.Subscript) and isinstance(node.value, ast.Attribute) \
                    and node.value.attr == "environ" and isinstance(node.slice, ast.Constant):
                key = node.slice.value
            if key is not None:
                assert key in declared, f"{path.name}: undeclared env var {key}"


def test_cli_pretrain_tiny_cpu_writes_report_and_checkpoint(tmp_path):
    env = dict(os.environ, OUTPUT_DIR=str(tmp_path / "out"), PYTHONPATH=str(ROOT))
    (tmp_path / "out").mkdir()
    r = subprocess.run([sys.executable, "-m", "training_engine_tensor", "pretrain", "--model", "tiny",
                        "--num-steps", "3", "--device", "cpu", "--micro-batch-size", "1",
                        "--global-batch-size", "2", "--seq-length", "64", "--save-dir",
                        str(tmp_path / "ck"), "--save-interval", "2", "--emit-loss-lines"],
                       capture_output=True, text=True, env=env, cwd=ROOT, timeout=300)
    assert r.returncode == 0, r.stderr[-2000:]
    assert "DONE" in r.stdout and "[LOSS] step=3" in r.stdout and "iteration" in r.stdout
    rep = json.loads((tmp_path / "out" / "training_report.json").read_text())
    assert len(rep["steps"]) == 3 and {"loss", "grad_norm", "lr", "total_step_time", "mfu_e2e",
                                       "mfu_e2e_standard"} <= set(rep["steps"][0])
    lines = (tmp_path / "out" / "3step" / "ours_results.jsonl").read_text().splitlines()
    assert len(lines) == 3 and json.loads(lines[0])["step_time"] > 0
    assert (tmp_path / "out" / "3step" / "DONE").read_text() == "ok\n"
    assert (tmp_path / "ck" / "step_0000002" / "training_state.pt").exists()
    assert (tmp_path / "ck" / "step_0000003" / "training_state.pt").exists()


def test_grad_norm_diag_prints_local_norms(capsys):
    """GRAD_NORM_DIAG: full pre-reduce norm and top per-parameter norms; the step itself is
    unchanged."""
    import torch
    from forgetrain_b200.config import load_model_spec
    from forgetrain_b200.engine_config import from_spec
    from forgetrain_b200.parallel.topology import Topology
    from forgetrain_b200.trainer import Trainer
    spec = load_model_spec("tiny")
    tok = torch.randint(0, spec.vocab_size, (2, 33), generator=torch.Generator().manual_seed(0))
    batch = {"tokens": tok[:, :-1].contiguous(), "labels": tok[:, 1:].contiguous()}
    out = {}
    for diag in (False, True):
        cfg = from_spec(spec, dtype="fp32", comm="nccl", warmup_iters=0, grad_norm_diag=diag,
                        no_grad_clip=True)
        tr = Trainer(spec, cfg, Topology(device=torch.device("cpu")), seq_length=32,
                     micro_batch_size=2, seed=0)
        r = tr.train_step([batch, batch])
        out[diag] = (float(r["loss"]), float(r["grad_norm"]))
    text = capsys.readouterr().out
    assert "[grad-norm-diag] pre_reduce_rank0_full=" in text and "[grad-norm-top]" in text
    full = float(text.split("pre_reduce_rank0_full=")[1].split()[0])
    assert full == pytest.approx(out[True][1], rel=1e-4)      # one rank: local norm == global
    assert out[True] == pytest.approx(out[False], rel=1e-6)


def test_export_checkpoint_root_receives_the_report_not_checkpoints(tmp_path):
    """--export-checkpoint-root is the directory of training_report.json (reference: 0.5B
    __main__.py:520-530); it does not turn on checkpoint saving."""
    from forgetrain_b200.cli import main
    root = tmp_path / "export" / "run1"
    rc = main(["pretrain", "--model", "tiny", "--num-steps", "2", "--device", "cpu",
               "--micro-batch-size", "1", "--global-batch-size", "1", "--seq-length", "64",
               "--export-checkpoint-root", str(root)])
    assert rc == 0
    rep = json.loads((root / "training_report.json").read_text())
    assert len(rep["steps"]) == 2
    assert not list(root.glob("step_*"))


def test_data_parallel_rank_flag_selects_that_ranks_data(tmp_path):
    """Without a launcher, --data-parallel-rank R makes the single process read rank R's data
    shard (the reference uses the flag as the RANK fallback, 0.5B __main__.py:288-305)."""
    from forgetrain_b200.cli import main
    losses = {}
    for r in (0, 1):
        root = tmp_path / f"r{r}"
        main(["pretrain", "--model", "tiny", "--num-steps", "1", "--device", "cpu",
              "--micro-batch-size", "1", "--global-batch-size", "1", "--seq-length", "64",
              "--data-parallel-rank", str(r), "--data-parallel-ranks", "2",
              "--export-checkpoint-root", str(root)])
        losses[r] = json.loads((root / "training_report.json").read_text())["steps"][0]["loss"]
    assert losses[0] != losses[1]            # same weights, different shard of the data
    with pytest.raises(SystemExit):
        main(["pretrain", "--model", "tiny", "--device", "cpu", "--data-parallel-rank", "3",
              "--data-parallel-ranks", "2"])


def test_checkpoint_train_loop_on_pretokenized_inputs(tmp_path):
    """The reference's gate run: start from a checkpoint, replay one pre-tokenised batch for the
    requested steps (0.5B __main__.py:140-146, train_loop.py:487-505). The dump of step 0 of a run
    is a valid --tokenized-inputs file, and replaying it gives that run's first loss."""
    import torch
    from forgetrain_b200.cli import main
    from forgetrain_b200.data.tokenized import FixedBatchSource
    common = ["--model", "tiny", "--device", "cpu", "--micro-batch-size", "2", "--global-batch-size", "2",
              "--seq-length", "64"]
    main(["pretrain", *common, "--num-steps", "2", "--save-dir", str(tmp_path / "ck"), "--save-interval", "1",
          "--dump-inputs-dir", str(tmp_path / "dump"), "--export-checkpoint-root", str(tmp_path / "a")])
    first = json.loads((tmp_path / "a" / "training_report.json").read_text())["steps"]
    inputs = tmp_path / "dump" / "inputs_step0000001.pt"
    assert inputs.exists()
    main(["checkpoint-train-loop", "--model", "tiny", "--device", "cpu", "--micro-batch-size", "2",
          "--checkpoint-root", str(tmp_path / "ck" / "step_0000001"), "--tokenized-inputs", str(inputs),
          "--step-indices", "1", "2", "3", "--export-checkpoint-root", str(tmp_path / "b")])
    rep = json.loads((tmp_path / "b" / "training_report.json").read_text())["steps"]
    assert len(rep) == 3
    assert rep[0]["loss"] == pytest.approx(first[1]["loss"], abs=1e-6)     # same weights, same rows
    assert rep[2]["loss"] < rep[0]["loss"]                                  # one batch, memorised
    # row selection per rank and micro-batch, and the size check
    data = {"tokens": torch.arange(8 * 4).view(8, 4), "labels": torch.arange(8 * 4).view(8, 4)}
    src = FixedBatchSource(data, 2, dp_rank=1, dp_size=2, num_local_microbatches=2)
    assert next(src)["tokens"][:, 0].tolist() == [16, 20] and next(src)["tokens"][:, 0].tolist() == [24, 28]
    assert next(src)["tokens"][:, 0].tolist() == [16, 20] and float(next(src)["loss_mask"].sum()) == 8.0
    with pytest.raises(ValueError, match="rows"):
        FixedBatchSource(data, 4, dp_rank=0, dp_size=2, num_local_microbatches=2)


def test_train_subcommand_needs_a_starting_point_and_accepts_resume_alone(tmp_path):
    from forgetrain_b200.cli import main
    from forgetrain_b200.ckpt.convert_to_hf import main as export_main
    common = ["--model", "tiny", "--device", "cpu", "--micro-batch-size", "1", "--global-batch-size", "1",
              "--seq-length", "64"]
    with pytest.raises(SystemExit, match="checkpoint-root or --resume"):
        main(["train", *common])
    main(["pretrain", *common, "--num-steps", "1", "--save-dir", str(tmp_path / "run1")])
    main(["train", *common, "--num-steps", "1", "--resume", str(tmp_path / "run1" / "step_0000001"),
          "--save-dir", str(tmp_path / "run1")])
    assert (tmp_path / "run1" / "step_0000002" / "training_state.pt").exists()
    # the exporter takes the reference's --input spelling too
    assert export_main(["--input", str(tmp_path / "run1" / "step_0000002"), "--output", str(tmp_path / "hf"),
                        "--model", "tiny"]) == 0
    assert (tmp_path / "hf" / "model.safetensors").exists() and (tmp_path / "hf" / "config.json").exists()


def test_reference_module_names_resolve_to_this_engine():
    """``training_engine_tensor.<module>`` exists for every module a user of the reference imports
    from, each ``__all__`` is a literal list and every name in it is defined (the reference checks
    its own ``__all__`` lists the same way, tests/test_public_api.py)."""
    import importlib
    pkg = ROOT / "training_engine_tensor"
    names = {"engine_config", "config", "train_loop", "parameters", "optimizer", "nccl", "data",
             "hf_dataloader", "profiling", "kernels", "forward", "backward", "entry"}
    assert names <= {p.stem for p in pkg.glob("*.py")}
    for name in sorted(names):
        tree = ast.parse((pkg / f"{name}.py").read_text())
        alls = [n for n in tree.body if isinstance(n, ast.Assign)
                and any(isinstance(t, ast.Name) and t.id == "__all__" for t in n.targets)]
        assert len(alls) == 1
        exported = ast.literal_eval(alls[0].value)
        mod = importlib.import_module(f"training_engine_tensor.{name}")
        assert exported and all(hasattr(mod, x) for x in exported), name
    from training_engine_tensor.config import load_model_spec, mup_residual_scale, mup_width_scale
    spec = load_model_spec("0.5b")
    assert mup_width_scale(spec) == 4.0 and abs(mup_residual_scale(spec) - 1.4 / 24 ** 0.5) < 1e-9
    from training_engine_tensor.optimizer import compute_lr
    assert compute_lr(0, 1e-2, 0.0, 10, 100, 0) == 0.0


def test_functional_forward_backward_aliases_drive_the_model():
    import torch
    from forgetrain_b200.config import load_model_spec
    from forgetrain_b200.models.params import ParamStore
    from training_engine_tensor.backward import backward_pass, cross_entropy_loss_backward
    from training_engine_tensor.forward import MiniCPM4, forward_pass_with_save
    spec = load_model_spec("tiny")
    st = ParamStore(spec, "cpu", torch.float32)
    st.init_random(0)
    tok = torch.randint(0, spec.vocab_size, (2, 33), generator=torch.Generator().manual_seed(0))
    a, b = MiniCPM4(spec, st), None
    logits = forward_pass_with_save(a, tok[:, :-1].contiguous())
    loss, dlogits = cross_entropy_loss_backward(a, logits, tok[:, 1:].contiguous())
    seen = []
    backward_pass(a, tok[:, :-1].contiguous(), dlogits, grad_sink=seen.append)
    g1 = st.flat_grads.clone()
    assert seen[0] == "output.weight" or seen[0] == "norm.weight"
    assert seen[-1] == "tok_embeddings.weight" and float(g1.abs().sum()) > 0
    st.flat_grads.zero_()
    loss2 = MiniCPM4(spec, st).forward_backward(tok[:, :-1].contiguous(), tok[:, 1:].contiguous())
    assert float(loss2) == float(loss) and torch.equal(st.flat_grads, g1)


def test_doctor_reports_the_environment():
    from forgetrain_b200 import doctor
    info = doctor.collect()
    assert {"python", "torch", "devices", "native_library", "peak_tflops_for_mfu", "problems",
            "can_train_on_gpu", "can_train_on_cpu"} <= set(info)
    assert info["backends"]["gloo"] is True and info["can_train_on_cpu"] is True
    assert "gemm_sm100.cu" in info["native_library"]["sources"]
    if not info["cuda_available"]:
        assert info["can_train_on_gpu"] is False and doctor.main([]) == 0


def test_doctor_self_test_trains_a_few_steps(capsys):
    from forgetrain_b200 import doctor
    import torch
    if torch.cuda.is_available():
        pytest.skip("the CPU form of the self-test")
    assert doctor.main(["--self-test"]) == 0
    out = capsys.readouterr().out
    assert "self-test on cpu: losses" in out and out.rstrip().endswith(": ok")
    t = doctor.self_test()
    assert t["ok"] and len(t["losses"]) == 3 and t["losses"][2] < t["losses"][0]


def test_batch_defaults_come_from_the_model_spec():
    """No batch flags: micro-batch, sequence length and global batch are the model spec's
    (the reference pins the same in tests/test_cli_defaults.py)."""
    import types
    from forgetrain_b200.cli import _resolve_local_microbatches, build_parser
    from forgetrain_b200.config import load_model_spec
    a = build_parser().parse_args(["pretrain"])
    assert a.micro_batch_size is None and a.global_batch_size is None and a.seq_length is None
    s05, s8 = load_model_spec("0.5b"), load_model_spec("8b")
    assert (s05.micro_batch_size, s05.global_batch_size, s05.seq_length) == (10, 160, 4096)
    assert _resolve_local_microbatches(a, s05, 1, s05.micro_batch_size) == 16
    assert _resolve_local_microbatches(a, s05, 8, s05.micro_batch_size) == 2
    assert _resolve_local_microbatches(a, s05, 3, s05.micro_batch_size) == 1      # 160 / 30: no
    assert _resolve_local_microbatches(a, s8, 4, s8.micro_batch_size) == 8        # the spec's GAS
    b = build_parser().parse_args(["pretrain", "--global-batch-size", "40"])
    assert _resolve_local_microbatches(b, s05, 2, 10) == 2
    with pytest.raises(SystemExit):
        _resolve_local_microbatches(b, s05, 3, 10)
