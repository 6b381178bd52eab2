"""Command line: ``python -m training_engine_tensor pretrain ...`` (also ``python -m
forgetrain_b200 ...``).

Sub-commands and flags follow the reference's CLIs
(exports/train_engine_0.5B/src/training_engine_tensor/__main__.py:65-235 and
exports/train_engine_8b/src/training_engine_tensor/__main__.py:57-224):

* ``pretrain``               random-init (or ``--resume``) training; synthetic uniform tokens
                             unless ``--hf-dataset`` is given
* ``train``                  start from ``--checkpoint-root``: a Megatron export
                             (``canonical_state_fp32.pt`` + optional optimizer state) or one of
                             this engine's own checkpoints
* ``checkpoint-train-loop``  train with periodic checkpoints (defaults to 200 steps)

Every :class:`~forgetrain_b200.engine_config.EngineConfig` field is also exposed as
``--<field>`` / ``--no-<field>``. Additions over the reference: ``--model``, ``--dtype``,
``--backend``, ``--tensor-parallel-size``, ``--sequence-parallel``, ``--tie-embeddings``,
``--comm {fused,nccl}``.
"""
from __future__ import annotations

import argparse
import dataclasses
import json
import os
import sys
from pathlib import Path

from . import engine_config as ec
from .config import load_model_spec


def _add_engine_config_args(p: argparse.ArgumentParser) -> None:
    grp = p.add_argument_group("engine config (one flag per EngineConfig field)")
    for f in dataclasses.fields(ec.EngineConfig):
        flag = "--" + f.name.replace("_", "-")
        if f.type in ("bool", bool):
            grp.add_argument(flag, dest=f"cfg_{f.name}", action=argparse.BooleanOptionalAction,
                             default=None)
        else:
            typ = {"int": int, "float": float, "str": str}.get(str(f.type), str)
            grp.add_argument(flag, dest=f"cfg_{f.name}", type=typ, default=None)
    # the reference engines' own spellings: renamed fields translate, path selectors that
    # have no counterpart here are accepted and reported as having no effect
    old = p.add_argument_group("reference-engine spellings")
    own = {f.name for f in dataclasses.fields(ec.EngineConfig)}
    for name, (fld, conv) in sorted(ec.LEGACY_FIELD_ALIASES.items()):
        flag = "--" + name.replace("_", "-")
        if conv is bool or name == "fp32_mode":
            old.add_argument(flag, dest=f"legacy_{name}", action=argparse.BooleanOptionalAction,
                             default=None, help=f"same as --{fld.replace('_', '-')}")
        else:
            old.add_argument(flag, dest=f"legacy_{name}", type=conv, default=None,
                             help=f"same as --{fld.replace('_', '-')}")
    for name in sorted(ec.LEGACY_NOOP_FIELDS - own):
        flag = "--" + name.replace("_", "-")
        if flag in p._option_string_actions:
            continue
        old.add_argument(flag, "--no-" + name.replace("_", "-"), dest=f"noop_{name}", nargs="?",
                         const=True, default=None, help=argparse.SUPPRESS)


def build_parser() -> argparse.ArgumentParser:
    p = argparse.ArgumentParser(prog="training_engine_tensor",
                                description="B200-native MiniCPM4 pretraining engine")
    p.add_argument("command", choices=["pretrain", "train", "checkpoint-train-loop"])
    p.add_argument("--model", default="0.5b", help="built-in spec (tiny, 0.5b, 8b) or a model_spec.toml")
    p.add_argument("--num-steps", type=int, default=None)
    p.add_argument("--step-indices", nargs="+", type=int, default=None,
                   help="run len(STEP_INDICES) steps (alternative to --num-steps)")
    p.add_argument("--tokenized-inputs", default=None,
                   help=".pt file of pre-tokenised rows (tokens, labels, loss_mask[, position_ids]); "
                        "the same rows are replayed every step")
    p.add_argument("--global-batch-size", type=int, default=None)
    p.add_argument("--micro-batch-size", type=int, default=None)
    p.add_argument("--grad-accum-steps", type=int, default=None)
    p.add_argument("--seq-length", type=int, default=None)
    p.add_argument("--num-local-microbatches", type=int, default=None)
    p.add_argument("--num-workers", type=int, default=0)
    p.add_argument("--dump-inputs-dir", default=None)
    p.add_argument("--save-interval", type=int, default=0)
    p.add_argument("--save-dir", "--save-checkpoint-dir", dest="save_dir", default=None)
    p.add_argument("--resume", default=None)
    p.add_argument("--checkpoint-root", default=None)
    p.add_argument("--export-checkpoint-root", default=None)
    p.add_argument("--export-report", default=None)
    p.add_argument("--data-parallel-rank", type=int, default=None)
    p.add_argument("--data-parallel-ranks", type=int, default=None)
    p.add_argument("--seed", type=int, default=1234)
    p.add_argument("--device", default=None)
    p.add_argument("--backend", choices=["nccl", "gloo"], default=None)
    p.add_argument("--tie-embeddings", action=argparse.BooleanOptionalAction, default=None)
    p.add_argument("--vocab-size", type=int, default=None)
    p.add_argument("--num-layers", type=int, default=None, help="override the spec's layer count")
    hf = p.add_argument_group("HuggingFace dataset")
    hf.add_argument("--hf-dataset", default=None)
    hf.add_argument("--tokenizer-path", default=None)
    hf.add_argument("--hf-dataset-config", default=None)
    hf.add_argument("--hf-dataset-split", default="train")
    hf.add_argument("--hf-text-field", nargs="+", default=None,
                    help="text column name(s); auto-detected when omitted")
    hf.add_argument("--hf-text-template", default=None)
    hf.add_argument("--hf-data-format", default=None)
    hf.add_argument("--hf-data-files", default=None)
    hf.add_argument("--max-packed-rows", type=int, default=None)
    hf.add_argument("--hf-stream", action="store_true",
                    help="tokenise on demand instead of packing the whole slice up front")
    hf.add_argument("--hf-doc-positions", action="store_true",
                    help="rotary positions restart at every document of a packed row")
    hf.add_argument("--hf-shuffle", action=argparse.BooleanOptionalAction, default=True,
                    help="new permutation of the packed rows on every pass (seed + data-parallel rank)")
    _add_engine_config_args(p)
    return p


def _validate_resume_save_dir_mutex(args) -> None:
    if args.resume and args.save_dir:
        a, b = Path(args.resume).resolve(), Path(args.save_dir).resolve()
        # equal paths only: resuming from <run>/step_N while saving later steps into <run> is
        # the normal way to continue a run (each step has its own sub-directory)
        if a == b:
            raise SystemExit("--resume and --save-dir point at the same directory: a resumed run "
                             "would overwrite the checkpoint it was started from")


def _resolve_local_microbatches(args, spec, dp_size: int, mbs: int) -> int:
    if args.num_local_microbatches:
        return args.num_local_microbatches
    if args.grad_accum_steps:
        return args.grad_accum_steps
    gbs = args.global_batch_size
    if gbs:
        if gbs % (mbs * dp_size):
            raise SystemExit(f"global batch {gbs} is not a multiple of micro-batch {mbs} x DP {dp_size}")
        return gbs // (mbs * dp_size)
    if getattr(args, "command", None) == "checkpoint-train-loop" and getattr(args, "tokenized_inputs", None):
        return 1              # the gate run replays one micro-batch per rank unless told otherwise
    if spec.grad_accum_steps:
        return spec.grad_accum_steps
    # no flag: the model spec's global batch, as in the reference CLI (its defaults come from
    # model_spec.toml); when this world cannot split it evenly, one micro-batch per step
    if spec.global_batch_size and spec.global_batch_size % (mbs * dp_size) == 0:
        return spec.global_batch_size // (mbs * dp_size)
    return 1


def main(argv: list[str] | None = None) -> int:
    args = build_parser().parse_args(argv)
    _validate_resume_save_dir_mutex(args)
    spec = load_model_spec(args.model, tie_embeddings=args.tie_embeddings, vocab_size=args.vocab_size,
                           num_layers=args.num_layers)
    overrides = {k[4:]: v for k, v in vars(args).items() if k.startswith("cfg_") and v is not None}
    for k, v in vars(args).items():
        if k.startswith("legacy_") and v is not None:
            fld, conv = ec.LEGACY_FIELD_ALIASES[k[7:]]
            overrides.setdefault(fld, conv(v))
    ignored = sorted(k[5:] for k, v in vars(args).items() if k.startswith("noop_") and v is not None)
    if ignored:
        print("[CONFIG] no effect here (the fused kernels are the only path): " + " ".join(ignored),
              file=sys.stderr)
    env_cfg = ec.from_env()
    base = ec.from_spec(spec)
    # precedence: CLI > environment > model spec defaults
    defaults = ec.EngineConfig()
    merged = {}
    for f in dataclasses.fields(ec.EngineConfig):
        v_spec, v_env = getattr(base, f.name), getattr(env_cfg, f.name)
        merged[f.name] = v_env if v_env != getattr(defaults, f.name) else v_spec
    merged.update(overrides)
    device = args.device
    import torch
    if device is None:
        device = "cuda" if torch.cuda.is_available() else "cpu"
    if device == "cpu" and "dtype" not in overrides and "FT_DTYPE" not in os.environ:
        merged["dtype"] = "fp32"
    cfg = ec.EngineConfig(**merged)
    ec.validate_config(cfg)
    if ec.has_global_config():
        ec.reset_global_config()
    ec.set_global_config(cfg)

    from .parallel.topology import init_topology, shutdown
    from .trainer import run_training_loop
    topo = init_topology(cfg.tensor_parallel_size, device=device, backend=args.backend,
                         num_kv_groups=spec.num_query_groups)
    if topo.rank == 0:
        ec.print_config_summary(cfg)
        if cfg.mup_emb_scale > 0 or cfg.mup_depth_scale > 0:
            res = cfg.mup_depth_scale / spec.num_layers ** 0.5 if cfg.mup_depth_scale > 0 else 1.0
            print(f"[muP] emb_scale={cfg.mup_emb_scale} depth_scale={cfg.mup_depth_scale} "
                  f"residual_scale={res:.6f} width_scale={spec.mup_width_scale:.1f}", flush=True)
        if cfg.mtp_num_layers > 0:
            print(f"[MTP] num_layers={cfg.mtp_num_layers} "
                  f"loss_scaling_factor={cfg.mtp_loss_scaling_factor} "
                  f"per_layer_scale={cfg.mtp_loss_scaling_factor / cfg.mtp_num_layers:.6f}", flush=True)
    mbs = args.micro_batch_size or spec.micro_batch_size
    seq = args.seq_length or spec.seq_length
    n_mb = _resolve_local_microbatches(args, spec, topo.dp_size, mbs)
    num_steps = args.num_steps or (len(args.step_indices) if args.step_indices else
                                   (200 if args.command == "checkpoint-train-loop" else 1))
    resume = args.resume
    if args.command == "train":
        # continues a run: from a save directory of this engine (--resume) or from an initial
        # checkpoint such as a Megatron export (--checkpoint-root); --resume wins when both are given
        if not args.checkpoint_root and not resume:
            raise SystemExit("train needs --checkpoint-root or --resume")
        resume = resume or args.checkpoint_root
    elif args.command == "pretrain" and args.checkpoint_root and not resume:
        # the 8B engine's `pretrain --checkpoint-root`: start from given weights instead of random
        # ones (reference: 8B __main__.py:360-455)
        resume = args.checkpoint_root
    save_dir = args.save_dir
    if args.command == "checkpoint-train-loop":
        # two forms: from a checkpoint on pre-tokenised inputs (the reference's gate run), or a
        # long run that writes periodic checkpoints
        if args.tokenized_inputs:
            resume = resume or args.checkpoint_root
        elif not save_dir:
            raise SystemExit("checkpoint-train-loop needs --tokenized-inputs (with --checkpoint-root) "
                             "or --save-dir")
    source = None
    # One process standing in for data-parallel rank R of N (no launcher): it reads the data
    # shard that rank would read. Under a launcher the ranks come from the environment.
    data_topo = topo
    if topo.world == 1 and args.data_parallel_rank is not None:
        n = args.data_parallel_ranks or args.data_parallel_rank + 1
        if not 0 <= args.data_parallel_rank < n:
            raise SystemExit(f"--data-parallel-rank {args.data_parallel_rank} outside 0..{n - 1}")
        data_topo = dataclasses.replace(topo, dp_rank=args.data_parallel_rank, dp_size=n)
    if args.tokenized_inputs:
        from .data.tokenized import FixedBatchSource
        source = FixedBatchSource(args.tokenized_inputs, mbs, data_topo.dp_rank, data_topo.dp_size,
                                  n_mb, pin=topo.device.type == "cuda")
        if args.seq_length is None:
            seq = source.seq_length
        elif seq != source.seq_length:
            raise SystemExit(f"--seq-length {seq} but the tokenised inputs have rows of "
                             f"{source.seq_length}")
    elif args.hf_dataset or args.hf_data_files:
        from .data.hf_dataloader import build_hf_dataloader
        source = build_hf_dataloader(args, spec, mbs, seq, data_topo)
    else:
        if topo.rank == 0:
            print("no --hf-dataset given: using synthetic uniform token ids", flush=True)
        if data_topo is not topo:
            from .data.synthetic import SyntheticTokenSource
            source = SyntheticTokenSource(spec.vocab_size, mbs, seq, seed=args.seed,
                                          dp_rank=data_topo.dp_rank, pin=topo.device.type == "cuda")
    out_dir = os.environ.get("OUTPUT_DIR")
    # --export-checkpoint-root names the directory that receives training_report.json
    # (reference: 0.5B __main__.py:520-530), --export-report a file; OUTPUT_DIR is the fallback
    report_path = args.export_report
    if report_path is None and args.export_checkpoint_root:
        report_path = str(Path(args.export_checkpoint_root) / "training_report.json")
    if report_path is None and out_dir:
        report_path = str(Path(out_dir) / "training_report.json")
    rep = run_training_loop(spec=spec, cfg=cfg, topo=topo, num_steps=num_steps, micro_batch_size=mbs,
                            seq_length=seq, num_local_microbatches=n_mb, seed=args.seed,
                            save_dir=save_dir, save_interval=args.save_interval, resume=resume,
                            data_source=source, dump_inputs_dir=args.dump_inputs_dir,
                            report_path=report_path)
    if topo.rank == 0:
        if out_dir:
            d = Path(out_dir) / f"{num_steps}step"
            d.mkdir(parents=True, exist_ok=True)
            with open(d / "ours_results.jsonl", "w") as f:
                for s in rep["steps"]:
                    # `step_time` is the 8B engine's name of the same figure
                    f.write(json.dumps({**s, "step_time": s.get("total_step_time")}) + "\n")
            (d / "DONE").write_text("ok\n")           # tombstone a job watcher polls for
        print("DONE", flush=True)
    shutdown()
    return 0


if __name__ == "__main__":
    sys.exit(main())
