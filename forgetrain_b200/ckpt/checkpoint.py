"""Checkpoint save / resume in the reference's layout.

``<save_dir>/step_{N:07d}/training_state.pt`` holds ``{format_version: 1, step, num_samples,
param_names, params (compute dtype, CPU), optimizer_state {master_weights, exp_avg,
exp_avg_sq, step_count, num_samples}, dataloader_state}``
(exports/train_engine_0.5B/src/training_engine_tensor/parameters.py:547-674). Only rank 0
writes; the file is written as ``*.tmp`` and renamed, by a background thread with a single
writer at a time; a failure in the thread is re-raised by the next ``wait_for_async_save``.
Tensor-parallel runs add per-rank shards ``rank_<R>.pt`` next to it
(exports/train_engine_8b/src/training_engine_tensor/parameters.py:375-449).
"""
from __future__ import annotations

import os
import threading
from pathlib import Path

import torch

FORMAT_VERSION = 1
_writer_lock = threading.Lock()
_writer_thread: threading.Thread | None = None
_writer_error: list[BaseException] = []


def step_dir_name(step: int) -> str:
    return f"step_{step:07d}"


def should_save_after_step(step: int, num_steps_total: int, save_interval: int,
                           start_step: int = 0) -> bool:
    """Save every ``save_interval`` completed steps and after the final step; never at step 0.
    ``step`` is the 1-based count of completed steps."""
    if step <= 0 or step <= start_step:
        return False
    if step == num_steps_total:
        return True
    return save_interval > 0 and step % save_interval == 0


def wait_for_async_save() -> None:
    """Join the writer thread (if any) and re-raise what it failed with."""
    global _writer_thread
    t = _writer_thread
    if t is not None:
        t.join()
        _writer_thread = None
    if _writer_error:
        err = _writer_error.pop()
        _writer_error.clear()
        raise RuntimeError(f"asynchronous checkpoint write failed: {err}") from err


def _write_atomic(payload: dict, path: Path) -> None:
    tmp = path.with_suffix(path.suffix + ".tmp")
    try:
        torch.save(payload, tmp)
        os.replace(tmp, path)
    except BaseException:
        try:
            if tmp.exists():
                tmp.unlink()
        finally:
            raise


def save_checkpoint(save_dir: str | os.PathLike, step: int, *, params: dict, param_names: list,
                    optimizer_state: dict | None, num_samples: int = 0,
                    dataloader_state: dict | None = None, rank: int = 0, async_io: bool = True,
                    extra: dict | None = None, filename: str = "training_state.pt") -> Path | None:
    """Write one checkpoint. Non-zero ranks return ``None`` without touching the disk. Tensors
    are moved to the CPU on the caller's thread; serialisation happens in the background when
    ``async_io`` is set."""
    global _writer_thread
    if rank != 0:
        return None
    wait_for_async_save()
    out_dir = Path(save_dir) / step_dir_name(step)
    out_dir.mkdir(parents=True, exist_ok=True)
    payload = {
        "format_version": FORMAT_VERSION,
        "step": int(step),
        "num_samples": int(num_samples),
        "param_names": list(param_names),
        # a snapshot the writer thread owns: `.to("cpu")` copies device tensors but aliases host
        # ones, which training would go on modifying while the file is written
        "params": {k: (v.detach().to("cpu") if v.device.type != "cpu" else v.detach().clone())
                   for k, v in params.items()},
        "optimizer_state": optimizer_state,
        "dataloader_state": dataloader_state or {},
    }
    if extra:
        payload.update(extra)
    path = out_dir / filename

    def _run():
        try:
            _write_atomic(payload, path)
        except BaseException as e:  # surfaced by wait_for_async_save
            _writer_error.append(e)

    if async_io:
        with _writer_lock:
            _writer_thread = threading.Thread(target=_run, name="ckpt-writer", daemon=True)
            _writer_thread.start()
    else:
        _write_atomic(payload, path)
    return path


def latest_step_dir(root: str | os.PathLike, pattern: str = "training_state.pt") -> Path | None:
    """The ``step_<N>`` directory under ``root`` with the largest N that holds a finished file
    matching ``pattern``. By step NUMBER: names are zero-padded to 7 digits, so a plain sort
    would put step 10,000,000 before step 9,999,999; directories in which the writer never got
    to its rename are not resume points."""
    cands = []
    for p in Path(root).glob("step_*"):
        num = p.name[len("step_"):]
        if num.isdigit() and any(p.glob(pattern)):
            cands.append((int(num), p))
    return max(cands)[1] if cands else None


def latest_checkpoint(root: str | os.PathLike) -> Path | None:
    root = Path(root)
    if (root / "training_state.pt").exists():
        return root / "training_state.pt"
    d = latest_step_dir(root)
    return d / "training_state.pt" if d is not None else None


def load_resume_checkpoint(path: str | os.PathLike, expected_vocab: int | None = None) -> dict:
    """Load a checkpoint (a ``training_state.pt`` file, a step directory, or a save root whose
    latest step is taken). Validates the format version and the vocabulary size."""
    p = Path(path)
    if not p.exists():
        raise FileNotFoundError(f"checkpoint {str(p)!r} does not exist (expected a training_state.pt file, a "
                                f"step_<N> directory or a save directory that holds some)")
    if p.is_dir():
        f = latest_checkpoint(p)
        if f is None:
            raise FileNotFoundError(f"no training_state.pt under {p}")
        p = f
    state = torch.load(p, map_location="cpu", weights_only=False)
    ver = state.get("format_version")
    if ver != FORMAT_VERSION:
        raise ValueError(f"unsupported checkpoint format_version {ver!r} (expected {FORMAT_VERSION})")
    if expected_vocab is not None and "tok_embeddings.weight" in state["params"]:
        v = state["params"]["tok_embeddings.weight"].shape[0]
        if v != expected_vocab:
            raise ValueError(f"checkpoint vocabulary {v} != model vocabulary {expected_vocab}")
    return state
