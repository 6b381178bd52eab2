"""Spawn helper: run ``fn(rank, world, *args)`` in ``world`` CPU processes with gloo."""
import os
import socket
import traceback

import torch.multiprocessing as mp


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _pack(obj) -> bytes:
    """Results travel as plain bytes: tensors put on a multiprocessing queue are shared through
    file descriptors that die with the child, which may have exited before the parent reads."""
    import io
    import torch
    buf = io.BytesIO()
    torch.save(obj, buf)
    return buf.getvalue()


def _unpack(data: bytes):
    import io
    import torch
    return torch.load(io.BytesIO(data), map_location="cpu", weights_only=False)


def _entry(rank, world, port, fn, args, q):
    os.environ.update(RANK=str(rank), WORLD_SIZE=str(world), LOCAL_RANK=str(rank),
                      MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    try:
        out = fn(rank, world, *args)
        q.put((rank, "ok", _pack(out)))
    except BaseException as e:  # noqa: BLE001
        q.put((rank, "err", "".join(traceback.format_exception(e))))
    finally:
        import torch.distributed as dist
        if dist.is_initialized():
            dist.destroy_process_group()


def run_ranks(fn, world: int, *args, timeout: float = 600.0):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_entry, args=(r, world, port, fn, args, q)) for r in range(world)]
    for p in procs:
        p.start()
    results = {}
    try:
        for _ in range(world):
            rank, status, out = q.get(timeout=timeout)
            if status != "ok":
                raise RuntimeError(f"rank {rank} failed:\n{out}")
            results[rank] = _unpack(out)
    finally:
        for p in procs:
            p.join(timeout=30)
            if p.is_alive():
                p.kill()
    return [results[r] for r in range(world)]
