"""Host-side fault injection for recovery tests.

``FT_INJECT_FAILURE="step=K[,rank=R][,once=PATH][,exit=CODE]"`` makes rank R (default 0) fail
right before optimizer step K (1-based) starts, i.e. with K-1 steps done and no kernel or
collective of its own in flight: it raises ``InjectedFailure`` (or leaves through ``os._exit(CODE)``
when ``exit`` is given, the shape of a killed process). With ``once=PATH`` the failure happens only
while PATH does not exist and creates it first, so a relaunched job passes the same step.

Failures are injected on the host only: nothing here touches the device, and a rank leaves between
steps. What the other ranks then see is what they would see after any lost peer: the launcher
ends them, or their next collective times out.
"""
from __future__ import annotations

import os


class InjectedFailure(RuntimeError):
    pass


def parse(text: str | None) -> dict | None:
    if not text:
        return None
    out = {"rank": 0, "once": None, "exit": None}
    for part in text.split(","):
        key, sep, val = part.strip().partition("=")
        if not sep or key not in ("step", "rank", "once", "exit"):
            raise ValueError(f"FT_INJECT_FAILURE: cannot read {part!r} (step=K[,rank=R][,once=PATH][,exit=CODE])")
        out[key] = val if key == "once" else int(val)
    if "step" not in out:
        raise ValueError("FT_INJECT_FAILURE needs step=K")
    return out


def maybe_fail(next_step: int, rank: int, env=None) -> None:
    """Call at the top of the training loop with the 1-based number of the step about to run."""
    spec = parse(os.environ.get("FT_INJECT_FAILURE") if env is None else env.get("FT_INJECT_FAILURE"))
    if spec is None or spec["step"] != next_step or spec["rank"] != rank:
        return
    if spec["once"]:
        try:
            fd = os.open(spec["once"], os.O_CREAT | os.O_EXCL | os.O_WRONLY)
        except FileExistsError:
            return
        os.write(fd, f"failed before step {next_step} on rank {rank}\n".encode())
        os.close(fd)
    try:        # leave with nothing of this rank in flight on a device
        import torch
        if torch.cuda.is_available() and torch.cuda.is_initialized():
            torch.cuda.synchronize()
    except ImportError:
        pass
    if spec["exit"] is not None:
        os._exit(spec["exit"])
    raise InjectedFailure(f"injected failure before step {next_step} on rank {rank}")
