"""ctypes loader for the native sm_100a library.

The library is built in-tree by :mod:`forgetrain_b200.build` and exposes a plain C ABI
(raw device pointers + a CUDA stream handle). Loading is lazy; on a machine with a GPU a
missing library is an error (ops never fall back silently to PyTorch on CUDA tensors).
"""
from __future__ import annotations

import ctypes
import os
import threading
from pathlib import Path

import torch

_LIB = None
_LOCK = threading.Lock()
LIB_PATH = Path(os.environ.get("FT_B200_LIB") or
                Path(__file__).resolve().parent.parent / "lib" / "libft_b200.so")

c_int = ctypes.c_int
c_long = ctypes.c_int64
c_float = ctypes.c_float
c_void_p = ctypes.c_void_p


class NativeLibraryMissing(RuntimeError):
    pass


def lib():
    """Return the loaded native library, building it first when it is absent."""
    global _LIB
    if _LIB is not None:
        return _LIB
    with _LOCK:
        if _LIB is not None:
            return _LIB
        if not LIB_PATH.exists():
            if os.environ.get("FT_B200_NO_AUTOBUILD") == "1":
                raise NativeLibraryMissing(
                    f"{LIB_PATH} is missing; run `python -m forgetrain_b200.build`")
            from .. import build as _build
            _build.build()
        try:
            _LIB = _CountingLib(ctypes.CDLL(str(LIB_PATH)))
        except OSError as e:  # pragma: no cover - depends on the box
            raise NativeLibraryMissing(f"cannot load {LIB_PATH}: {e}") from e
        return _LIB


# kernels launched per entry point (entry points not listed launch one kernel)
_KERNELS_PER_CALL = {"ft_rmsnorm_bwd": 2, "ft_attn_bwd": 3, "ft_rmsnorm_bwd_partials": 0,
                     "ft_tmap_cache_clear": 0}
_LAUNCHES = [0]


class _CountingLib:
    """Forwards to the ctypes library and counts the kernels this process launched."""

    def __init__(self, cdll):
        self._cdll = cdll
        self._cache = {}

    def __getattr__(self, name):
        fn = self._cache.get(name)
        if fn is None:
            raw = getattr(self._cdll, name)
            n = _KERNELS_PER_CALL.get(name, 1)

            def fn(*a, _raw=raw, _n=n):
                _LAUNCHES[0] += _n
                return _raw(*a)
            self._cache[name] = fn
        return fn

    def has(self, name: str) -> bool:
        return hasattr(self._cdll, name)


def launch_count() -> int:
    return _LAUNCHES[0]


def reset_launch_count() -> None:
    _LAUNCHES[0] = 0


def available() -> bool:
    """True when CUDA kernels can run here (a GPU is visible and the library loads)."""
    if not torch.cuda.is_available():
        return False
    lib()
    return True


def ptr(t: torch.Tensor | None) -> c_void_p:
    return c_void_p(0 if t is None else t.data_ptr())


def stream() -> c_void_p:
    return c_void_p(torch.cuda.current_stream().cuda_stream)


_STATUS: dict[int, torch.Tensor] = {}

STATUS_MESSAGES = {
    1: "consumer timed out waiting for a TMA stage",
    2: "producer timed out waiting for a free stage",
    3: "epilogue timed out waiting for an accumulator",
    4: "MMA issuer timed out waiting for a drained accumulator",
    5: "a peer flag did not arrive in time",
    6: "bounded wait ran out",
}


def status_word(device: torch.device | int | None = None) -> torch.Tensor:
    """Per-device int32 word that kernels set when one of their bounded waits gives up."""
    dev = torch.cuda.current_device() if device is None else torch.device(device).index
    if dev is None:
        dev = torch.cuda.current_device()
    t = _STATUS.get(dev)
    if t is None:
        t = torch.zeros(4, dtype=torch.int32, device=f"cuda:{dev}")
        _STATUS[dev] = t
    return t


def check_status(device=None, reset: bool = True) -> None:
    """Synchronising check of the status word; raises if a kernel reported a failed wait."""
    t = status_word(device)
    code = int(t[0].item())
    if code != 0:
        if reset:
            t.zero_()
        raise RuntimeError(
            f"forgetrain_b200 kernel reported status {code}: {STATUS_MESSAGES.get(code, '?')}")


# What the entry points' negative return codes mean (one convention across the library; the exact
# condition is at the `return` site of the entry point in csrc/).
_RC_HINTS = {
    -1: "a shape or size precondition does not hold (dimension <= 0, or not a multiple the kernel needs)",
    -2: "an argument combination the entry point does not take (see its comment in csrc/)",
    -3: "a device memset or the scratch buffer of the call failed",
    -4: "no TMA descriptor for the first operand: base pointer not 16-byte aligned, or leading dimension "
        "not a multiple of 16 bytes",
    -5: "no TMA descriptor for the second operand: base pointer not 16-byte aligned, or leading dimension "
        "not a multiple of 16 bytes",
    -6: "no TMA descriptor for an output: base pointer not 16-byte aligned, or leading dimension not a "
        "multiple of 16 bytes",
    -7: "the grid of a kernel whose CTAs wait for one another would not be resident at once",
    -8: "no TMA descriptor for a scratch buffer of the call (the attention backward's fp32 accumulator)",
    -10: "the kernel's dynamic shared memory could not be reserved",
    -11: "the kernel launch failed",
    -100: "the kernel launch failed",
}


def check_rc(rc: int, what: str) -> None:
    if rc != 0:
        hint = _RC_HINTS.get(int(rc))
        raise RuntimeError(f"{what} failed with code {rc}" + (f": {hint}" if hint else ""))
