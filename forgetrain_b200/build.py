"""In-tree build of the native library (``forgetrain_b200/lib/libft_b200.so``).

Every ``csrc/*.cu`` file is compiled for sm_100a only
(``-gencode arch=compute_100a,code=sm_100a``) and linked into one shared object with a plain
C ABI that :mod:`forgetrain_b200.ops._lib` loads through ``ctypes``. nvcc cross-compiles, so
the build needs no GPU. Objects are rebuilt only when their source (or a header) changed.

The host C++ reference ops of ``csrc/ref_cpu`` are built with g++ into
``forgetrain_b200/lib/libft_ref_cpu.so`` by the same command.

Usage: ``python -m forgetrain_b200.build [--force] [--verbose]``
"""
from __future__ import annotations

import hashlib
import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

PKG_DIR = Path(__file__).resolve().parent
CSRC = PKG_DIR / "csrc"
OBJ_DIR = CSRC / "build"
LIB_DIR = PKG_DIR / "lib"
LIB_PATH = LIB_DIR / "libft_b200.so"
REF_SRC = CSRC / "ref_cpu" / "ref_ops.cpp"
REF_LIB_PATH = LIB_DIR / "libft_ref_cpu.so"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=default",
    "--expt-relaxed-constexpr",
]


def _nvcc() -> str:
    cand = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(cand):
        raise RuntimeError("nvcc not found; the native library cannot be built")
    return cand


def _headers_digest() -> str:
    h = hashlib.sha256()
    for p in sorted(list(CSRC.glob("*.cuh")) + list(CSRC.glob("*.h"))):
        h.update(p.name.encode())
        h.update(p.read_bytes())
    h.update(" ".join(NVCC_FLAGS).encode())
    return h.hexdigest()


def _needs_build(src: Path, obj: Path, stamp: str) -> bool:
    tag = obj.with_suffix(".tag")
    if not obj.exists() or not tag.exists():
        return True
    want = hashlib.sha256(src.read_bytes()).hexdigest() + stamp
    return tag.read_text() != want


def _compile(src: Path, obj: Path, stamp: str, verbose: bool) -> str:
    cmd = [_nvcc(), *NVCC_FLAGS, "-I", str(CSRC), "-c", str(src), "-o", str(obj)]
    if verbose:
        cmd.insert(1, "-Xptxas")
        cmd.insert(2, "-v")
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"nvcc failed for {src.name}:\n{r.stdout}\n{r.stderr}")
    obj.with_suffix(".tag").write_text(hashlib.sha256(src.read_bytes()).hexdigest() + stamp)
    return r.stderr if verbose else ""


def sources() -> list[Path]:
    return sorted(CSRC.glob("*.cu"))


def build(force: bool = False, verbose: bool = False) -> Path:
    """Compile what is stale and link the shared library; returns its path."""
    OBJ_DIR.mkdir(parents=True, exist_ok=True)
    LIB_DIR.mkdir(parents=True, exist_ok=True)
    stamp = _headers_digest()
    srcs = sources()
    objs = [OBJ_DIR / (s.stem + ".o") for s in srcs]
    todo = [(s, o) for s, o in zip(srcs, objs) if force or _needs_build(s, o, stamp)]
    if todo:
        with ThreadPoolExecutor(max_workers=min(8, len(todo))) as ex:
            for log in ex.map(lambda so: _compile(so[0], so[1], stamp, verbose), todo):
                if log:
                    print(log, file=sys.stderr)
    if todo or not LIB_PATH.exists():
        tmp = LIB_PATH.with_suffix(".so.tmp")
        cmd = [_nvcc(), "-shared", "-o", str(tmp), *[str(o) for o in objs],
               "-gencode", "arch=compute_100a,code=sm_100a"]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"link failed:\n{r.stdout}\n{r.stderr}")
        os.replace(tmp, LIB_PATH)
    return LIB_PATH


def build_ref_cpu(force: bool = False) -> Path:
    """Compile the host C++ reference ops (``csrc/ref_cpu``) with g++ and OpenMP."""
    LIB_DIR.mkdir(parents=True, exist_ok=True)
    tag = REF_LIB_PATH.with_suffix(".tag")
    want = hashlib.sha256(REF_SRC.read_bytes()).hexdigest()
    if not force and REF_LIB_PATH.exists() and tag.exists() and tag.read_text() == want:
        return REF_LIB_PATH
    cxx = shutil.which("g++") or shutil.which("c++")
    if cxx is None:
        raise RuntimeError("g++ not found; the host reference library cannot be built")
    tmp = REF_LIB_PATH.with_suffix(".so.tmp")
    cmd = [cxx, "-O2", "-std=c++17", "-fPIC", "-shared", "-fopenmp", str(REF_SRC), "-o", str(tmp)]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"g++ failed for {REF_SRC.name}:\n{r.stdout}\n{r.stderr}")
    os.replace(tmp, REF_LIB_PATH)
    tag.write_text(want)
    return REF_LIB_PATH


def main() -> None:
    force = "--force" in sys.argv
    verbose = "--verbose" in sys.argv
    path = build(force=force, verbose=verbose)
    ref = build_ref_cpu(force=force)
    print(f"built {ref}")
    print(f"built {path} ({path.stat().st_size / 1e6:.1f} MB) from {len(sources())} sources")


if __name__ == "__main__":
    main()
