"""Environment check: ``python -m forgetrain_b200.doctor [--build] [--json] [--self-test]``.

Prints what the engine will find on this machine (interpreter, PyTorch, CUDA device and its
compute capability, compilers, the in-tree native libraries, the measured-peak file used for the
MFU lines, the distributed backends) and exits 0 when a training run can start here: on a GPU box
that means an sm_100 device plus a loadable native library, elsewhere the CPU path. The counterpart
of the reference's "verify install" step (0.5B README.md:149-153). ``--self-test`` also trains: three
steps of a small model on the device this machine offers (two decoder blocks of the 0.5B geometry on a
GPU through the native kernels, the tiny spec in fp32 on the CPU otherwise) and checks that the loss
of a repeated batch falls."""
from __future__ import annotations

import json
import shutil
import sys
from pathlib import Path


def collect(build: bool = False) -> dict:
    import torch
    import torch.distributed as dist
    from . import build as b
    from . import config as cfgmod
    info: dict = {"python": sys.version.split()[0], "torch": torch.__version__,
                  "torch_cuda": torch.version.cuda, "nvcc": shutil.which("nvcc"),
                  "gxx": shutil.which("g++"),
                  "backends": {"nccl": dist.is_nccl_available(), "gloo": dist.is_gloo_available()}}
    cuda = torch.cuda.is_available()
    info["cuda_available"] = cuda
    info["devices"] = []
    if cuda:
        for i in range(torch.cuda.device_count()):
            p = torch.cuda.get_device_properties(i)
            info["devices"].append({"index": i, "name": p.name, "sm": f"{p.major}{p.minor}",
                                    "sms": p.multi_processor_count,
                                    "memory_gb": round(p.total_memory / 2 ** 30, 1)})
    lib = Path(b.LIB_PATH)
    if build and not lib.exists():
        b.build()
    info["native_library"] = {"path": str(lib), "built": lib.exists(),
                              "sources": [Path(s).name for s in b.sources()]}
    info["reference_library_built"] = Path(b.REF_LIB_PATH).exists()
    info["peak_tflops_for_mfu"] = cfgmod.peak_tflops()
    problems = []
    if cuda:
        if not any(d["sm"].startswith("10") for d in info["devices"]):
            problems.append("no sm_100 device: the CUDA kernels are built for sm_100a only")
        if not lib.exists():
            problems.append("native library not built: run python -m forgetrain_b200.build")
    else:
        problems.append("no CUDA device: only the CPU (fp32, gloo) path can run here")
    info["problems"] = problems
    info["can_train_on_gpu"] = cuda and not problems
    info["can_train_on_cpu"] = True
    return info


def self_test() -> dict:
    """Three optimizer steps on one repeated batch; returns ``{"device", "losses", "ok"}``."""
    import torch
    from .config import load_model_spec
    from .engine_config import from_spec
    from .parallel.topology import Topology
    from .trainer import Trainer
    cuda = torch.cuda.is_available()
    if cuda:
        torch.cuda.set_device(0)
        spec = load_model_spec("0.5b", num_layers=2, seq_length=512, max_position_embeddings=512)
        dev, dtype, seq, mbs = torch.device("cuda", 0), "bf16", 512, 2
    else:
        spec = load_model_spec("tiny", num_layers=2, seq_length=64, max_position_embeddings=64)
        dev, dtype, seq, mbs = torch.device("cpu"), "fp32", 64, 2
    cfg = from_spec(spec, dtype=dtype, comm="nccl", warmup_iters=0, max_lr=1e-3)
    trainer = Trainer(spec, cfg, Topology(device=dev), seq_length=seq, micro_batch_size=mbs, seed=0)
    chunk = torch.randint(0, spec.vocab_size, (mbs, seq + 1), generator=torch.Generator().manual_seed(0))
    batch = {"tokens": chunk[:, :-1].contiguous().to(dev), "labels": chunk[:, 1:].contiguous().to(dev),
             "loss_mask": torch.ones(mbs, seq, device=dev)}
    losses = [float(trainer.train_step([batch])["loss"]) for _ in range(3)]
    if cuda:
        from .ops import _lib
        torch.cuda.synchronize()
        _lib.check_status()
    ok = all(l == l and abs(l) < 1e4 for l in losses) and losses[-1] < losses[0]
    return {"device": str(dev), "losses": losses, "ok": ok}


def main(argv: list[str] | None = None) -> int:
    argv = sys.argv[1:] if argv is None else argv
    info = collect(build="--build" in argv)
    if "--self-test" in argv and (info["can_train_on_gpu"] or not info["cuda_available"]):
        info["self_test"] = self_test()
    if "--json" in argv:
        print(json.dumps(info, indent=1))
    else:
        print(f"python {info['python']}  torch {info['torch']} (CUDA {info['torch_cuda']})")
        print(f"nvcc: {info['nvcc'] or 'not found'}   g++: {info['gxx'] or 'not found'}")
        print(f"backends: nccl={info['backends']['nccl']} gloo={info['backends']['gloo']}")
        for d in info["devices"]:
            print(f"  cuda:{d['index']} {d['name']} sm_{d['sm']} {d['sms']} SMs {d['memory_gb']} GiB")
        nl = info["native_library"]
        print(f"native library: {'built' if nl['built'] else 'NOT built'} ({nl['path']})")
        print(f"peak used for MFU: {info['peak_tflops_for_mfu']:.1f} TFLOP/s")
        for p in info["problems"]:
            print(f"note: {p}")
        print("GPU training: " + ("ready" if info["can_train_on_gpu"] else "not available here")
              + "; CPU path: ready")
        if "self_test" in info:
            t = info["self_test"]
            print(f"self-test on {t['device']}: losses {' -> '.join(f'{l:.4f}' for l in t['losses'])}: "
                  + ("ok" if t["ok"] else "FAILED"))
    if "self_test" in info and not info["self_test"]["ok"]:
        return 1
    return 0 if (info["can_train_on_gpu"] or not info["cuda_available"]) else 1


if __name__ == "__main__":
    sys.exit(main())
