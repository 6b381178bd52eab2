#!/usr/bin/env python
"""Headline benchmark: MiniCPM4-0.5B pretraining step, data parallel over N GPUs of one node.

    python bench.py --gpus N --steps K --warmup W            (N > 1: launched by torchrun)
    python bench.py --impl reference ...                      (the reference's own engine)

Primary config (the reference's 0.5B model at the benchmark shape): 24 layers, hidden 1024, 16
query / 2 KV heads of 64, SwiGLU 4096, vocab 73448, muP scaling; sequence 4096, micro-batch 4 per
GPU, one micro-batch per step, bf16 compute with fp32 master weights and fp32 gradient
accumulation, ZeRO-1 AdamW, bucketed gradient reduction overlapped with backward, parameter
update + all-gather overlapped with the next forward. Synthetic uniform token ids, random-init
weights. Weak scaling: per-GPU work is fixed.

Secondary config (N = 2, 4, 8; reported under ``"secondary"`` of the same JSON line): MiniCPM4-8B
with tensor parallelism 2 x data parallelism N/2, sequence-parallel activations, sequence 4096,
micro-batch 1, gradient accumulation 8, peer-memory collectives (the second headline of the
reference: TP=2 x DP=4 on one 8-GPU node).

Two numbers are measured per config, both as whole-job tokens/s:
  * ``value``  K steps timed with CUDA events between barriers, inputs already resident;
  * ``e2e``    K steps through ``Trainer.train_step`` fed by the pinned-memory prefetcher, with
               the host-to-device copy of every step's batch and a device-to-host read of the
               loss inside the timed region.
The step's working set (several GB of activations) is far larger than L2, so no explicit L2
flush is needed between iterations. One JSON line is printed by rank 0.
"""
from __future__ import annotations

import argparse
import gc
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

METRIC = "tokens_per_sec"
MODEL = "minicpm4-0.5b"
SEQ, MBS = 4096, 4
NOMINAL_BF16_TFLOPS = 2250.0       # B200 dense bf16, the like-for-like denominator of a published MFU
PUBLISHED_MFU = {"0.5b": 0.4413, "8b": 0.509}   # the reference's headlines (H100, nominal peak)
T_START = time.time()


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
         "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu = gpu_index
        self.proc = None
        self.lines: list[str] = []
        self.thread = None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "200",
                 "-i", str(self.gpu)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except Exception:
            self.proc = None
            return
        self.thread = threading.Thread(target=self._pump, daemon=True)
        self.thread.start()

    def _pump(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, mx, reasons, power = [], [], set(), []
        for ln in self.lines:
            parts = [p.strip() for p in ln.split(",")]
            if len(parts) < 9:
                continue
            try:
                sm.append(float(parts[1]))
                mx.append(float(parts[2]))
                power.append(float(parts[3]))
            except ValueError:
                continue
            for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown",
                                  "sw_power_cap"), parts[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None,
                "sm_max_mhz": max(mx) if mx else None,
                "power_w_max": max(power) if power else None,
                "samples": len(sm), "reasons": sorted(reasons)}


# ---------------------------------------------------------------------------------------------
# reference arm
# ---------------------------------------------------------------------------------------------
def _reference_unavailable(why: str) -> int:
    if int(os.environ.get("RANK", "0")) == 0:
        print(json.dumps({"impl": "reference", "unavailable": why}), flush=True)
    return 0


def run_reference(args) -> int:
    """Drive the UNMODIFIED reference 0.5B engine (installed under ``baseline/_ref/e05``) through
    its own command line (``python -m training_engine_tensor pretrain``) on a generated local
    text corpus of the benchmark's shape, and turn its per-iteration ``time(ms)`` lines into
    the same JSON line. Its kernels module imports TransformerEngine at import time and its
    stock path calls TransformerEngine for RMSNorm, attention, the weight-gradient GEMM and
    Adam; when that package cannot be imported nothing of the engine can run, and the arm says
    so in the agreed shape."""
    ref_root = os.path.join(ROOT, "baseline", "_ref", "e05")
    if not os.path.isdir(os.path.join(ref_root, "training_engine_tensor")):
        return _reference_unavailable(
            "the reference 0.5B engine is not installed under baseline/_ref/e05 (offline "
            "install: pip --no-index --no-deps --target baseline/_ref/e05 of a /tmp copy of "
            "exports/train_engine_0.5B)")
    probe = subprocess.run([sys.executable, "-c", "import transformer_engine, transformer_engine_torch"],
                           capture_output=True, text=True)
    if probe.returncode != 0:
        last = (probe.stderr.strip().splitlines() or ["import failed"])[-1]
        return _reference_unavailable(
            "reference 0.5B engine installed under baseline/_ref/e05 but not runnable: "
            "training_engine_tensor/kernels.py:31 imports transformer_engine at module import and "
            "its stock path calls it for RMSNorm, attention, wgrad GEMM and Adam; "
            f"transformer_engine is not installed and no wheel exists offline ({last})")
    # TransformerEngine is present: run the engine's own CLI. Its ``pretrain`` sub-command has no
    # synthetic source, so it gets a generated corpus and a word-level tokenizer written locally.
    rank = int(os.environ.get("RANK", "0"))
    import tempfile
    work = os.path.join(tempfile.gettempdir(), "ft_reference_arm")
    try:
        if rank == 0:
            _write_reference_corpus(work, args.seq, args.mbs * max(args.gpus, 1) * (args.steps + args.warmup + 2))
        env = dict(os.environ, PYTHONPATH=ref_root + os.pathsep + os.environ.get("PYTHONPATH", ""))
        cmd = [sys.executable, "-m", "training_engine_tensor", "pretrain",
               "--num-steps", str(args.steps + args.warmup), "--micro-batch-size", str(args.mbs),
               "--global-batch-size", str(args.mbs * max(args.gpus, 1)), "--seq-length", str(args.seq),
               "--hf-dataset", os.path.join(work, "data"), "--tokenizer-path", os.path.join(work, "tok")]
        out = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=780)
        if out.returncode != 0:
            tail = " | ".join((out.stderr or out.stdout).strip().splitlines()[-3:])
            return _reference_unavailable(f"the reference CLI exited {out.returncode}: {tail[:400]}")
        import re
        ms = [float(m) for m in re.findall(r"time\(ms\):\s*([0-9.]+)", out.stdout)]
        ms = ms[args.warmup:]
        if not ms:
            return _reference_unavailable("the reference CLI printed no per-iteration time lines")
        step_ms = sum(ms) / len(ms)
        tokens = args.mbs * args.seq * max(args.gpus, 1)
        if rank == 0:
            print(json.dumps({"impl": "reference", "metric": METRIC, "value": tokens / (step_ms / 1e3),
                              "unit": "tokens/s", "n_gpus": max(args.gpus, 1), "steps": len(ms),
                              "warmup": args.warmup, "ms_per_step": step_ms, "higher_is_better": True,
                              "scaling": "weak", "dtype": "bf16", "data": "synthetic text corpus",
                              "config": {"model": MODEL, "global_batch": args.mbs * max(args.gpus, 1),
                                         "seq_len": args.seq, "parallelism": f"dp{max(args.gpus, 1)}"},
                              "timing": "the engine's own per-iteration wall time"}), flush=True)
        return 0
    except Exception as e:  # noqa: BLE001
        return _reference_unavailable(f"driving the reference CLI failed: {type(e).__name__}: {e}")


def _write_reference_corpus(work: str, seq: int, rows: int) -> None:
    """What the reference's ``pretrain`` needs in place of a synthetic source: ``work/data`` with a
    JSON-lines corpus of random words (a directory, which its ``datasets.load_dataset(path,
    split="train")`` call resolves to the json builder; the tokenizer files must not sit next to
    it or they would be read as data) and ``work/tok`` with a word-level tokenizer that
    ``AutoTokenizer.from_pretrained`` loads (its ``--tokenizer-path``)."""
    import random
    data, tokdir = os.path.join(work, "data"), os.path.join(work, "tok")
    os.makedirs(data, exist_ok=True)
    os.makedirs(tokdir, exist_ok=True)
    rnd = random.Random(0)
    vocab = [f"w{i}" for i in range(4096)]
    with open(os.path.join(data, "corpus.jsonl"), "w") as f:
        for _ in range(rows):
            f.write(json.dumps({"text": " ".join(rnd.choice(vocab) for _ in range(seq + 8))}) + "\n")
    from tokenizers import Tokenizer, models, pre_tokenizers
    tok = Tokenizer(models.WordLevel({w: i for i, w in enumerate(["<unk>", "</s>"] + vocab)}, unk_token="<unk>"))
    tok.pre_tokenizer = pre_tokenizers.Whitespace()
    tok.save(os.path.join(tokdir, "tokenizer.json"))
    with open(os.path.join(tokdir, "tokenizer_config.json"), "w") as f:
        json.dump({"tokenizer_class": "PreTrainedTokenizerFast", "eos_token": "</s>", "unk_token": "<unk>"}, f)


# ---------------------------------------------------------------------------------------------
# our arm
# ---------------------------------------------------------------------------------------------
def time_config(*, model: str, tp: int, mbs: int, gas: int, seq: int, K: int, W: int, comm: str,
                graph: int, sequence_parallel: bool = True) -> dict:
    """Build the engine for one config, warm it up, time K steps on the device and K steps end
    to end, and return the raw figures (rank 0 gets the clock record)."""
    import torch
    import torch.distributed as dist

    from forgetrain_b200 import config as cfgmod
    from forgetrain_b200.config import load_model_spec
    from forgetrain_b200.data.prefetch import DataPrefetcher
    from forgetrain_b200.data.synthetic import SyntheticTokenSource
    from forgetrain_b200.engine_config import from_spec
    from forgetrain_b200.ops import _lib
    from forgetrain_b200.parallel.topology import init_topology
    from forgetrain_b200.trainer import Trainer

    spec = load_model_spec(model)
    cfg = from_spec(spec, dtype="bf16", comm=comm, tensor_parallel_size=tp,
                    sequence_parallel=sequence_parallel, init_scheme="normal", init_std=0.02,
                    step_cuda_graph=graph == 1, full_step_cuda_graph=graph == 2)
    topo = init_topology(tp, num_kv_groups=spec.num_query_groups)
    trainer = Trainer(spec, cfg, topo, seq_length=seq, micro_batch_size=mbs, seed=1234)
    source = SyntheticTokenSource(spec.vocab_size, mbs, seq, seed=1234, dp_rank=topo.dp_rank, pin=True)
    prefetch = DataPrefetcher(source, topo.device, depth=min(4, max(2, gas)))

    def barrier():
        if topo.world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def next_step_batches():
        return [next(prefetch) for _ in range(gas)]

    # ---- warm-up (also builds tensor maps, allocator pools, NCCL / peer-memory state)
    # a graph mode runs its own eager calls first and captures on the call after them: all of
    # that belongs to the warm-up, not to the timed region
    extra = cfg.step_cuda_graph_warmup + 1 if graph else 0
    for _ in range(W + extra):
        out = trainer.train_step(next_step_batches())
    trainer.finish_step()
    barrier()
    _lib.check_status(topo.device)

    # ---- device-timed region: inputs already resident on the device
    resident = [next_step_batches() for _ in range(min(K, 2))]
    torch.cuda.synchronize()
    sampler = ClockSampler(torch.cuda.current_device())
    if topo.rank == 0:
        sampler.start()
    _lib.reset_launch_count()
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(K):
        out = trainer.train_step(resident[i % len(resident)])
    trainer.finish_step()          # the last step's update / all-gather tail is inside the region
    e1.record()
    barrier()
    launches = _lib.launch_count()
    dev_ms = e0.elapsed_time(e1)

    # ---- end-to-end region: pinned host batches -> H2D every step, loss read back every step
    barrier()
    t0 = time.perf_counter()
    h2d = 0
    last_loss = 0.0
    pending = None
    for i in range(K):
        h2d = 0
        batches = []
        for _ in range(gas):
            batches.append(next(prefetch))
            h2d += prefetch.bytes_last
        out = trainer.train_step(batches)
        # device -> host: the loss (and gradient norm) of EVERY step is copied into pinned memory
        # inside the region; the host consumes it one step late, so it stays ahead of the device
        handle = trainer.loss_to_host_async()
        if pending is not None:
            last_loss, _ = pending.value()
        pending = handle
    last_loss, _ = pending.value()
    trainer.finish_step()
    torch.cuda.synchronize()
    e2e_s = time.perf_counter() - t0
    clocks = sampler.stop() if topo.rank == 0 else {}
    _lib.check_status(topo.device)

    # ---- the bf16 parameter buffer must be bit-identical on every data-parallel rank: with the
    # reference's hyper-parameters (2000 warm-up iterations) the loss cannot show a broken gather
    csum = trainer.store.flat_params.view(torch.int16).to(torch.int64).sum().reshape(1)
    lo, hi = csum.clone(), csum.clone()
    if topo.dp_size > 1:
        dist.all_reduce(lo, op=dist.ReduceOp.MIN, group=topo.dp_group)
        dist.all_reduce(hi, op=dist.ReduceOp.MAX, group=topo.dp_group)
    params_equal = torch.tensor([1.0 if int(lo) == int(hi) else 0.0], device=topo.device)
    t = torch.tensor([dev_ms, e2e_s * 1e3], dtype=torch.float64, device=topo.device)
    if topo.world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        dist.all_reduce(params_equal, op=dist.ReduceOp.MIN)
    dev_ms, e2e_ms = float(t[0]), float(t[1])
    tokens_per_step = mbs * seq * gas * topo.dp_size
    step_s = dev_ms / 1e3 / K
    flops_std = cfgmod.compute_training_flops_standard(spec, tokens_per_step, seq)
    flops_hw = cfgmod.compute_training_flops(spec, tokens_per_step, seq)
    res = {
        "world": topo.world, "dp": topo.dp_size, "tp": tp, "rank": topo.rank,
        "tokens_per_step": tokens_per_step, "ms_per_step": dev_ms / K,
        "value": tokens_per_step * K / (dev_ms / 1e3),
        "e2e_value": tokens_per_step * K / (e2e_ms / 1e3), "e2e_ms_per_step": e2e_ms / K,
        "h2d_bytes_per_step": int(h2d), "launches": int(launches), "clocks": clocks,
        "loss": last_loss, "params_equal": bool(float(params_equal) == 1.0),
        "param_checksum": int(csum),
        "mfu_standard": flops_std / step_s / (cfgmod.peak_tflops() * 1e12 * topo.world),
        "mfu_hardware": flops_hw / step_s / (cfgmod.peak_tflops() * 1e12 * topo.world),
        "mfu_standard_nominal": flops_std / step_s / (NOMINAL_BF16_TFLOPS * 1e12 * topo.world),
        "peak_tflops_used": cfgmod.peak_tflops(),
    }
    # release everything this config held (the next one needs the memory and fresh buffers)
    del trainer, prefetch, source, resident, out
    gc.collect()
    torch.cuda.empty_cache()
    barrier()
    return res


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=8)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--comm", default=os.environ.get("FT_COMM", "fused"), choices=["fused", "nccl"])
    ap.add_argument("--model", default="0.5b")
    ap.add_argument("--seq", type=int, default=SEQ)
    ap.add_argument("--mbs", type=int, default=MBS)
    ap.add_argument("--graph", type=int, default=int(os.environ.get("FT_BENCH_GRAPH", "0")),
                    help="0: eager; 1: CUDA graph of fwd + loss + bwd per micro-batch; "
                         "2: one graph for the whole optimizer step")
    ap.add_argument("--secondary", type=int, default=int(os.environ.get("FT_BENCH_SECONDARY", "1")),
                    help="1: at 2, 4 or 8 GPUs also time MiniCPM4-8B TP=2 x DP=N/2")
    args = ap.parse_args()
    if args.impl == "reference":
        return run_reference(args)

    import torch

    from forgetrain_b200.parallel.topology import shutdown

    world = int(os.environ.get("WORLD_SIZE", "1"))
    if world != args.gpus and args.gpus > 1 and world == 1:
        raise SystemExit("launch N>1 with: python -m torch.distributed.run --nnodes=1 "
                         f"--nproc-per-node {args.gpus} --master-addr 127.0.0.1 bench.py ...")
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device")
    W = max(args.warmup, 3)
    K = args.steps
    rank = int(os.environ.get("RANK", "0"))

    r = time_config(model=args.model, tp=1, mbs=args.mbs, gas=1, seq=args.seq, K=K, W=W,
                    comm=args.comm, graph=args.graph)

    secondary = None
    if args.secondary and world in (2, 4, 8) and args.model == "0.5b":
        if time.time() - T_START > 420:
            secondary = {"skipped": "the primary config used the time budget"}
        else:
            try:
                Ks, Ws = min(K, 5), 3
                s = time_config(model="8b", tp=2, mbs=1, gas=8, seq=4096, K=Ks, W=Ws,
                                comm=args.comm, graph=0)
                secondary = {
                    "metric": METRIC, "value": s["value"], "unit": "tokens/s",
                    "tokens_per_sec_per_gpu": s["value"] / s["world"], "ms_per_step": s["ms_per_step"],
                    "steps": Ks, "warmup": Ws, "n_gpus": s["world"],
                    "config": {"model": "minicpm4-8b", "parallelism": f"tp2 x dp{s['dp']}, sequence parallel",
                               "seq_len": 4096, "micro_batch": 1, "grad_accum": 8,
                               "global_batch": 8 * s["dp"], "comm": args.comm,
                               "optimizer": "adamw fp32 master, zero-1 over dp"},
                    "mfu_standard": s["mfu_standard"], "mfu_standard_nominal_peak": s["mfu_standard_nominal"],
                    "mfu_vs_published_mfu": s["mfu_standard_nominal"] / PUBLISHED_MFU["8b"],
                    "e2e": {"value": s["e2e_value"], "unit": "tokens/s", "ms_per_step": s["e2e_ms_per_step"],
                            "h2d_bytes_per_step": s["h2d_bytes_per_step"], "d2h_bytes_per_step": 8},
                    "gpu_launches": s["launches"], "clocks": s["clocks"], "loss": s["loss"],
                    "params_identical_across_dp_ranks": s["params_equal"],
                }
            except Exception as e:  # noqa: BLE001  (the primary line must still go out)
                secondary = {"error": f"{type(e).__name__}: {e}"[:400]}

    if rank == 0:
        line = {
            "metric": METRIC, "value": r["value"], "unit": "tokens/s", "n_gpus": r["world"], "steps": K,
            "warmup": W, "ms_per_step": r["ms_per_step"], "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"model": MODEL if args.model == "0.5b" else args.model,
                       "global_batch": args.mbs * r["world"], "micro_batch_per_gpu": args.mbs,
                       "seq_len": args.seq, "parallelism": f"dp{r['world']}", "comm": args.comm,
                       "optimizer": "adamw fp32 master, zero-1",
                       "cuda_graph": {0: False, 1: "compute step", 2: "whole step"}.get(args.graph, False),
                       # the whole-step graph (--graph 2) is built and tested; it is not the default
                       # because the step is device-bound (replay and eager differ by < 0.5 %) and a
                       # replay cannot overlap the parameter update with the next step's forward
                       "cuda_graph_note": "eager by default: device-bound step, see --graph 2",
                       "l2": "inputs larger than L2 (multi-GB activations per step)"},
            "tokens_per_sec_per_gpu": r["value"] / r["world"],
            "mfu_standard": r["mfu_standard"], "mfu_hardware": r["mfu_hardware"],
            "peak_tflops_used": r["peak_tflops_used"],
            # MFU against the nominal dense bf16 peak (2.25 PFLOP/s), the convention of the
            # reference's published 44.13 % (H100 nominal peak); the ratio below is nominal / nominal
            "mfu_standard_nominal_peak": r["mfu_standard_nominal"],
            "mfu_vs_published_mfu": r["mfu_standard_nominal"] / PUBLISHED_MFU["0.5b"]
            if args.model == "0.5b" else None,
            "e2e": {"value": r["e2e_value"], "unit": "tokens/s", "ms_per_step": r["e2e_ms_per_step"],
                    "h2d_bytes_per_step": r["h2d_bytes_per_step"], "d2h_bytes_per_step": 8,
                    "d2h": "loss and gradient norm of every step, consumed one step late"},
            "gpu_launches": r["launches"],
            "clocks": r["clocks"],
            "loss": r["loss"],
            "params_identical_across_dp_ranks": r["params_equal"],
            "param_checksum": r["param_checksum"],
            "impl": "ours",
        }
        if secondary is not None:
            line["secondary"] = secondary
        print(json.dumps(line), flush=True)
    shutdown()
    return 0


if __name__ == "__main__":
    sys.exit(main())
