#!/usr/bin/env python
"""Kernel and collective micro-benchmarks (device-timed with CUDA events, L2 flushed between
iterations, bf16 inputs N(0,1) from a fixed seed).

    python microbench.py attn  [--batch 4] [--seq 4096] [--shape 0.5b|8b] [--iters 20]
    python microbench.py gemm  [--tokens 16384] [--shape 0.5b|8b-tp2]
    python microbench.py elem  [--tokens 16384]
    python microbench.py comm  (under torchrun, N >= 2)  bucket reduce-scatter / all-gather sweep
    python microbench.py tp    (under torchrun, N = TP degree)  fused AG->GEMM / GEMM->RS [--tokens 4096]

Every sub-command prints one JSON line per case with the achieved rate and its fraction of the
measured peak (``MEASURED_PEAKS.json`` when present, else the stated fallback), and a ``clocks``
record: SM clock and throttle reasons read through NVML right after every timed iteration
(median clock, union of the reasons seen). ``--once`` runs each kernel a single time after one
warm-up, for captures under a profiler.
"""
from __future__ import annotations

import argparse
import json
import os
import sys

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

import torch  # noqa: E402


def peaks() -> dict:
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return {"hbm_gbs": d["hbm_gbs"], "bf16_tflops": d["bf16_tflops"], "kind": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "kind": "fallback"}


_flush_buf = None


class _Clocks:
    """SM clock / throttle reasons through NVML (read-only), sampled by ``time_ms``."""
    REASONS = {0x4: "sw_power_cap", 0x8: "hw_slowdown", 0x20: "sw_thermal_slowdown",
               0x40: "hw_thermal_slowdown", 0x80: "hw_power_brake_slowdown"}

    def __init__(self):
        self.h = None
        self.sm, self.reasons, self.max_sm = [], set(), None
        try:
            import pynvml
            pynvml.nvmlInit()
            idx = torch.cuda.current_device() if torch.cuda.is_available() else 0
            vis = os.environ.get("CUDA_VISIBLE_DEVICES")
            if vis:
                idx = int(vis.split(",")[idx])
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(idx)
            self.max_sm = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
        except Exception:
            self.h = None

    def sample(self):
        if self.h is None:
            return
        try:
            self.sm.append(self.nv.nvmlDeviceGetClockInfo(self.h, self.nv.NVML_CLOCK_SM))
            bits = self.nv.nvmlDeviceGetCurrentClocksEventReasons(self.h)
            for b, name in self.REASONS.items():
                if bits & b:
                    self.reasons.add(name)
        except Exception:
            pass

    def take(self) -> dict:
        """The record of the samples since the last call."""
        sm = sorted(self.sm)
        out = {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": self.max_sm,
               "samples": len(sm), "reasons": sorted(self.reasons)}
        self.sm, self.reasons = [], set()
        return out


_clocks = None


def clocks() -> _Clocks:
    global _clocks
    if _clocks is None:
        _clocks = _Clocks()
    return _clocks


def flush_l2():
    global _flush_buf
    if _flush_buf is None:
        _flush_buf = torch.empty(192 * 1024 * 1024, dtype=torch.uint8, device="cuda")
    _flush_buf.zero_()


def time_ms(fn, iters: int, once: bool = False) -> float:
    if once:
        fn()
        torch.cuda.synchronize()
        fn()
        torch.cuda.synchronize()
        return float("nan")
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    ts = []
    for _ in range(iters):
        flush_l2()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        clocks().sample()
        ts.append(e0.elapsed_time(e1))
    ts.sort()
    return Timed(ts[len(ts) // 2], clocks().take())


class Timed(float):
    """A median time in ms that remembers the clock record of its timed iterations."""
    def __new__(cls, ms, rec):
        obj = super().__new__(cls, ms)
        obj.clocks = rec
        return obj


def emit(**kw):
    for k, v in list(kw.items()):
        if isinstance(v, Timed):
            kw["clocks" if "clocks" not in kw else f"clocks_{k}"] = v.clocks
            kw[k] = float(v)
    print(json.dumps(kw), flush=True)


def bench_attn(args):
    from forgetrain_b200.ops import attention as A, _lib
    pk = peaks()
    shapes = {"0.5b": (2, 8, 64), "8b": (2, 16, 128), "8b-tp2": (1, 16, 128)}
    G, g, D = shapes[args.shape]
    B, S = args.batch, args.seq
    torch.manual_seed(0)
    qkv = torch.randn(B * S, G * (g + 2) * D, device="cuda").to(torch.bfloat16)
    out, lse = A.attention_fwd(qkv, B, G, g, D)
    dout = torch.randn_like(out)
    fl_fwd = 4 * B * G * g * S * S * D / 2
    t_f = time_ms(lambda: A.attention_fwd(qkv, B, G, g, D), args.iters, args.once)
    t_b = time_ms(lambda: A.attention_bwd(dout, qkv, out, lse, B, G, g, D), args.iters, args.once)
    _lib.check_status()
    for name, t, fl in (("attn_fwd", t_f, fl_fwd), ("attn_bwd", t_b, 2.5 * fl_fwd)):
        emit(kernel=name, batch=B, seq=S, q_heads=G * g, kv_heads=G, head_dim=D, ms=t,
             tflops_causal=fl / t / 1e9, frac_of_peak=fl / t / 1e9 / pk["bf16_tflops"],
             peak_kind=pk["kind"])
    if args.library:
        q = qkv.view(B, S, G, g + 2, D)
        qq = q[:, :, :, :g].reshape(B, S, G * g, D).transpose(1, 2).detach().requires_grad_()
        kk = q[:, :, :, g].transpose(1, 2).detach().requires_grad_()
        vv = q[:, :, :, g + 1].transpose(1, 2).detach().requires_grad_()
        f = lambda: torch.nn.functional.scaled_dot_product_attention(qq, kk, vv, is_causal=True,
                                                                     enable_gqa=True)
        t_lf = time_ms(lambda: f(), args.iters)
        oo = f()
        gg = torch.randn_like(oo)
        t_lb = time_ms(lambda: torch.autograd.grad(oo, (qq, kk, vv), gg, retain_graph=True), args.iters)
        emit(kernel="library_sdpa_fwd", ms=t_lf, tflops_causal=fl_fwd / t_lf / 1e9)
        emit(kernel="library_sdpa_bwd", ms=t_lb, tflops_causal=2.5 * fl_fwd / t_lb / 1e9)


GEMM_SHAPES = {
    "0.5b": {"qkv": (1280, 1024), "attn_out": (1024, 1024), "fc1": (8192, 1024), "fc2": (1024, 4096),
             "output": (73448, 1024)},
    "8b-tp2": {"qkv": (2304, 4096), "attn_out": (4096, 2048), "fc1": (16384, 4096),
               "fc2": (4096, 8192), "output": (36724 + 4, 4096)},
}


def bench_gemm(args):
    from forgetrain_b200.ops import gemm, _lib
    pk = peaks()
    T = args.tokens
    torch.manual_seed(0)
    for name, (N, K) in GEMM_SHAPES[args.shape].items():
        if args.only and name != args.only:
            continue
        x = torch.randn(T, K, device="cuda").to(torch.bfloat16)
        w = (torch.randn(N, K, device="cuda") * 0.05).to(torch.bfloat16)
        dy = torch.randn(T, N, device="cuda").to(torch.bfloat16)
        y = torch.empty(T, N, device="cuda", dtype=torch.bfloat16)
        dx = torch.empty(T, K, device="cuda", dtype=torch.bfloat16)
        dw = torch.empty(N, K, device="cuda", dtype=torch.float32)
        fl = 2.0 * T * N * K
        res = {}
        res["fwd"] = time_ms(lambda: gemm.linear_fwd(x, w, out=y), args.iters, args.once)
        res["dgrad"] = time_ms(lambda: gemm.linear_dgrad(dy, w, out=dx), args.iters, args.once)
        res["wgrad"] = time_ms(lambda: gemm.linear_wgrad(dy, x, out=dw), args.iters, args.once)
        _lib.check_status()
        lib = {}
        if args.library:
            lib["fwd"] = time_ms(lambda: torch.mm(x, w.t(), out=y), args.iters)
            lib["dgrad"] = time_ms(lambda: torch.mm(dy, w, out=dx), args.iters)
            lib["wgrad"] = time_ms(lambda: torch.mm(dy.t(), x), args.iters)
        if name == "fc1" and (N // 2) % 128 == 0:
            from forgetrain_b200.ops import cuda_ops as C
            t_two = time_ms(lambda: C.swiglu_fwd(gemm.linear_fwd(x, w, out=y)), args.iters, args.once)
            t_one = time_ms(lambda: gemm.linear_swiglu_fwd(x, w), args.iters, args.once)
            _lib.check_status()
            emit(kernel="fc1_fwd_plus_swiglu_two_kernels", M=T, N=N, K=K, ms=t_two)
            emit(kernel="fc1_fwd_swiglu_epilogue", M=T, N=N, K=K, ms=t_one, tflops=fl / t_one / 1e9)
        if name == "fc2" and K % 64 == 0:
            from forgetrain_b200.ops import cuda_ops as C
            y1 = torch.randn(T, 2 * K, device="cuda").to(torch.bfloat16)
            t_two = time_ms(lambda: C.swiglu_bwd(gemm.linear_dgrad(dy, w, out=dx), y1), args.iters, args.once)
            t_one = time_ms(lambda: gemm.linear_dgrad_swiglu_bwd(dy, w, y1), args.iters, args.once)
            _lib.check_status()
            emit(kernel="fc2_dgrad_plus_swiglu_bwd_two_kernels", M=T, N=K, K=N, ms=t_two)
            emit(kernel="fc2_dgrad_swiglu_bwd_epilogue", M=T, N=K, K=N, ms=t_one, tflops=fl / t_one / 1e9)
            del y1
        for k, t in res.items():
            emit(kernel=f"gemm_{name}_{k}", M=T, N=N, K=K, ms=t, tflops=fl / t / 1e9,
                 frac_of_peak=fl / t / 1e9 / pk["bf16_tflops"], peak_kind=pk["kind"],
                 library_tflops=(fl / lib[k] / 1e9 if k in lib else None))


def sweep_gemm(args):
    """Tile / split sweep per projection shape (the role of the reference's persistent-config
    sweep, exports/train_engine_0.5B/tests/sweep_v3_persistent.py): every forward / dgrad GEMM
    with both tile widths and, for the weight gradients, every split-K factor the kernel accepts;
    one line per candidate and one ``best`` line per GEMM, against the default rule's choice."""
    from forgetrain_b200.ops import gemm, _lib
    T = args.tokens
    torch.manual_seed(0)
    for name, (N, K) in GEMM_SHAPES[args.shape].items():
        if args.only and name != args.only:
            continue
        x = torch.randn(T, K, device="cuda").to(torch.bfloat16)
        w = (torch.randn(N, K, device="cuda") * 0.05).to(torch.bfloat16)
        dy = torch.randn(T, N, device="cuda").to(torch.bfloat16)
        y = torch.empty(T, N, device="cuda", dtype=torch.bfloat16)
        dx = torch.empty(T, K, device="cuda", dtype=torch.bfloat16)
        dw = torch.empty(N, K, device="cuda", dtype=torch.float32)
        fl = 2.0 * T * N * K
        cands = {
            "fwd": [({"bn": bn}, (lambda bn=bn: gemm.linear_fwd(x, w, out=y, bn=bn))) for bn in (128, 256)],
            "dgrad": [({"bn": bn}, (lambda bn=bn: gemm.linear_dgrad(dy, w, out=dx, bn=bn))) for bn in (128, 256)],
            "wgrad": [({"bn": bn, "splitk": sk},
                       (lambda bn=bn, sk=sk: gemm.linear_wgrad(dy, x, out=dw, bn=bn, splitk=sk)))
                      for bn in (128, 256) for sk in (1, 2, 4, 8, 16)],
        }
        defaults = {"fwd": lambda: gemm.linear_fwd(x, w, out=y),
                    "dgrad": lambda: gemm.linear_dgrad(dy, w, out=dx),
                    "wgrad": lambda: gemm.linear_wgrad(dy, x, out=dw)}
        for kind, lst in cands.items():
            t_def = time_ms(defaults[kind], args.iters, args.once)
            best = None
            for cfg, fn in lst:
                t = time_ms(fn, args.iters, args.once)
                _lib.check_status()
                emit(kernel=f"sweep_{name}_{kind}", M=T, N=N, K=K, ms=t, tflops=fl / t / 1e9, **cfg)
                if best is None or t < best[0]:
                    best = (t, cfg)
            emit(kernel=f"best_{name}_{kind}", M=T, N=N, K=K, ms=best[0], tflops=fl / best[0] / 1e9,
                 default_rule_ms=t_def, default_rule_tflops=fl / t_def / 1e9, **best[1])


def bench_elem(args):
    from forgetrain_b200.ops import cuda_ops as C, reference as R, _lib
    pk = peaks()
    T, H, F, V = args.tokens, 1024, 4096, 73448
    x = torch.randn(T, H, device="cuda").to(torch.bfloat16)
    res = torch.randn(T, H, device="cuda").to(torch.bfloat16)
    w = torch.ones(H, device="cuda", dtype=torch.bfloat16)
    h, y, rs = C.add_rmsnorm_fwd(res, x, w, 1e-6)
    dw = torch.zeros(H, device="cuda")
    y1 = torch.randn(T, 2 * F, device="cuda").to(torch.bfloat16)
    da = torch.randn(T, F, device="cuda").to(torch.bfloat16)
    lg = torch.randn(T, V, device="cuda").to(torch.bfloat16)
    lab = torch.randint(0, V, (T,), device="cuda")
    qkv = torch.randn(T, 1280, device="cuda").to(torch.bfloat16)
    cos, sin = R.rope_tables(4096, 64, 10000.0, device="cuda")
    ids = torch.randint(0, V, (T,), device="cuda")
    gw = torch.zeros(V, H, device="cuda")
    n = 64 * 1024 * 1024
    p32 = torch.randn(n, device="cuda"); m = torch.zeros(n, device="cuda"); v = torch.zeros(n, device="cuda")
    g = torch.randn(n, device="cuda"); pb = torch.empty(n, device="cuda", dtype=torch.bfloat16)
    hyper = torch.tensor([1e-3, 0.9, 0.95, 1e-8, 0.1, 0.05, 1.0, 0], device="cuda")
    se = torch.tensor([n], device="cuda", dtype=torch.int64); sw = torch.tensor([0.1], device="cuda")
    sl = torch.tensor([1.0], device="cuda")
    cases = [
        ("add_rmsnorm_fwd", lambda: C.add_rmsnorm_fwd(res, x, w, 1e-6), 4 * T * H * 2),
        ("rmsnorm_bwd", lambda: C.rmsnorm_bwd(x, h, w, rs, res, dw, False), 4 * T * H * 2),
        ("swiglu_fwd", lambda: C.swiglu_fwd(y1), 3 * T * F * 2),
        ("swiglu_bwd", lambda: C.swiglu_bwd(da, y1), 5 * T * F * 2),
        ("cross_entropy_fwd_bwd", lambda: C.cross_entropy_fwd_bwd(lg, lab, None, 1.0), 2 * T * V * 2),
        ("rope", lambda: C.rope_(qkv, cos, sin, T // 4096, 2, 8, 64), 2 * T * 1152 * 2),
        ("adamw", lambda: C.adamw_flat(p32, m, v, g, pb, hyper, se, sw, sl), n * (4 * 7 + 2)),
        ("embedding_bwd", lambda: C.embedding_bwd(ids, x, 12.0, gw), T * H * (2 + 4 + 4)),
    ]
    for name, fn, nbytes in cases:
        if args.only and name != args.only:
            continue
        t = time_ms(fn, args.iters, args.once)
        emit(kernel=name, tokens=T, ms=t, gbs=nbytes / t / 1e6, frac_of_peak=nbytes / t / 1e6 / pk["hbm_gbs"],
             peak_kind=pk["kind"])
    _lib.check_status()


def bench_comm(args):
    from forgetrain_b200.parallel import commbench
    commbench.main(args)


def bench_tp(args):
    from forgetrain_b200.parallel import commbench
    commbench.tp_main(args)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("what", choices=["attn", "gemm", "elem", "comm", "tp"])
    ap.add_argument("--batch", type=int, default=4)
    ap.add_argument("--seq", type=int, default=4096)
    ap.add_argument("--tokens", type=int, default=16384)
    ap.add_argument("--shape", default="0.5b")
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--only", default=None)
    ap.add_argument("--once", action="store_true")
    ap.add_argument("--library", action="store_true", help="also time the library kernel (cuBLAS / SDPA)")
    ap.add_argument("--sweep", action="store_true", help="gemm: sweep tile width and split-K per shape")
    ap.add_argument("--min-mb", type=float, default=1.0)
    ap.add_argument("--max-mb", type=float, default=1024.0)
    args = ap.parse_args()
    if args.what == "gemm" and args.sweep:
        return sweep_gemm(args)
    {"attn": bench_attn, "gemm": bench_gemm, "elem": bench_elem, "comm": bench_comm,
     "tp": bench_tp}[args.what](args)


if __name__ == "__main__":
    main()
