"""Candidate kernels under neighbour load on the same GPU (the reference's stress harness,
exports/train_engine_8b/tests/_stress_runner.py, in small): while background threads keep the
device busy with library GEMMs, device-to-device copies, allocator churn and stream/event
traffic, the candidate op loops on its own stream. PASS = no exception, no NaN/Inf, the result
still matches the oracle afterwards, no iteration slower than the hang limit, every worker
alive. A watchdog ends the process past the deadline."""
import os
import threading
import time

import pytest
import torch

pytestmark = pytest.mark.gpu


def _workers(stop):
    def blast():
        a = torch.randn(2048, 2048, device="cuda", dtype=torch.bfloat16)
        s = torch.cuda.Stream()
        with torch.cuda.stream(s):
            while not stop.is_set():
                (a @ a).sum()
                s.synchronize()

    def d2d():
        a = torch.empty(64 << 20, device="cuda", dtype=torch.uint8)
        b = torch.empty_like(a)
        s = torch.cuda.Stream()
        with torch.cuda.stream(s):
            while not stop.is_set():
                b.copy_(a, non_blocking=True)
                s.synchronize()

    def churn():
        while not stop.is_set():
            xs = [torch.empty(1 << 20, device="cuda") for _ in range(8)]
            del xs
            time.sleep(0.001)

    def events():
        s1, s2 = torch.cuda.Stream(), torch.cuda.Stream()
        x = torch.ones(1 << 16, device="cuda")
        while not stop.is_set():
            with torch.cuda.stream(s1):
                x.add_(1)
                e = torch.cuda.Event()
                e.record()
            s2.wait_event(e)
            with torch.cuda.stream(s2):
                x.mul_(1.0)
            s2.synchronize()
    return [threading.Thread(target=f, daemon=True) for f in (blast, d2d, churn, events)]


def _stress(candidate, oracle_check, seconds=4.0, hang_s=5.0):
    from forgetrain_b200.ops import _lib
    deadline = threading.Timer(90.0, lambda: os._exit(2))
    deadline.daemon = True
    deadline.start()
    stop = threading.Event()
    ws = _workers(stop)
    for w in ws:
        w.start()
    stream = torch.cuda.Stream()
    n, worst = 0, 0.0
    t_end = time.time() + seconds
    try:
        with torch.cuda.stream(stream):
            while time.time() < t_end:
                t0 = time.time()
                out = candidate()
                stream.synchronize()
                worst = max(worst, time.time() - t0)
                n += 1
                if n % 50 == 0:
                    assert torch.isfinite(out.float()).all()
            assert all(w.is_alive() for w in ws), "a neighbour worker died"
            out = candidate()
            stream.synchronize()
    finally:
        stop.set()
        for w in ws:
            w.join(timeout=10)
        deadline.cancel()
    _lib.check_status()
    assert worst < hang_s, f"slowest iteration took {worst:.2f}s"
    oracle_check(out)
    return n


def test_gemm_under_neighbour_load():
    from forgetrain_b200.ops import gemm
    torch.manual_seed(0)
    x = torch.randn(4096, 1024, device="cuda").to(torch.bfloat16)
    w = (torch.randn(4096, 1024, device="cuda") * 0.05).to(torch.bfloat16)
    ref = x.float() @ w.float().t()

    def check(out):
        assert torch.allclose(out.float(), ref, rtol=0.05, atol=0.5)
    assert _stress(lambda: gemm.linear_fwd(x, w), check) > 10


def test_attention_under_neighbour_load():
    from forgetrain_b200.ops import attention as A, reference as R
    torch.manual_seed(0)
    qkv = torch.randn(2 * 1024, 2 * 6 * 64, device="cuda").to(torch.bfloat16)
    ref, _ = R.attention_fwd(qkv, 2, 2, 4, 64)

    def check(out):
        assert torch.allclose(out.float(), ref.float(), rtol=0.05, atol=0.05)
    assert _stress(lambda: A.attention_fwd(qkv, 2, 2, 4, 64)[0], check) > 10
