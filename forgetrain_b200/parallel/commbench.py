"""Bucket reduce-scatter / all-gather sweep: fused peer-memory kernels vs the NCCL calls they
replace. Run under torchrun with N >= 2 ranks through ``python microbench.py comm``.

Times are device times (CUDA events), max over ranks. ``bus_gbs`` follows the usual convention
for reduce-scatter / all-gather: bytes of the full buffer x (W-1)/W / time. The roofline
denominator is the measured per-direction NVLink copy rate (770 GB/s on this pool)."""
from __future__ import annotations

import json
import os

import torch
import torch.distributed as dist

LINK_GBS = 770.0


def _time(fn, iters, group):
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    dist.barrier(group=group)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    t = torch.tensor([e0.elapsed_time(e1) / iters], device="cuda", dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t)


def main(args) -> None:
    from ..ops import _lib
    from .buckets import Bucket
    from .fused_dp import FusedDPComm, SymmetricBuffers
    from .topology import init_topology
    topo = init_topology(1)
    W, r = topo.world, topo.rank
    assert W >= 2, "run under torchrun with at least 2 ranks"
    max_elems = int(args.max_mb * 1e6 / 4) // (W * 128) * (W * 128)
    symm = SymmetricBuffers(max_elems, topo.device, topo.dp_group, r, W)
    comm = FusedDPComm(symm)
    sumsq = torch.zeros(1, device="cuda")
    nccl_in = torch.empty(max_elems, device="cuda", dtype=torch.float32)
    mb = args.min_mb
    while mb <= args.max_mb * 1.0001:
        n = int(mb * 1e6 / 4) // (W * 128) * (W * 128)
        b = Bucket(0, 0, n)
        symm.grads[:n].normal_()
        iters = 20 if mb <= 64 else 8
        t_f = _time(lambda: comm.reduce_scatter_bucket(b, sumsq), iters, topo.dp_group)

        def nccl_rs():
            v = nccl_in[:n]
            v.mul_(1.0 / W)
            dist.reduce_scatter_tensor(v[r * (n // W):(r + 1) * (n // W)], v, group=topo.dp_group)
            sumsq.add_(v[r * (n // W):(r + 1) * (n // W)].pow(2).sum())
        t_n = _time(nccl_rs, iters, topo.dp_group)
        t_ag = _time(lambda: comm.all_gather_bucket(b), iters, topo.dp_group)
        pv = symm.params[:n]
        t_nag = _time(lambda: dist.all_gather_into_tensor(pv, pv[r * (n // W):(r + 1) * (n // W)],
                                                          group=topo.dp_group), iters, topo.dp_group)
        if r == 0:
            rs_bytes = n * 4 * (W - 1) / W
            ag_bytes = n * 2 * (W - 1) / W
            print(json.dumps({
                "op": "bucket_reduce_scatter_fp32", "world": W, "mbytes": n * 4 / 1e6,
                "fused_ms": t_f, "nccl_ms": t_n, "fused_bus_gbs": rs_bytes / t_f / 1e6,
                "nccl_bus_gbs": rs_bytes / t_n / 1e6,
                "fused_roofline_frac": rs_bytes / t_f / 1e6 / LINK_GBS,
                "multimem": bool(symm.mc_grads)}), flush=True)
            print(json.dumps({
                "op": "bucket_all_gather_bf16", "world": W, "mbytes": n * 2 / 1e6,
                "fused_ms": t_ag, "nccl_ms": t_nag, "fused_bus_gbs": ag_bytes / t_ag / 1e6,
                "nccl_bus_gbs": ag_bytes / t_nag / 1e6,
                "fused_roofline_frac": ag_bytes / t_ag / 1e6 / LINK_GBS}), flush=True)
        mb *= 4
    torch.cuda.synchronize()
    _lib.check_status()
    dist.barrier()


def tp_main(args) -> None:
    """Fused all-gather->GEMM / GEMM->reduce-scatter vs NCCL collective + the same GEMM, at the
    8B tensor-parallel shapes (hidden 4096, ffn 16384, 32 q / 2 kv heads of 128)."""
    from ..ops import _lib
    from .fused_tp import FusedTPContext
    from .topology import init_topology
    from .tp import TPContext
    W = int(os.environ.get("WORLD_SIZE", "1"))
    topo = init_topology(W)
    tp, r = topo.tp_size, topo.tp_rank
    assert tp >= 2, "run under torchrun with at least 2 ranks"
    T, H, F = args.tokens, 4096, 16384
    ctx = FusedTPContext(topo.tp_group, tp, r, topo.device, T, H, 8)
    base = TPContext(topo.tp_group, tp, r, True)
    torch.manual_seed(1234)
    qkv_n = (32 // tp + 2 * max(1, 2 // tp)) * 128
    peak = 1652.5
    cases = [("ag_gemm_qkv", "ag", qkv_n, H), ("ag_gemm_fc1", "ag", 2 * F // tp, H),
             ("gemm_rs_attn_out", "rs", H, 32 * 128 // tp), ("gemm_rs_fc2", "rs", H, F // tp)]
    for name, kind, N, K in cases:
        w = (torch.randn(N, K, device="cuda") * 0.05).to(torch.bfloat16)
        g = torch.Generator(device="cuda").manual_seed(10 + r)
        if kind == "ag":
            x = torch.randn(T // tp, K, device="cuda", generator=g).to(torch.bfloat16)
            f_fused = lambda: ctx.linear_gather(x, w, 1.0, key=name)
            f_base = lambda: base.linear_gather(x, w, 1.0)
            link_bytes = (tp - 1) / tp * T * K * 2
        else:
            x = torch.randn(T, K, device="cuda", generator=g).to(torch.bfloat16)
            f_fused = lambda: ctx.linear_scatter(x, w, 1.0)
            f_base = lambda: base.linear_scatter(x, w, 1.0)
            link_bytes = (tp - 1) / tp * T * N * 2
        a, b = f_fused(), f_base()
        a = a[0] if isinstance(a, tuple) else a
        b = b[0] if isinstance(b, tuple) else b
        err = float((a.float() - b.float()).abs().max() / (b.float().abs().max() + 1e-9))
        t_f = _time(f_fused, 20, topo.tp_group)
        t_b = _time(f_base, 20, topo.tp_group)
        flops = 2.0 * T * N * K
        roof_ms = max(flops / (peak * 1e12), link_bytes / (LINK_GBS * 1e9)) * 1e3
        if r == 0:
            print(json.dumps({"op": name, "tp": tp, "M": T, "N": N, "K": K, "fused_ms": t_f,
                              "nccl_plus_gemm_ms": t_b, "fused_tflops": flops / t_f / 1e9,
                              "roofline_ms": roof_ms, "fused_roofline_frac": roof_ms / t_f,
                              "max_rel_diff_vs_nccl_path": err}), flush=True)
    torch.cuda.synchronize()
    _lib.check_status()
    dist.barrier()
