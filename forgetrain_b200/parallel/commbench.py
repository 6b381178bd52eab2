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
