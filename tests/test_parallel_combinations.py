"""Feature combinations against one process: every case trains three steps on CPU ranks (gloo) and
must follow, to fp32 rounding, the single-process run that sees the same micro-batches in one
gradient-accumulation loop. The cases pair switches that meet in the same code (gradient
accumulation with tensor-parallel gradient collectives, tied tables with vocabulary parallelism,
recomputation with document positions, the MTP head with sharded and unsharded optimizers). Tensor
parallelism above the KV groups with gradient accumulation is in ``test_dist_gloo.py``."""
import os
import sys

import pytest
import torch

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
from dist_util import run_ranks  # noqa: E402


def _spec(**kw):
    from forgetrain_b200.config import load_model_spec
    base = dict(num_layers=2, vocab_size=512, hidden_size=128, ffn_hidden_size=256,
                num_attention_heads=8, num_query_groups=2, head_dim=32, seq_length=64,
                max_position_embeddings=64, tie_embeddings=False)
    base.update(kw)
    return load_model_spec("tiny", **base)


def _batch(i, positions):
    g = torch.Generator().manual_seed(100 + i)
    c = torch.randint(0, 512, (2, 65), generator=g)
    b = {"tokens": c[:, :-1].contiguous(), "labels": c[:, 1:].contiguous(), "loss_mask": torch.ones(2, 64)}
    b["loss_mask"][:, :5] = 0                       # a masked prefix, as after a prompt
    if positions:                                   # two documents per row
        p = torch.arange(64, dtype=torch.int32).repeat(2, 1)
        p[:, 30:] -= 30
        b["position_ids"] = p
    return b


def _worker(rank, world, tp, n_micro_batches, spec_kw, cfg_kw, positions):
    from forgetrain_b200.engine_config import from_spec
    from forgetrain_b200.parallel.topology import init_topology
    from forgetrain_b200.trainer import Trainer
    spec = _spec(**spec_kw)
    topo = init_topology(tp, device="cpu", num_kv_groups=spec.num_query_groups)
    kw = dict(dtype="fp32", comm="nccl", max_lr=1e-3, warmup_iters=0, tensor_parallel_size=tp,
              wgrad_bucket_target_elems=60_000, rs_buckets=0)
    kw.update(cfg_kw)
    tr = Trainer(spec, from_spec(spec, **kw), topo, seq_length=64, micro_batch_size=2, seed=0)
    per = n_micro_batches // topo.dp_size
    mine = [_batch(topo.dp_rank * per + k, positions) for k in range(per)]
    out = []
    for _ in range(3):
        o = tr.train_step(mine)
        out.append((float(o["loss"]), float(o["grad_norm"])))
    return out


CASES = {
    # name: (ranks, tp, micro-batches of the whole job, spec overrides, config of the ranks, config of the one process, positions)
    "tied tables, TP=2 x DP=2, two micro-batches per rank, replicated residual stream":
        (4, 2, 4, dict(tie_embeddings=True), dict(sequence_parallel=False), {}, False),
    "recomputation with document positions, TP=2 sequence parallel, two micro-batches":
        (2, 2, 2, {}, dict(sequence_parallel=True, recompute_attn=True, recompute_mlp=True), {}, True),
    "two MTP layers with recomputation, DP=2":
        (2, 1, 2, {}, dict(mtp_num_layers=2, recompute_attn=True, recompute_mlp=True), dict(mtp_num_layers=2), False),
    "MTP head with an unsharded optimizer and layer-aligned buckets, DP=2, two micro-batches per rank":
        (2, 1, 4, {}, dict(mtp_num_layers=1, sharded_optimizer=False, rs_buckets=3), dict(mtp_num_layers=1), False),
}


@pytest.mark.parametrize("name", list(CASES))
def test_combination_follows_the_single_process_run(name):
    ranks, tp, n_mb, spec_kw, cfg_kw, ref_kw, positions = CASES[name]
    want = run_ranks(_worker, 1, 1, n_mb, spec_kw, ref_kw, positions)[0]
    got = run_ranks(_worker, ranks, tp, n_mb, spec_kw, cfg_kw, positions)
    for rank in range(ranks):
        for (loss, norm), (wl, wn) in zip(got[rank], want):
            assert loss == pytest.approx(wl, abs=5e-6) and norm == pytest.approx(wn, rel=5e-6), (rank, got[rank], want)
    assert want[-1][0] < want[0][0]                 # and the run does train
