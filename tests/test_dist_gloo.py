"""Multi-process CPU (gloo) runs: data parallel, tensor parallel, checkpoint round-trip."""
import os
import sys

import pytest
import torch

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
from dist_util import run_ranks  # noqa: E402


def _spec(**kw):
    from forgetrain_b200.config import load_model_spec
    base = dict(num_layers=2, vocab_size=512, hidden_size=128, ffn_hidden_size=256,
                num_attention_heads=4, num_query_groups=2, head_dim=32, seq_length=64,
                max_position_embeddings=64, tie_embeddings=True)
    base.update(kw)
    return load_model_spec("tiny", **base)


def _cfg(spec, **kw):
    from forgetrain_b200.engine_config import from_spec
    base = dict(dtype="fp32", comm="nccl", wgrad_bucket_target_elems=60_000, max_lr=1e-3,
                warmup_iters=0, rs_buckets=0)
    base.update(kw)
    return from_spec(spec, **base)


def _batches(seed, n, mbs, seq, vocab):
    g = torch.Generator().manual_seed(seed)
    out = []
    for _ in range(n):
        c = torch.randint(0, vocab, (mbs, seq + 1), generator=g)
        out.append({"tokens": c[:, :-1].contiguous(), "labels": c[:, 1:].contiguous(),
                    "loss_mask": torch.ones(mbs, seq)})
    return out


# ------------------------------------------------------------------------------------------
def _dp_worker(rank, world, steps):
    from forgetrain_b200.parallel.topology import init_topology
    from forgetrain_b200.trainer import Trainer
    spec = _spec()
    topo = init_topology(1, device="cpu")
    tr = Trainer(spec, _cfg(spec), topo, seq_length=64, micro_batch_size=2, seed=0)
    data = _batches(100 + rank, 1, 2, 64, spec.vocab_size)      # one fixed batch per rank
    losses = []
    for _ in range(steps):
        out = tr.train_step(data)
        losses.append(float(out["loss"]))
    return losses, tr.store.named_cpu_params(), float(out["grad_norm"])


def _single_worker_equivalent(steps):
    from forgetrain_b200.parallel.topology import Topology
    from forgetrain_b200.trainer import Trainer
    spec = _spec()
    tr = Trainer(spec, _cfg(spec), Topology(), seq_length=64, micro_batch_size=2, seed=0)
    data = _batches(100, 1, 2, 64, spec.vocab_size) + _batches(101, 1, 2, 64, spec.vocab_size)
    losses = []
    for _ in range(steps):
        out = tr.train_step(data)           # two micro-batches == two DP ranks
        losses.append(float(out["loss"]))
    return losses, tr.store.named_cpu_params(), float(out["grad_norm"])


def test_dp2_matches_gradient_accumulation_and_loss_decreases():
    res = run_ranks(_dp_worker, 2, 5)
    (l0, p0, n0), (l1, p1, n1) = res
    assert l0 == l1 and n0 == n1 and all(torch.equal(p0[k], p1[k]) for k in p0)   # replicas identical
    assert l0[-1] < l0[0]
    ls, ps, ns = _single_worker_equivalent(5)
    assert max(abs(a - b) for a, b in zip(l0, ls)) < 1e-4
    assert all(torch.allclose(p0[k], ps[k], atol=2e-5) for k in ps)
    assert abs(n0 - ns) < 1e-4


# ------------------------------------------------------------------------------------------
def _tp_worker(rank, world, sp, steps, tp=2, heads=4, micro_batches=1):
    from forgetrain_b200.parallel.topology import init_topology
    from forgetrain_b200.trainer import Trainer
    spec = _spec(tie_embeddings=False, num_attention_heads=heads)
    topo = init_topology(tp, device="cpu", num_kv_groups=spec.num_query_groups)
    tr = Trainer(spec, _cfg(spec, tensor_parallel_size=tp, sequence_parallel=sp), topo, seq_length=64,
                 micro_batch_size=2, seed=0)
    data = _batches(7, micro_batches, 2, 64, spec.vocab_size)
    losses, norms = [], []
    for _ in range(steps):
        out = tr.train_step(data)
        losses.append(float(out["loss"]))
        norms.append(float(out["grad_norm"]))
    return losses, norms


@pytest.mark.parametrize("sp", [True, False])
def test_tp2_matches_tp1(sp):
    from forgetrain_b200.parallel.topology import Topology
    from forgetrain_b200.trainer import Trainer
    res = run_ranks(_tp_worker, 2, sp, 3)
    assert res[0][0] == pytest.approx(res[1][0], abs=1e-6)
    spec = _spec(tie_embeddings=False)
    tr = Trainer(spec, _cfg(spec), Topology(), seq_length=64, micro_batch_size=2, seed=0)
    data = _batches(7, 1, 2, 64, spec.vocab_size)
    for i in range(3):
        out = tr.train_step(data)
        assert float(out["loss"]) == pytest.approx(res[0][0][i], abs=2e-4)
        assert float(out["grad_norm"]) == pytest.approx(res[0][1][i], rel=2e-3)


# ------------------------------------------------------------------------------------------
def _ckpt_worker(rank, world, root):
    from forgetrain_b200.parallel.topology import init_topology
    from forgetrain_b200.trainer import run_training_loop
    spec = _spec()
    topo = init_topology(1, device="cpu")
    cfg = _cfg(spec)
    a = run_training_loop(spec=spec, cfg=cfg, topo=topo, num_steps=4, micro_batch_size=1, seq_length=64,
                          seed=3, save_dir=os.path.join(root, "full"), save_interval=2)
    losses_full = [s["loss"] for s in a["steps"]]
    b = run_training_loop(spec=spec, cfg=cfg, topo=topo, num_steps=2, micro_batch_size=1, seq_length=64,
                          seed=3, resume=os.path.join(root, "full", "step_0000002"))
    losses_resumed = [s["loss"] for s in b["steps"]]
    return losses_full, losses_resumed


def test_dp2_checkpoint_resume_continues_the_run(tmp_path):
    res = run_ranks(_ckpt_worker, 2, str(tmp_path))
    full, resumed = res[0]
    assert (tmp_path / "full" / "step_0000002" / "training_state.pt").exists()
    assert resumed == pytest.approx(full[2:], abs=1e-5)


def test_tp4_with_replicated_kv_heads_and_gradient_accumulation_matches_tp1():
    """The sum of the k / v gradients over the replicas of a KV group is taken once, when the
    gradient is complete: summing the buffer after every micro-batch would count the earlier
    micro-batches once per replica (the first loss after an update would still agree, the
    gradient norm and everything after it would not)."""
    from forgetrain_b200.parallel.topology import Topology
    from forgetrain_b200.trainer import Trainer
    res = run_ranks(_tp_worker, 4, True, 3, 4, 8, 3)
    spec = _spec(tie_embeddings=False, num_attention_heads=8)
    tr = Trainer(spec, _cfg(spec), Topology(), seq_length=64, micro_batch_size=2, seed=0)
    data = _batches(7, 3, 2, 64, spec.vocab_size)
    for i in range(3):
        out = tr.train_step(data)
        assert float(out["loss"]) == pytest.approx(res[0][0][i], abs=5e-6)
        assert float(out["grad_norm"]) == pytest.approx(res[0][1][i], rel=5e-6)


# ------------------------------------------------------------------------------------------
def _tp_dp_worker(rank, world, steps):
    """World 4 = TP 2 x DP 2 (consecutive ranks form a TP group): the 8B topology in miniature."""
    from forgetrain_b200.parallel.topology import init_topology
    from forgetrain_b200.trainer import Trainer
    spec = _spec(tie_embeddings=False)
    topo = init_topology(2, device="cpu", num_kv_groups=spec.num_query_groups)
    assert (topo.tp_size, topo.dp_size) == (2, 2) and topo.dp_rank == rank // 2
    tr = Trainer(spec, _cfg(spec, tensor_parallel_size=2, sequence_parallel=True), topo,
                 seq_length=64, micro_batch_size=2, seed=0)
    data = _batches(100 + topo.dp_rank, 1, 2, 64, spec.vocab_size)   # one batch per DP replica
    losses, norms = [], []
    for _ in range(steps):
        out = tr.train_step(data)
        losses.append(float(out["loss"]))
        norms.append(float(out["grad_norm"]))
    return losses, norms


def test_tp2_x_dp2_matches_one_process_with_two_microbatches():
    from forgetrain_b200.parallel.topology import Topology
    from forgetrain_b200.trainer import Trainer
    res = run_ranks(_tp_dp_worker, 4, 3)
    for r in range(1, 4):                      # the loss is the global mean on every rank
        assert res[r][0] == pytest.approx(res[0][0], abs=1e-6)
        assert res[r][1] == pytest.approx(res[0][1], rel=1e-6)
    spec = _spec(tie_embeddings=False)
    tr = Trainer(spec, _cfg(spec), Topology(), seq_length=64, micro_batch_size=2, seed=0)
    data = _batches(100, 1, 2, 64, spec.vocab_size) + _batches(101, 1, 2, 64, spec.vocab_size)
    for i in range(3):
        out = tr.train_step(data)
        assert float(out["loss"]) == pytest.approx(res[0][0][i], abs=3e-4)
        # TP-duplicated norm gradients are counted once, sharded ones on every TP rank
        assert float(out["grad_norm"]) == pytest.approx(res[0][1][i], rel=2e-3)


def _tp_ckpt_worker(rank, world, root):
    from forgetrain_b200.parallel.topology import init_topology
    from forgetrain_b200.trainer import run_training_loop
    spec = _spec(tie_embeddings=False)
    topo = init_topology(2, device="cpu", num_kv_groups=spec.num_query_groups)
    cfg = _cfg(spec, tensor_parallel_size=2, sequence_parallel=True)
    a = run_training_loop(spec=spec, cfg=cfg, topo=topo, num_steps=4, micro_batch_size=1, seq_length=64,
                          seed=3, save_dir=os.path.join(root, "full"), save_interval=2)
    b = run_training_loop(spec=spec, cfg=cfg, topo=topo, num_steps=2, micro_batch_size=1, seq_length=64,
                          seed=3, resume=os.path.join(root, "full", "step_0000002"))
    return [s["loss"] for s in a["steps"]], [s["loss"] for s in b["steps"]]


def test_tp2_x_dp2_per_rank_shards_resume(tmp_path):
    """With tensor parallelism every TP rank of the first DP replica writes ``rank_<R>.pt`` (its
    parameter shard plus the DP-gathered optimizer state of that shard); a resumed run continues
    the loss curve (reference: 8B parameters.py:375-449)."""
    res = run_ranks(_tp_ckpt_worker, 4, str(tmp_path))
    d = tmp_path / "full" / "step_0000002"
    assert sorted(p.name for p in d.iterdir()) == ["rank_0.pt", "rank_1.pt"]
    st = torch.load(d / "rank_1.pt", map_location="cpu", weights_only=False)
    assert st["tp_size"] == 2 and st["tp_rank"] == 1 and st["format_version"] == 1
    # column-parallel weights hold half of the rows, row-parallel ones half of the columns
    assert st["params"]["layers.0.feed_forward.wfc1.weight"].shape == (256, 128)
    assert st["params"]["layers.0.feed_forward.w2.weight"].shape == (128, 128)
    full, resumed = res[0]
    assert resumed == pytest.approx(full[2:], abs=1e-5)
    for r in range(1, 4):
        assert res[r][1] == pytest.approx(resumed, abs=1e-6)


def _reshard_worker(rank, world, root, phase):
    """phase 'save': TP2 run that saves at step 2 of 4. phase 'resume': TP2 run resumed from the
    checkpoint that a single process (TP1) wrote."""
    from forgetrain_b200.parallel.topology import init_topology
    from forgetrain_b200.trainer import run_training_loop
    spec = _spec(tie_embeddings=False)
    topo = init_topology(2, device="cpu", num_kv_groups=spec.num_query_groups)
    cfg = _cfg(spec, tensor_parallel_size=2, sequence_parallel=True)
    if phase == "save":
        a = run_training_loop(spec=spec, cfg=cfg, topo=topo, num_steps=4, micro_batch_size=1,
                              seq_length=64, seed=3, save_dir=os.path.join(root, "tp2"), save_interval=2)
    else:
        a = run_training_loop(spec=spec, cfg=cfg, topo=topo, num_steps=2, micro_batch_size=1,
                              seq_length=64, seed=3, resume=os.path.join(root, "tp1", "step_0000002"))
    return [s["loss"] for s in a["steps"]]


def test_checkpoints_move_between_tensor_parallel_degrees(tmp_path):
    """A TP2 checkpoint resumes in one process and a one-process checkpoint resumes at TP2: shards
    (parameters and Adam state) are merged to full tensors and cut again for the new degree."""
    from forgetrain_b200.parallel.topology import Topology
    from forgetrain_b200.trainer import run_training_loop
    tp2 = run_ranks(_reshard_worker, 2, str(tmp_path), "save")[0]
    spec = _spec(tie_embeddings=False)
    one = run_training_loop(spec=spec, cfg=_cfg(spec), topo=Topology(), num_steps=2, micro_batch_size=1,
                            seq_length=64, seed=3, resume=str(tmp_path / "tp2" / "step_0000002"))
    assert [s["loss"] for s in one["steps"]] == pytest.approx(tp2[2:], abs=3e-4)
    full = run_training_loop(spec=spec, cfg=_cfg(spec), topo=Topology(), num_steps=4, micro_batch_size=1,
                             seq_length=64, seed=3, save_dir=str(tmp_path / "tp1"), save_interval=2)
    back = run_ranks(_reshard_worker, 2, str(tmp_path), "resume")[0]
    assert back == pytest.approx([s["loss"] for s in full["steps"]][2:], abs=3e-4)


def _megatron_tp_worker(rank, world, root):
    from forgetrain_b200.parallel.topology import init_topology
    from forgetrain_b200.trainer import Trainer
    spec = _spec(tie_embeddings=False)
    topo = init_topology(2, device="cpu", num_kv_groups=spec.num_query_groups)
    tr = Trainer(spec, _cfg(spec, tensor_parallel_size=2, sequence_parallel=True), topo,
                 seq_length=64, micro_batch_size=1, seed=0)
    tr.load(root)
    st = tr.opt.gather_full_state()
    name = "layers.1.feed_forward.wfc1.weight"
    out = tr.train_step(_batches(5, 1, 1, 64, spec.vocab_size))
    return (tr.opt.step_count, tuple(st["exp_avg"][name].shape), st["exp_avg"][name].clone(),
            st["master_weights"][name].clone(), tr.store.params[name].shape, float(out["loss"]))


def test_megatron_export_with_adam_state_loads_at_tp2(tmp_path):
    """Every TP rank reads the full Megatron tensors and keeps its shard of the parameters AND of
    the Adam moments / master weights."""
    from forgetrain_b200.ckpt import megatron_import as mg
    from forgetrain_b200.models.params import all_param_specs, shard_for_tp
    spec = _spec(tie_embeddings=False)
    g = torch.Generator().manual_seed(1)
    ours = {ps.name: torch.randn(ps.shape, generator=g) * 0.02 for ps in all_param_specs(spec)}
    inv = {k: v for k, v in mg.megatron_name_map(spec.num_layers, 0).items()
           if not (k.startswith("decoder.layers") and (k.endswith("input_layernorm.weight")
                                                       or k.endswith("pre_mlp_layernorm.weight")))}
    ck = {k: ours[v].clone() for k, v in inv.items() if v in ours}
    mom = {k: torch.randn(v.shape, generator=g) * 1e-3 for k, v in ck.items()}
    torch.save(ck, tmp_path / mg.PARAMS_FILE)
    torch.save({"master_weights": ck, "exp_avg": mom, "exp_avg_sq": {k: v * v for k, v in mom.items()},
                "step_count": 9, "num_samples": 18}, tmp_path / mg.OPTIM_FILE)
    res = run_ranks(_megatron_tp_worker, 2, str(tmp_path))
    name = "layers.1.feed_forward.wfc1.weight"
    ps = next(p for p in all_param_specs(spec) if p.name == name)
    mkey = next(k for k, v in inv.items() if v == name)
    for r in range(2):
        steps, shape, m, master, pshape, loss = res[r]
        assert steps == 10 and shape == (256, 128) == tuple(pshape)
        assert torch.allclose(m, shard_for_tp(ps, mom[mkey], spec, r, 2))
        assert torch.allclose(master, shard_for_tp(ps, ours[name], spec, r, 2))
    assert res[0][5] == pytest.approx(res[1][5], abs=1e-6)


def _dp_save_worker(rank, world, root):
    from forgetrain_b200.parallel.topology import init_topology
    from forgetrain_b200.trainer import run_training_loop
    spec = _spec()
    topo = init_topology(1, device="cpu")
    rep = run_training_loop(spec=spec, cfg=_cfg(spec), topo=topo, num_steps=2, micro_batch_size=1,
                            seq_length=64, seed=3, save_dir=os.path.join(root, "dp2"), save_interval=2)
    tr = rep["trainer"]
    st = tr.opt.gather_full_state()
    return tr.store.named_cpu_params(), st["exp_avg"]["norm.weight"], st["master_weights"]["norm.weight"]


def test_a_dp2_checkpoint_loads_in_one_process(tmp_path):
    """The checkpoint does not depend on the number of data-parallel ranks that wrote it: ZeRO-1
    shards of the optimizer state are gathered before the write."""
    from forgetrain_b200.parallel.topology import Topology
    from forgetrain_b200.trainer import Trainer
    res = run_ranks(_dp_save_worker, 2, str(tmp_path))
    params, m_norm, master_norm = res[0]
    spec = _spec()
    tr = Trainer(spec, _cfg(spec), Topology(), seq_length=64, micro_batch_size=1, seed=99)
    state = tr.load(str(tmp_path / "dp2" / "step_0000002"))
    assert state["step"] == 2 and tr.opt.step_count == 2
    for name, t in params.items():
        assert torch.equal(tr.store.params[name], t), name
    full = tr.opt.gather_full_state()
    assert torch.equal(full["exp_avg"]["norm.weight"], m_norm)
    assert torch.equal(full["master_weights"]["norm.weight"], master_norm)
    out = tr.train_step(_batches(1, 1, 1, 64, spec.vocab_size))
    assert torch.isfinite(out["loss"]).all() and tr.opt.step_count == 3


def _unsharded_worker(rank, world, sharded):
    from forgetrain_b200.parallel.topology import init_topology
    from forgetrain_b200.trainer import Trainer
    spec = _spec()
    topo = init_topology(1, device="cpu")
    tr = Trainer(spec, _cfg(spec, sharded_optimizer=sharded), topo, seq_length=64, micro_batch_size=2,
                 seed=0)
    data = _batches(100 + rank, 1, 2, 64, spec.vocab_size)
    losses = [float(tr.train_step(data)["loss"]) for _ in range(3)]
    return losses, tr.store.named_cpu_params(), tr.opt.master.numel(), float(tr.opt.grad_norm)


def test_unsharded_optimizer_matches_zero1():
    """SHARDED_OPTIMIZER=0: all-reduced gradients and a full Adam state on every rank give the
    same training as the ZeRO-1 path, at twice the optimizer memory on two ranks."""
    z = run_ranks(_unsharded_worker, 2, True)
    u = run_ranks(_unsharded_worker, 2, False)
    assert u[0][0] == pytest.approx(z[0][0], abs=1e-6) and u[1][0] == pytest.approx(u[0][0], abs=1e-7)
    assert u[0][3] == pytest.approx(z[0][3], rel=1e-6)
    for name, t in z[0][1].items():
        assert torch.allclose(u[0][1][name], t, atol=1e-6), name
        assert torch.equal(u[0][1][name], u[1][1][name]), name       # replicas stay identical
    assert u[0][2] == 2 * z[0][2]


# ------------------------------------------------------------------------------------------
def _mtp_worker(rank, world, out_dir):
    """MTP losses: mean over micro-batches on each rank, mean over the data-parallel ranks,
    one value per extra layer in every step record (reference train_loop.py:326-364)."""
    from forgetrain_b200.parallel.topology import init_topology
    from forgetrain_b200.trainer import Trainer, run_training_loop
    spec = _spec(tie_embeddings=False)
    topo = init_topology(1, device="cpu")
    cfg = _cfg(spec, mtp_num_layers=2, mtp_loss_scaling_factor=0.3,
               profile_range="1,3", profile_output=os.path.join(out_dir, "prof.json"),
               profile_deep=True)
    rep = run_training_loop(spec=spec, cfg=cfg, topo=topo, num_steps=3, micro_batch_size=1,
                            seq_length=64, num_local_microbatches=2, seed=5)
    tr = rep["trainer"]
    # this rank's own per-layer losses of one more step, before any cross-rank averaging
    data = _batches(11 + rank, 2, 1, 64, spec.vocab_size)
    local = torch.zeros(2)
    for b in data:
        tr.mtp.forward_backward(b["tokens"], b["labels"], b.get("loss_mask"), 0.5, False)
        local += torch.stack([l.detach().reshape(()) for l in tr.mtp.last_mtp_losses]).float() / 2
    out = tr.train_step(data)
    return [s["mtp_loss_per_layer"] for s in rep["steps"]], [s["mtp_loss"] for s in rep["steps"]], \
        local, out["mtp_loss_per_layer"].clone()


def test_mtp_losses_are_averaged_over_microbatches_and_ranks_and_reported(tmp_path):
    res = run_ranks(_mtp_worker, 2, str(tmp_path))
    per_layer, total, _, _ = res[0]
    assert len(per_layer) == 3 and all(len(p) == 2 for p in per_layer)
    assert all(t == pytest.approx(sum(p) / 2) for p, t in zip(per_layer, total))
    assert res[0][0] == res[1][0]                      # every rank reports the global mean
    want = (res[0][2] + res[1][2]) / 2                 # mean of the two ranks' local means
    assert torch.allclose(res[0][3], want, atol=1e-5) and torch.allclose(res[1][3], want, atol=1e-5)
    # the deep profile of the same run: phases of a micro-batch and the closing gather segment
    import json
    doc = json.loads((tmp_path / "prof.json").read_text())
    assert doc["deep_mode"] is True and len(doc["records"]) == 2
    segs = doc["records"][0]["segments_ms"]
    assert {"mb_data", "microbatches", "reduce_scatter", "grad_norm", "optimizer",
            "loss_allreduce", "allgather"} <= set(segs)


# ------------------------------------------------------------------------------------------
def _accessor_worker(rank, world):
    import training_engine_tensor.nccl as N
    before = (N.get_rank(), N.get_world_size(), N.is_distributed())
    topo = N.init_topology(2, device="cpu")
    loss = torch.tensor(float(1 + topo.dp_rank))
    mean = N.allreduce_loss(loss)
    N.barrier()
    after = (N.get_rank(), N.get_world_size(), N.is_distributed(), N.get_tp_rank(), N.get_tp_size(),
             N.get_dp_rank(), N.get_dp_size(), N.get_tp_group() is topo.tp_group,
             N.get_dp_group() is topo.dp_group)
    return before, after, mean


def test_module_level_topology_accessors_follow_init_topology():
    """The accessors of ``training_engine_tensor.nccl`` describe one process before the groups are
    up and the rank's place in the TP x DP mesh afterwards (4 ranks: TP groups {0,1},{2,3}, DP
    groups {0,2},{1,3}); ``allreduce_loss`` averages over the data-parallel group."""
    res = run_ranks(_accessor_worker, 4)
    for rank in range(4):
        before, after, mean = res[rank]
        assert before == (0, 1, False)
        assert after == (rank, 4, True, rank % 2, 2, rank // 2, 2, True, True)
        assert mean == 1.5


# ------------------------------------------------------------------------------------------
def _padded_vocab_worker(rank, world, tp, mask=False, steps=1):
    from forgetrain_b200.parallel.topology import init_topology
    from forgetrain_b200.trainer import Trainer
    spec = _spec(vocab_size=500, tie_embeddings=False)
    topo = init_topology(tp, device="cpu")
    tr = Trainer(spec, _cfg(spec, tensor_parallel_size=tp, sequence_parallel=tp > 1, mask_vocab_padding=mask),
                 topo, seq_length=64, micro_batch_size=2, seed=0)
    data = _batches(7, 1, 2, 64, spec.vocab_size)
    losses = [float(tr.train_step(data)["loss"]) for _ in range(steps)]
    pad = tr.store.params["output.weight"][max(0, spec.vocab_size - tr.model.vocab_start):]
    return (losses[0] if steps == 1 else losses), tr.model.vocab_rows, float(pad.abs().sum())


def test_padded_vocabulary_rows_take_part_in_the_softmax_like_megatrons():
    """500 tokens over two ranks: 256 rows per rank, 12 zero-initialised pad rows in all. Their
    columns are in the softmax, so the first loss is above the TP = 1 loss by about
    log(1 + 12 / 500) (exactly that if every logit were zero)."""
    import math
    one, rows1, _ = run_ranks(_padded_vocab_worker, 1, 1)[0]
    two, rows2, _ = run_ranks(_padded_vocab_worker, 2, 2)[0]
    assert rows1 == 500 and rows2 == 256
    shift = two - one
    assert 0.5 * math.log(1 + 12 / 500) < shift < 1.2 * math.log(1 + 12 / 500), shift


def test_masked_vocabulary_padding_gives_the_loss_of_a_run_without_tensor_parallelism():
    """``mask_vocab_padding``: the pad columns carry no probability and no gradient, so TP = 2 over a
    vocabulary of 500 follows TP = 1 to fp32 rounding and the pad rows of the output table stay
    zero, where the default convention trains them."""
    one = run_ranks(_padded_vocab_worker, 1, 1, True, 3)[0][0]
    res = run_ranks(_padded_vocab_worker, 2, 2, True, 3)
    for rank in range(2):
        assert res[rank][0] == pytest.approx(one, abs=5e-6)
    assert res[1][2] == 0.0                                   # rank 1 holds the 12 pad rows
    default = run_ranks(_padded_vocab_worker, 2, 2, False, 3)
    assert default[1][2] > 0.0
