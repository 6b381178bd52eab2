"""Data-parallel reduction + ZeRO-1 optimizer at world sizes 2..8 in ONE process (threads as ranks).

The reference tests the same logic with simulated multi-rank shard overlap on CPU
(exports/train_engine_0.5B/tests/test_bucketed_grad_reducer.py:1386-1865); here the real
``BucketedGradReducer`` and ``ShardedAdamW`` run unmodified against an in-process stand-in for the
process group."""
import math

import pytest
import torch

from forgetrain_b200.config import load_model_spec
from forgetrain_b200.models.params import ParamStore
from forgetrain_b200.optim import adamw as adamw_mod
from forgetrain_b200.optim.adamw import ShardedAdamW
from forgetrain_b200.parallel import dp as dp_mod
from forgetrain_b200.parallel.buckets import compute_grad_buckets
from forgetrain_b200.parallel.dp import BucketedGradReducer
from sim_world import SimDist

TARGET = 40_000


def _spec():
    return load_model_spec("tiny", num_layers=2, vocab_size=256, hidden_size=128, ffn_hidden_size=256,
                           num_attention_heads=4, num_query_groups=2, head_dim=32, tie_embeddings=False)


def _store(world):
    st = ParamStore(_spec(), "cpu", torch.float32, pad_to=128 * world, align=128 * world)
    st.init_random(0)
    return st


def _close(a, b):
    """Equal up to fp32 summation order. Where a mean gradient is ~0 the Adam ratio g/(|g|+eps) is
    ill-conditioned and 1/W is inexact for W = 3, so a handful of elements may move by ~1e-5."""
    d = (a - b).abs()
    return int((d > 2e-6).sum()) <= max(1, a.numel() // 10_000) and float(d.max()) < 2e-4


def _rank_grads(st, step, rank):
    """Deterministic per-(step, rank) gradients, zero in the padding."""
    g = torch.Generator().manual_seed(1000 * step + rank)
    for ps in st.order:
        st.grads[ps.name].copy_(torch.randn(st.shapes[ps.name], generator=g))


def _reference(world, steps, lr=1e-2):
    """One process, gradients = mean over the ranks' gradients."""
    st = _store(world)      # same padding as the ranks, so flat offsets agree
    opt = ShardedAdamW(st, compute_grad_buckets(st.entries(), 1, TARGET), 1, 0, None)
    norms = []
    tmp = _store(world)
    for s in range(steps):
        acc = torch.zeros_like(st.flat_grads)
        for r in range(world):
            _rank_grads(tmp, s, r)
            acc += tmp.flat_grads / world
        st.flat_grads.copy_(acc)
        opt.compute_clip(acc.pow(2).sum().reshape(1))
        norms.append(float(opt.grad_norm))
        opt.step(lr)
    return st, opt, norms


def _run_ranks(sim, world, steps, monkeypatch, lr=1e-2, state_in=None):
    monkeypatch.setattr(dp_mod, "dist", sim)
    monkeypatch.setattr(adamw_mod, "dist", sim)

    def rank_main(r):
        st = _store(world)
        red = BucketedGradReducer(st.flat_grads, st.entries(), world, r, None, TARGET, backend="gloo")
        opt = ShardedAdamW(st, red.buckets, world, r, None, norm_reduce=lambda t: sim.all_reduce(t))
        if state_in is not None:
            opt.load_full_state(state_in[0], state_in[1])
            opt.sync_params_from_master()
        norms = []
        for s in range(opt.step_count, opt.step_count + steps):
            _rank_grads(st, s, r)
            red.start_step()
            for ps in st.order:                       # backward order = flat order
                red.on_grad_ready(ps.name)
            red.wait_all()
            opt.compute_clip(red.local_sumsq())
            norms.append(float(opt.grad_norm))
            opt.step(lr)
        return st, opt, norms, red

    return sim.run(rank_main)


@pytest.mark.parametrize("world", [2, 3, 4, 8])
def test_sharded_training_matches_one_process(world, monkeypatch):
    steps = 3
    ref_st, ref_opt, ref_norms = _reference(world, steps)
    out = _run_ranks(SimDist(world), world, steps, monkeypatch)
    for st, opt, norms, red in out:
        assert norms == pytest.approx(ref_norms, rel=1e-5)          # padding excluded, 1/W applied
        assert _close(st.flat_params, ref_st.flat_params)
        assert opt.step_count == steps
    # a parameter straddles rank shards inside a bucket (the case the segment tables exist for)
    red = out[0][3]
    assert any(b.param_sizes[n] > b.shard_size(world) for b in red.buckets for n in b.params)
    # every rank holds 1/W of the optimizer state
    assert out[0][1].master.numel() * world == sum(b.size for b in red.buckets)


def test_collective_schedule_is_one_reduce_per_bucket_then_norm_then_gathers(monkeypatch):
    world = 4
    sim = SimDist(world)
    out = _run_ranks(sim, world, 1, monkeypatch)
    nb = len(out[0][3].buckets)
    assert nb >= 3
    kinds = [c.split("[")[0] for c in sim.calls]
    assert kinds == ["all_reduce"] * nb + ["all_reduce"] + ["all_gather"] * nb
    assert sim.calls[nb] == "all_reduce[1]"                          # the squared norm
    sizes = [int(c.split("[")[1][:-1]) for c in sim.calls[:nb]]
    assert sizes == [b.size for b in out[0][3].buckets]


def test_state_is_rank_count_independent(monkeypatch):
    """State gathered at world 4 equals the one-process state, and loads at world 2 and 8."""
    ref_st, ref_opt, _ = _reference(4, 2)
    want = ref_opt.gather_full_state()
    sim = SimDist(4)
    out = _run_ranks(sim, 4, 2, monkeypatch)
    states = sim.run(lambda r: out[r][1].gather_full_state())
    for state in states:
        for field in ("master_weights", "exp_avg", "exp_avg_sq"):
            assert set(state[field]) == set(want[field])
            for name in want[field]:
                assert _close(state[field][name], want[field][name]), (field, name)
    # continue for one more step from that state at other world sizes
    ref4_st, _, _ = _reference(4, 3)
    for world in (2, 8):
        # per-rank gradients differ with the world size, so build the matching reference:
        # restart it from the gathered state and take one step with this world's mean gradient
        st = _store(world)
        opt = ShardedAdamW(st, compute_grad_buckets(st.entries(), 1, TARGET), 1, 0, None)
        opt.load_full_state(states[0], 2)
        opt.sync_params_from_master()
        tmp = _store(world)
        acc = torch.zeros_like(st.flat_grads)
        for r in range(world):
            _rank_grads(tmp, 2, r)
            acc += tmp.flat_grads / world
        st.flat_grads.copy_(acc)
        opt.compute_clip(acc.pow(2).sum().reshape(1))
        opt.step(1e-2)
        res = _run_ranks(SimDist(world), world, 1, monkeypatch, state_in=(states[0], 2))
        for rst, ropt, _, _ in res:
            assert ropt.step_count == 3
            for ps in st.order:        # offsets differ with the padding: compare per parameter
                assert _close(rst.params[ps.name], st.params[ps.name]), ps.name


def test_a_rank_that_raises_ends_the_others(monkeypatch):
    """Host-side failure: one simulated rank raises before its collective; the others are released
    from the rendezvous instead of waiting for ever, and the error reaches the caller."""
    sim = SimDist(3)
    monkeypatch.setattr(dp_mod, "dist", sim)

    def rank_main(r):
        if r == 1:
            raise RuntimeError("rank 1 lost its data loader")
        t = torch.ones(4)
        sim.all_reduce(t)
        return t

    with pytest.raises(RuntimeError, match="rank 1 lost"):
        sim.run(rank_main)


def test_unreported_gradient_is_an_error_not_a_hang(monkeypatch):
    world = 2
    sim = SimDist(world)
    monkeypatch.setattr(dp_mod, "dist", sim)

    def rank_main(r):
        st = _store(world)
        red = BucketedGradReducer(st.flat_grads, st.entries(), world, r, None, 10 ** 9, backend="gloo")
        red.start_step()
        for ps in st.order[:-1]:                      # the last gradient never arrives
            red.on_grad_ready(ps.name)
        with pytest.raises(RuntimeError, match="never became ready"):
            red.wait_all()
        return True

    assert sim.run(rank_main) == [True, True]


def test_clip_uses_the_global_norm(monkeypatch):
    world = 4
    out = _run_ranks(SimDist(world), world, 1, monkeypatch)
    norms = [o[2][0] for o in out]
    assert max(norms) - min(norms) < 1e-6 * max(norms)
    clip = [float(o[1].hyper[6]) for o in out]
    assert all(math.isclose(c, min(1.0, 1.0 / (norms[0] + 1e-6)), rel_tol=1e-5) for c in clip)
