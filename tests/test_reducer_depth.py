"""Bucket layout, reducer life cycle and the sharded optimizer's bookkeeping, case by case.

The reference covers this host-side logic with about a hundred CPU cases (layout, life cycle,
round trips, parameters that straddle rank shards, state gathering, several micro-batches:
exports/train_engine_0.5B/tests/test_bucketed_grad_reducer.py:146-2387). The design here has no
pack / unpack step (gradients are produced in place in the flat buffer and reduced in place), so
the cases below check the in-place contract instead: what a rank's shard holds after the
reduction, which elements the optimizer of each rank owns, and what the gathered state is.
Ranks are threads of one process (``sim_world.SimDist``)."""
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


def _entries(sizes):
    out, off = [], 0
    for i, n in enumerate(sizes):
        out.append((f"p{i}", off, n))
        off += n
    return out


def _spec(layers=1):
    kw = dict(num_layers=layers, vocab_size=128, hidden_size=128, ffn_hidden_size=256,
              num_attention_heads=4, num_query_groups=2, head_dim=32, tie_embeddings=False)
    return load_model_spec("tiny", **kw)


def _store(world=1, layers=1, dtype=torch.float32, seed=0):
    st = ParamStore(_spec(layers), "cpu", dtype, pad_to=128 * world, align=128 * world)
    st.init_random(seed)
    return st


def _zero_padding(st):
    for name, off, n in st.entries():
        st.flat_grads[off + st.numel(name):off + n] = 0


# ---------------------------------------------------------------------------------------------
# layout
# ---------------------------------------------------------------------------------------------
def test_bucket_closes_exactly_at_the_target():
    b = compute_grad_buckets(_entries([8, 8, 8, 8]), world=2, target=16)
    assert [x.size for x in b] == [16, 16]
    b = compute_grad_buckets(_entries([8, 8, 8, 8]), world=2, target=17)
    assert [x.size for x in b] == [24, 8]                       # the last bucket may stay short


def test_target_above_the_total_gives_one_bucket_with_everything():
    e = _entries([8, 16, 24])
    b = compute_grad_buckets(e, world=8, target=10 ** 9)
    assert len(b) == 1 and b[0].size == 48 and b[0].params == ["p0", "p1", "p2"]
    assert b[0].param_offsets == {"p0": 0, "p1": 8, "p2": 24}


def test_target_of_one_element_gives_one_bucket_per_parameter():
    b = compute_grad_buckets(_entries([8, 16, 24]), world=8, target=1)
    assert [x.params for x in b] == [["p0"], ["p1"], ["p2"]]
    assert [x.start for x in b] == [0, 8, 24]
    assert all(x.param_offsets[x.params[0]] == 0 for x in b)


def test_world_one_accepts_any_size():
    b = compute_grad_buckets(_entries([3, 5, 7]), world=1, target=8)
    assert [x.size for x in b] == [8, 7]
    assert b[1].shard_range(0, 1) == (8, 15)


def test_a_flat_buffer_that_does_not_start_at_zero_keeps_its_base():
    e = [("a", 128, 8), ("b", 136, 8)]
    b = compute_grad_buckets(e, world=2, target=8)
    assert [x.start for x in b] == [128, 136]
    assert b[1].shard_range(1, 2) == (140, 144)


def test_zero_sized_and_overlapping_entries_are_rejected():
    with pytest.raises(ValueError, match="no elements"):
        compute_grad_buckets([("a", 0, 0)], world=1, target=8)
    with pytest.raises(ValueError, match="not contiguous"):
        compute_grad_buckets([("a", 0, 8), ("b", 4, 8)], world=1, target=8)


def test_error_message_of_an_unsplittable_bucket_names_the_bucket():
    with pytest.raises(ValueError, match="bucket 1 size 6"):
        compute_grad_buckets(_entries([8, 6]), world=4, target=8)


def test_layout_of_the_half_billion_model_under_the_default_target():
    """The 0.5B model at 8 data-parallel ranks with the default target: every parameter in one
    bucket, buckets in flat (= backward) order, and the embedding, which backward produces last,
    closes the last bucket."""
    from forgetrain_b200.engine_config import EngineConfig
    from forgetrain_b200.models.params import flat_buffer_order
    spec = load_model_spec("0.5b")
    pad = 128 * 8
    entries, off = [], 0
    for ps in flat_buffer_order(spec):
        n = (ps.numel + pad - 1) // pad * pad
        entries.append((ps.name, off, n))
        off += n
    buckets = compute_grad_buckets(entries, 8, EngineConfig().wgrad_bucket_target_elems)
    assert [n for b in buckets for n in b.params] == [e[0] for e in entries]
    assert buckets[-1].params[-1] == "tok_embeddings.weight"
    assert sum(b.size for b in buckets) == off
    assert all(b.shard_size(8) % 128 == 0 for b in buckets)     # 16-byte aligned bf16 / fp32 shards
    assert 2 <= len(buckets) <= 16


# ---------------------------------------------------------------------------------------------
# reducer: construction and life cycle
# ---------------------------------------------------------------------------------------------
def _reducer(world=1, rank=0, target=20000, layers=1, **kw):
    st = _store(world, layers)
    red = BucketedGradReducer(st.flat_grads, st.entries(), world, rank, None, target, backend="gloo", **kw)
    return st, red


def test_reducer_maps_every_parameter_to_its_bucket():
    st, red = _reducer(target=20000, layers=2)
    assert len(red.buckets) >= 3
    assert set(red.bucket_of) == set(st.offsets)
    for name, bi in red.bucket_of.items():
        assert name in red.buckets[bi].params
        assert red.buckets[bi].start + red.buckets[bi].param_offsets[name] == st.offsets[name]


def test_cpu_reducer_has_no_side_stream():
    _, red = _reducer(world=4, rank=0, overlap=True)
    assert red.overlap is False and red.comm_stream is None
    assert red.done_events == [None] * len(red.buckets)


def test_a_bucket_is_reduced_when_its_last_parameter_reports_in_any_order(monkeypatch):
    st, red = _reducer(target=20000, layers=2)
    issued = []
    monkeypatch.setattr(red, "_issue_bucket_reduce", lambda b: issued.append(b.index))
    red.start_step()
    order = [ps.name for ps in st.order]
    g = torch.Generator().manual_seed(3)
    perm = [order[i] for i in torch.randperm(len(order), generator=g).tolist()]
    left = {b.index: set(b.params) for b in red.buckets}
    for name in perm:
        bi = red.bucket_of[name]
        before = list(issued)
        red.on_grad_ready(name)
        left[bi].discard(name)
        assert (issued == before + [bi]) if not left[bi] else (issued == before)
    assert sorted(issued) == list(range(len(red.buckets)))


def test_backward_order_releases_buckets_front_to_back(monkeypatch):
    st, red = _reducer(target=20000, layers=2)
    issued = []
    monkeypatch.setattr(red, "_issue_bucket_reduce", lambda b: issued.append(b.index))
    red.start_step()
    for ps in st.order:                                          # flat order is backward order
        red.on_grad_ready(ps.name)
    assert issued == list(range(len(red.buckets)))


def test_start_step_forgets_an_aborted_step():
    st, red = _reducer(target=20000, layers=2)
    st.flat_grads.fill_(1.0)
    red.start_step()
    for name in red.buckets[0].params:
        red.on_grad_ready(name)                                   # bucket 0 is summed ...
    assert float(red.sumsq) > 0
    red.start_step()                                              # ... and the step is dropped
    assert float(red.sumsq) == 0 and not red.seen
    assert red.pending == [len(b.params) for b in red.buckets]
    for ps in st.order:
        red.on_grad_ready(ps.name)                                # no "reported twice"
    red.wait_all()


def test_a_failed_wait_keeps_the_step_open_for_the_late_gradient():
    st, red = _reducer()
    red.start_step()
    for ps in st.order[:-1]:
        red.on_grad_ready(ps.name)
    with pytest.raises(RuntimeError):
        red.wait_all()
    red.on_grad_ready(st.order[-1].name)
    red.wait_all()
    assert red._active is False


def test_unknown_parameter_does_not_consume_a_report():
    st, red = _reducer()
    red.start_step()
    before = list(red.pending)
    with pytest.raises(KeyError):
        red.on_grad_ready("layers.9.attention.wo.weight")
    assert red.pending == before and not red.seen


# ---------------------------------------------------------------------------------------------
# reducer: what the buffer holds after the reduction (ranks as threads)
# ---------------------------------------------------------------------------------------------
def _fill(st, rank, step=0):
    g = torch.Generator().manual_seed(17 + 1000 * step + rank)
    for ps in st.order:
        st.grads[ps.name].copy_(torch.randn(st.shapes[ps.name], generator=g))


def _reduce_once(world, monkeypatch, all_reduce=False, target=20000, layers=2, steps=1, order=None):
    sim = SimDist(world)
    monkeypatch.setattr(dp_mod, "dist", sim)

    def rank_main(r):
        st = _store(world, layers)
        red = BucketedGradReducer(st.flat_grads, st.entries(), world, r, None, target, backend="gloo",
                                  all_reduce=all_reduce)
        for s in range(steps):
            st.flat_grads.zero_()
            _fill(st, r, s)
            red.start_step()
            names = [ps.name for ps in st.order]
            for name in (order(names) if order else names):
                red.on_grad_ready(name)
            red.wait_all()
        return st, red

    return sim, sim.run(rank_main)


def _mean_grads(world, layers=2, step=0):
    acc = None
    for r in range(world):
        st = _store(world, layers)
        st.flat_grads.zero_()
        _fill(st, r, step)
        acc = st.flat_grads.clone() if acc is None else acc + st.flat_grads
    return acc / world


@pytest.mark.parametrize("world", [2, 3, 4])
def test_each_rank_holds_the_mean_of_its_own_shard(world, monkeypatch):
    _, out = _reduce_once(world, monkeypatch)
    want = _mean_grads(world)
    for r, (st, red) in enumerate(out):
        for b in red.buckets:
            lo, hi = b.shard_range(r, world)
            assert torch.allclose(st.flat_grads[lo:hi], want[lo:hi], rtol=1e-6, atol=1e-7)


def test_all_reduce_mode_leaves_the_whole_mean_on_every_rank(monkeypatch):
    world = 3
    _, out = _reduce_once(world, monkeypatch, all_reduce=True)
    want = _mean_grads(world)
    for st, _ in out:
        assert torch.allclose(st.flat_grads, want, rtol=1e-6, atol=1e-7)


def test_padding_stays_zero_through_reductions(monkeypatch):
    world = 4
    _, out = _reduce_once(world, monkeypatch, steps=3)
    for st, _ in out:
        for name, off, n in st.entries():
            assert not st.flat_grads[off + st.numel(name):off + n].any(), name


def test_rank_norms_add_up_to_the_norm_of_the_mean_gradient(monkeypatch):
    world = 4
    _, out = _reduce_once(world, monkeypatch)
    want = float(_mean_grads(world).pow(2).sum())
    parts = [float(red.local_sumsq()) for _, red in out]
    assert sum(parts) == pytest.approx(want, rel=1e-5)
    assert all(p > 0 for p in parts)


def test_norm_in_all_reduce_mode_still_counts_every_element_once(monkeypatch):
    world = 4
    _, out = _reduce_once(world, monkeypatch, all_reduce=True)
    want = float(_mean_grads(world).pow(2).sum())
    assert sum(float(red.local_sumsq()) for _, red in out) == pytest.approx(want, rel=1e-5)


def test_second_step_does_not_see_the_first(monkeypatch):
    world = 2
    _, out = _reduce_once(world, monkeypatch, steps=2)
    want = _mean_grads(world, step=1)
    for r, (st, red) in enumerate(out):
        for b in red.buckets:
            lo, hi = b.shard_range(r, world)
            assert torch.allclose(st.flat_grads[lo:hi], want[lo:hi], rtol=1e-6, atol=1e-7)
        total = sum(float(x[1].local_sumsq()) for x in out)
    assert total == pytest.approx(float(want.pow(2).sum()), rel=1e-5)


def test_the_same_arrival_order_on_every_rank_gives_the_same_collective_order(monkeypatch):
    """Buckets are reduced in the order in which they complete; ranks must agree on it, which they
    do because every rank runs the same backward. An order other than the flat one is fine."""
    world = 2
    sim, out = _reduce_once(world, monkeypatch, order=lambda names: list(reversed(names)))
    sizes = [int(c.split("[")[1][:-1]) for c in sim.calls]
    assert sizes == [b.size for b in reversed(out[0][1].buckets)]
    want = _mean_grads(world)
    for r, (st, red) in enumerate(out):
        for b in red.buckets:
            lo, hi = b.shard_range(r, world)
            assert torch.allclose(st.flat_grads[lo:hi], want[lo:hi], rtol=1e-6, atol=1e-7)


# ---------------------------------------------------------------------------------------------
# gradient norm: excluded ranges against rank shards
# ---------------------------------------------------------------------------------------------
def _norm_with_exclusion(world, rank, exclude, fill=1.0):
    st, red = _reducer(world=world, rank=rank, target=10 ** 9, norm_exclude=exclude)
    st.flat_grads.fill_(fill)
    # single-process stand-in: the reduction itself is not under test here, only the ranges
    red.start_step()
    red.sumsq += sum(red.shard_view(b).pow(2).sum() for b in red.buckets)
    return st, red


def test_excluded_range_inside_the_shard_is_subtracted_once():
    st, red = _norm_with_exclusion(4, 1, [])
    b = red.buckets[0]
    lo, hi = b.shard_range(1, 4)
    red.norm_exclude = [(lo + 10, lo + 110)]
    assert float(red.local_sumsq()) == (hi - lo) - 100


def test_excluded_range_that_straddles_the_shard_counts_only_the_overlap():
    st, red = _norm_with_exclusion(4, 1, [])
    lo, hi = red.buckets[0].shard_range(1, 4)
    red.norm_exclude = [(lo - 50, lo + 30)]
    assert float(red.local_sumsq()) == (hi - lo) - 30
    red.norm_exclude = [(hi - 7, hi + 1000)]
    assert float(red.local_sumsq()) == (hi - lo) - 7


def test_excluded_range_outside_the_shard_changes_nothing():
    st, red = _norm_with_exclusion(4, 1, [])
    lo, hi = red.buckets[0].shard_range(1, 4)
    red.norm_exclude = [(0, lo), (hi, hi + 64)]
    assert float(red.local_sumsq()) == hi - lo


def test_exclusion_over_all_ranks_removes_the_range_exactly_once():
    world = 4
    st0, _ = _reducer(world=world, rank=0, target=10 ** 9)
    name = "layers.0.attention.wqkv.weight"
    o, n = st0.offsets[name], st0.numel(name)
    total = 0.0
    for r in range(world):
        st, red = _norm_with_exclusion(world, r, [(o, o + n)], fill=2.0)
        total += float(red.local_sumsq())
    assert total == 4.0 * (st0.flat_grads.numel() - n)


def test_local_sumsq_does_not_change_the_accumulator():
    st, red = _norm_with_exclusion(2, 0, [])
    lo, hi = red.buckets[0].shard_range(0, 2)
    red.norm_exclude = [(lo, lo + 10)]
    a = float(red.local_sumsq())
    assert float(red.local_sumsq()) == a and float(red.sumsq) == hi - lo


# ---------------------------------------------------------------------------------------------
# sharded optimizer: ownership tables
# ---------------------------------------------------------------------------------------------
def _opt(world=1, rank=0, target=20000, layers=2, dtype=torch.float32, **kw):
    st = _store(world, layers, dtype)
    buckets = compute_grad_buckets(st.entries(), world, target)
    return st, ShardedAdamW(st, buckets, world, rank, None, **kw)


def test_segment_tables_tile_every_shard():
    for world, rank in ((1, 0), (4, 0), (4, 3), (8, 5)):
        st, opt = _opt(world, rank)
        for b, segs in zip(opt.buckets, opt.segments):
            ends = [s[0] for s in segs]
            assert ends == sorted(ends) and len(set(ends)) == len(ends)
            assert ends[-1] == b.shard_size(world) and ends[0] > 0


def test_segments_carry_the_class_of_their_parameter():
    st, opt = _opt(4, 1, weight_decay=0.25)
    for segs in opt.segments:
        for end, wd, lrm, name in segs:
            ps = st.by_name[name]
            assert wd == (0.25 if ps.has_weight_decay else 0.0)
            assert ps.is_norm == (wd == 0.0)
            want_lrm = 1.0 / st.spec.mup_width_scale if (ps.mup_lr_scaled and st.spec.mup_enabled) else 1.0
            assert lrm == want_lrm


def test_a_parameter_that_straddles_shards_is_owned_piecewise_by_its_ranks():
    world = 4
    pieces = {}
    for r in range(world):
        st, opt = _opt(world, r, target=10 ** 9)
        b = opt.buckets[0]
        s_lo, _ = b.shard_range(r, world)
        a = 0
        for end, _, _, name in opt.segments[0]:
            pieces.setdefault(name, []).append((s_lo + a, s_lo + end))
            a = end
    st, opt = _opt(world, 0, target=10 ** 9)
    b = opt.buckets[0]
    assert any(len(v) > 1 for v in pieces.values())              # the case exists at this size
    for name, spans in pieces.items():
        spans.sort()
        assert spans[0][0] == b.start + b.param_offsets[name]
        assert spans[-1][1] == spans[0][0] + b.param_sizes[name]
        assert all(x[1] == y[0] for x, y in zip(spans, spans[1:]))


def test_mup_learning_rate_class_can_be_switched_off():
    st, opt = _opt(1, 0, mup_lr_scaling=False)
    assert all(s[2] == 1.0 for segs in opt.segments for s in segs)


# ---------------------------------------------------------------------------------------------
# sharded optimizer: one step
# ---------------------------------------------------------------------------------------------
def test_prepare_host_launches_nothing():
    st, opt = _opt()
    before = st.flat_params.clone()
    opt.prepare_host(1e-2)
    assert opt.step_count == 1 and torch.equal(st.flat_params, before)
    assert not opt.exp_avg.any()


def test_zero_gradient_decays_matrices_and_leaves_norm_weights():
    st, opt = _opt(weight_decay=0.1)
    st.flat_grads.zero_()
    before = {n: p.clone() for n, p in st.params.items()}
    opt.compute_clip(torch.zeros(1))
    opt.step(1e-2)
    for ps in st.order:
        lrm = 1.0 / st.spec.mup_width_scale if (ps.mup_lr_scaled and st.spec.mup_enabled) else 1.0
        if ps.is_norm:
            assert torch.equal(st.params[ps.name], before[ps.name]), ps.name
        else:
            want = before[ps.name] * (1.0 - 1e-2 * lrm * 0.1)
            assert torch.allclose(st.params[ps.name], want, rtol=1e-6, atol=1e-9), ps.name


def test_parameter_padding_stays_zero_after_steps():
    st, opt = _opt(world=1)
    for s in range(3):
        _fill(st, 0, s)
        _zero_padding(st)
        opt.compute_clip(st.flat_grads.pow(2).sum().reshape(1))
        opt.step(1e-2)
    for name, off, n in st.entries():
        assert not st.flat_params[off + st.numel(name):off + n].any(), name


def test_clip_is_one_when_clipping_is_off_or_the_norm_is_small():
    st, opt = _opt(max_grad_norm=0.0)
    opt.compute_clip(torch.tensor([1e6]))
    assert float(opt.hyper[6]) == 1.0 and float(opt.grad_norm) == pytest.approx(1e3)
    st, opt = _opt(max_grad_norm=1.0)
    opt.compute_clip(torch.tensor([0.25]))
    assert float(opt.hyper[6]) == 1.0
    opt.compute_clip(torch.tensor([16.0]))
    assert float(opt.hyper[6]) == pytest.approx(1.0 / (4.0 + 1e-6))


def test_clip_scales_the_gradient_the_update_sees():
    """Adam's first step moves every weight by lr * sign(g) whatever the scale, so the clip shows in
    the moments: m = (1 - beta1) * clip * g."""
    st, opt = _opt(weight_decay=0.0)
    _fill(st, 0)
    _zero_padding(st)
    g = st.flat_grads.clone()
    opt.compute_clip(g.pow(2).sum().reshape(1))
    clip = float(opt.hyper[6])
    assert clip < 1.0
    opt.step(1e-3)
    for i, b in enumerate(opt.buckets):
        lo, hi = b.shard_range(0, 1)
        _, m, v = opt._views(i)
        assert torch.allclose(m, 0.1 * clip * g[lo:hi], rtol=1e-5, atol=1e-9)
        assert torch.allclose(v, 0.05 * (clip * g[lo:hi]) ** 2, rtol=1e-4, atol=1e-12)


def test_cpu_wait_calls_are_no_ops():
    st, opt = _opt()
    opt.step(1e-3)
    assert opt.ag_events == [None] * len(opt.buckets)
    opt.wait_bucket(0)
    opt.wait_all_gathers()
    opt.set_schedule(1e-2, 1e-3, 10, 100, 10)                     # device schedule: CUDA only
    assert opt.sched is None and opt.step_dev is None


# ---------------------------------------------------------------------------------------------
# sharded optimizer: state in and out
# ---------------------------------------------------------------------------------------------
def _train(st, opt, steps, first=0):
    for s in range(first, first + steps):
        _fill(st, 0, s)
        _zero_padding(st)
        opt.compute_clip(st.flat_grads.pow(2).sum().reshape(1))
        opt.step(1e-2)


def test_gathered_state_has_every_field_name_and_shape():
    st, opt = _opt()
    _train(st, opt, 2)
    state = opt.gather_full_state()
    assert set(state) == {"master_weights", "exp_avg", "exp_avg_sq"}
    for field in state:
        assert set(state[field]) == set(st.offsets)
        for name, t in state[field].items():
            assert tuple(t.shape) == tuple(st.shapes[name]) and t.dtype == torch.float32
    for name in st.offsets:
        assert torch.equal(state["master_weights"][name], st.params[name])    # fp32 store
        assert state["exp_avg_sq"][name].min() >= 0


def test_gathered_state_does_not_alias_the_optimizer():
    st, opt = _opt()
    _train(st, opt, 1)
    state = opt.gather_full_state()
    keep = {n: t.clone() for n, t in state["exp_avg"].items()}
    _train(st, opt, 1, first=1)
    for n in keep:
        assert torch.equal(state["exp_avg"][n], keep[n])


def test_state_round_trip_continues_bit_for_bit():
    st_a, opt_a = _opt()
    _train(st_a, opt_a, 2)
    state = opt_a.gather_full_state()
    st_b, opt_b = _opt(target=7000)                               # another bucket layout
    assert len(opt_b.buckets) != len(opt_a.buckets)
    opt_b.load_full_state(state, opt_a.step_count)
    opt_b.sync_params_from_master()
    assert opt_b.step_count == 2
    for n in st_a.offsets:
        assert torch.equal(st_b.params[n], st_a.params[n])
    _train(st_a, opt_a, 2, first=2)
    _train(st_b, opt_b, 2, first=2)
    for n in st_a.offsets:
        assert torch.equal(st_b.params[n], st_a.params[n]), n


def test_loading_a_state_into_a_rank_fills_only_its_elements():
    st1, opt1 = _opt()
    _train(st1, opt1, 1)
    state = opt1.gather_full_state()
    world = 4
    for r in range(world):
        st, opt = _opt(world, r)
        opt.load_full_state(state, 1)
        for i, b in enumerate(opt.buckets):
            s_lo, s_hi = b.shard_range(r, world)
            m = opt._views(i)[1]
            for name in b.params:
                p_lo = b.start + b.param_offsets[name]
                a, z = max(p_lo, s_lo), min(p_lo + st.numel(name), s_hi)
                if z > a:
                    want = state["exp_avg"][name].reshape(-1)[a - p_lo:z - p_lo]
                    assert torch.equal(m[a - s_lo:z - s_lo], want)


def test_master_and_parameters_sync_both_ways():
    st, opt = _opt(dtype=torch.bfloat16)
    for i in range(len(opt.buckets)):
        opt.master_view(i).add_(0.5)
    opt.sync_params_from_master()
    for i, b in enumerate(opt.buckets):
        lo, hi = b.shard_range(0, 1)
        assert torch.equal(st.flat_params[lo:hi], opt.master_view(i).to(torch.bfloat16))
    st.flat_params.mul_(2)
    opt.sync_master_from_params()
    for i, b in enumerate(opt.buckets):
        lo, hi = b.shard_range(0, 1)
        assert torch.equal(opt.master_view(i), st.flat_params[lo:hi].float())


# ---------------------------------------------------------------------------------------------
# reducer + optimizer over ranks: gathers and the state of all three fields
# ---------------------------------------------------------------------------------------------
def _ranks(world, steps, monkeypatch, target=20000, dtype=torch.float32):
    sim = SimDist(world)
    monkeypatch.setattr(dp_mod, "dist", sim)
    monkeypatch.setattr(adamw_mod, "dist", sim)

    def rank_main(r):
        st = _store(world, 2, dtype)
        red = BucketedGradReducer(st.flat_grads, st.entries(), world, r, None, target, backend="gloo")
        opt = ShardedAdamW(st, red.buckets, world, r, None, norm_reduce=lambda t: sim.all_reduce(t))
        for s in range(steps):
            st.flat_grads.zero_()
            _fill(st, r, s)
            red.start_step()
            for ps in st.order:
                red.on_grad_ready(ps.name)
            red.wait_all()
            opt.compute_clip(red.local_sumsq())
            opt.step(1e-2)
        return st, opt

    return sim, sim.run(rank_main)


@pytest.mark.parametrize("world", [2, 4])
def test_every_rank_ends_a_step_with_identical_parameters(world, monkeypatch):
    _, out = _ranks(world, 2, monkeypatch, dtype=torch.bfloat16)
    for st, _ in out[1:]:
        assert torch.equal(st.flat_params, out[0][0].flat_params)
    fresh = _store(world, 2, torch.bfloat16)
    assert not torch.equal(out[0][0].flat_params, fresh.flat_params)   # and they did move


def test_gathers_follow_the_update_order(monkeypatch):
    world = 2
    sim, out = _ranks(world, 1, monkeypatch)
    buckets = out[0][1].buckets
    gathers = [int(c.split("[")[1][:-1]) for c in sim.calls if c.startswith("all_gather")]
    assert gathers == [b.shard_size(world) for b in reversed(buckets)]


def test_state_gather_over_ranks_returns_all_three_fields_whole(monkeypatch):
    world = 4
    sim, out = _ranks(world, 2, monkeypatch)
    states = sim.run(lambda r: out[r][1].gather_full_state())
    for field in ("master_weights", "exp_avg", "exp_avg_sq"):
        for name in out[0][0].offsets:
            for s in states[1:]:
                assert torch.equal(s[field][name], states[0][field][name])
            assert states[0][field][name].abs().sum() > 0, (field, name)
    # the gathered master weights are what the parameters hold (fp32 store: exactly)
    for name in out[0][0].offsets:
        assert torch.equal(states[0]["master_weights"][name], out[0][0].params[name])


def test_optimizer_state_per_rank_is_one_nth(monkeypatch):
    world = 4
    _, out = _ranks(world, 1, monkeypatch)
    total = out[0][0].flat_params.numel()
    for _, opt in out:
        assert opt.master.numel() * world == total


def test_ranks_that_do_not_write_take_part_in_the_gathers_without_keeping_the_state(monkeypatch):
    world = 4
    sim, out = _ranks(world, 1, monkeypatch)
    sim.calls.clear()
    states = sim.run(lambda r: out[r][1].gather_full_state(keep=(r == 0)))
    n_gathers = len([c for c in sim.calls if c.startswith("all_gather")])
    assert n_gathers == 3 * len(out[0][1].buckets)               # the same collectives as before
    assert set(states[0]["exp_avg"]) == set(out[0][0].offsets)
    for s in states[1:]:
        assert s == {"master_weights": {}, "exp_avg": {}, "exp_avg_sq": {}}
