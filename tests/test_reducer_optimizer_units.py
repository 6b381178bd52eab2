"""Unit tests of the data-parallel plumbing on CPU: bucket layout, reducer lifecycle, gradient
norm over shards, the sharded optimizer's segment tables / state layout / update order, the
per-bucket gather events and the forward gate that waits for them. Modelled on the groups of
the reference's reducer suite (exports/train_engine_0.5B/tests/test_bucketed_grad_reducer.py:
layout 146-311, lifecycle 314-493, norm 756-848, all-gather pipeline 851-1037, sharded optimizer
1386-1697, state gather 1700-1864, multi-micro-batch 1867-2387), restated for an engine whose
weight gradients are written in place into the flat buffer (no staging buffers to test)."""
import pytest
import torch

from forgetrain_b200.config import load_model_spec
from forgetrain_b200.models.params import ParamStore
from forgetrain_b200.optim.adamw import ShardedAdamW
from forgetrain_b200.parallel.buckets import Bucket, compute_grad_buckets
from forgetrain_b200.parallel.dp import BucketedGradReducer


def _entries(sizes):
    out, off = [], 0
    for i, n in enumerate(sizes):
        out.append((f"p{i}", off, n))
        off += n
    return out


def _store(world=1, **kw):
    spec = load_model_spec("tiny", tie_embeddings=False, **kw)
    st = ParamStore(spec, "cpu", torch.float32, pad_to=128 * world, align=128 * world)
    st.init_random(0)
    return st


# ------------------------------------------------------------------------------ bucket layout
def test_single_param_smaller_than_target_is_one_bucket():
    (b,) = compute_grad_buckets(_entries([64]), world=4, target=1000)
    assert (b.index, b.start, b.size, b.params) == (0, 0, 64, ["p0"])
    assert b.param_offsets == {"p0": 0} and b.param_sizes == {"p0": 64}


def test_param_larger_than_target_gets_a_bucket_of_its_own():
    b = compute_grad_buckets(_entries([8, 400, 8, 8]), world=4, target=16)
    assert [x.params for x in b] == [["p0", "p1"], ["p2", "p3"]]
    b = compute_grad_buckets(_entries([400, 8, 8]), world=4, target=16)
    assert [x.params for x in b] == [["p0"], ["p1", "p2"]]


def test_offsets_inside_a_bucket_are_sequential_and_cover_it():
    b = compute_grad_buckets(_entries([8, 24, 16, 8, 40]), world=8, target=48)
    for x in b:
        pos = 0
        for n in x.params:
            assert x.param_offsets[n] == pos
            pos += x.param_sizes[n]
        assert pos == x.size


def test_buckets_tile_the_flat_buffer_without_gaps_or_overlap():
    ent = _entries([16, 8, 8, 64, 24, 8])
    b = compute_grad_buckets(ent, world=8, target=32)
    assert b[0].start == 0
    for x, y in zip(b[:-1], b[1:]):
        assert x.start + x.size == y.start
    assert b[-1].start + b[-1].size == sum(n for _, _, n in ent)
    assert sorted(n for x in b for n in x.params) == sorted(n for n, _, _ in ent)


@pytest.mark.parametrize("world", [1, 2, 4, 8])
def test_rank_shards_partition_every_bucket(world):
    st = _store(world)
    for b in compute_grad_buckets(st.entries(), world, 150_000):
        ranges = [b.shard_range(r, world) for r in range(world)]
        assert ranges[0][0] == b.start and ranges[-1][1] == b.start + b.size
        assert all(a[1] == c[0] for a, c in zip(ranges[:-1], ranges[1:]))
        assert all(hi - lo == b.shard_size(world) for lo, hi in ranges)
        assert b.shard_size(world) % 128 == 0          # 16-byte aligned in bf16, whole vectors


def test_layer_aligned_bucket_count_follows_rs_buckets():
    st = _store(4)
    total = st.total
    for k in (2, 4, 8):
        b = compute_grad_buckets(st.entries(), 4, max(1, total // k))
        assert 1 <= len(b) <= k + 1


# ------------------------------------------------------------------------------ reducer lifecycle
def _reducer(st, world=1, rank=0, target=150_000, **kw):
    return BucketedGradReducer(st.flat_grads, st.entries(), world, rank, None, target, backend="gloo", **kw)


def test_start_step_arms_one_pending_count_per_bucket():
    st = _store()
    red = _reducer(st)
    red.start_step()
    assert red.pending == [len(b.params) for b in red.buckets]
    assert float(red.sumsq) == 0.0 and not red.seen


def test_each_report_decrements_only_its_bucket():
    st = _store()
    red = _reducer(st)
    red.start_step()
    first = red.buckets[0].params[0]
    before = list(red.pending)
    red.on_grad_ready(first)
    assert red.pending[0] == before[0] - 1 and red.pending[1:] == before[1:]


def test_reports_outside_a_step_twice_or_unknown_are_errors():
    st = _store()
    red = _reducer(st)
    with pytest.raises(RuntimeError):
        red.on_grad_ready(st.order[0].name)           # before start_step
    red.start_step()
    with pytest.raises(KeyError):
        red.on_grad_ready("no.such.weight")
    red.on_grad_ready(st.order[0].name)
    with pytest.raises(RuntimeError):
        red.on_grad_ready(st.order[0].name)           # twice in one step


def test_wait_all_names_the_buckets_that_never_filled():
    st = _store()
    red = _reducer(st)
    red.start_step()
    for n in red.buckets[0].params:
        red.on_grad_ready(n)
    with pytest.raises(RuntimeError, match="never became ready"):
        red.wait_all()


def test_bucket_norm_is_accumulated_when_its_last_gradient_arrives():
    st = _store()
    st.flat_grads.normal_()
    red = _reducer(st)
    red.start_step()
    b0 = red.buckets[0]
    for n in b0.params[:-1]:
        red.on_grad_ready(n)
    assert float(red.sumsq) == 0.0
    red.on_grad_ready(b0.params[-1])
    want = st.flat_grads[b0.start:b0.start + b0.size].pow(2).sum()
    assert float(red.sumsq) == pytest.approx(float(want), rel=1e-5)


def test_views_address_the_flat_buffer_in_place():
    st = _store(4)
    red = _reducer(st, world=1)
    b = red.buckets[-1]
    red.bucket_view(b).fill_(3.0)
    assert float(st.flat_grads[b.start]) == 3.0 and float(st.flat_grads[b.start + b.size - 1]) == 3.0
    assert red.bucket_view(b).data_ptr() == st.flat_grads[b.start:].data_ptr()


def test_two_steps_are_independent():
    st = _store()
    red = _reducer(st)
    norms = []
    for step in range(2):
        st.flat_grads.fill_(float(step + 1))
        red.start_step()
        for ps in st.order:
            red.on_grad_ready(ps.name)
        red.wait_all()
        norms.append(float(red.local_sumsq()))
    assert norms[1] == pytest.approx(4 * norms[0], rel=1e-5)


# ------------------------------------------------------------------------------ gradient norm
def test_local_norm_covers_exactly_this_ranks_shards():
    st = _store(4)
    st.flat_grads.normal_()
    for rank in range(4):
        red = _reducer(st, world=1)                     # world 1 skips the collective ...
        red.world, red.rank = 4, rank                   # ... but the shard arithmetic is rank 4's
        red.start_step()
        red._active = True
        for b in red.buckets:
            red._accumulate_norm(b)
        want = sum(float(st.flat_grads[lo:hi].pow(2).sum())
                   for lo, hi in (b.shard_range(rank, 4) for b in red.buckets))
        assert float(red.local_sumsq()) == pytest.approx(want, rel=1e-5)


def test_norm_exclusion_only_removes_the_overlap_with_the_shard():
    st = _store(2)
    st.flat_grads.fill_(1.0)
    b0 = compute_grad_buckets(st.entries(), 2, 150_000)[0]
    lo, hi = b0.shard_range(0, 2)
    red = _reducer(st, world=1, norm_exclude=[(hi - 10, hi + 50)])
    red.world, red.rank = 2, 0
    red.start_step()
    for b in red.buckets:
        red._accumulate_norm(b)
    total = sum(b.shard_size(2) for b in red.buckets)
    assert float(red.local_sumsq()) == pytest.approx(total - 10)


# ------------------------------------------------------------------------------ sharded optimizer
def _opt(st, world=1, rank=0, target=150_000, **kw):
    buckets = compute_grad_buckets(st.entries(), world, target)
    return ShardedAdamW(st, buckets, world, rank, None, **kw)


@pytest.mark.parametrize("world", [1, 2, 8])
def test_state_is_one_shard_of_every_bucket(world):
    st = _store(world)
    opt = _opt(st, world, rank=world - 1)
    want = sum(b.size for b in opt.buckets) // world
    assert opt.master.numel() == opt.exp_avg.numel() == opt.exp_avg_sq.numel() == want
    assert opt.shard_off == [sum(b.shard_size(world) for b in opt.buckets[:i]) for i in range(len(opt.buckets))]
    assert float(opt.exp_avg.abs().sum()) == 0.0 and float(opt.exp_avg_sq.abs().sum()) == 0.0


def test_master_weights_start_as_the_shard_of_the_parameters():
    st = _store(4)
    for rank in (0, 3):
        opt = _opt(st, 4, rank)
        for i, b in enumerate(opt.buckets):
            lo, hi = b.shard_range(rank, 4)
            assert torch.equal(opt.master_view(i), st.flat_params[lo:hi].float())


def test_segment_tables_follow_parameters_across_shard_boundaries():
    st = _store(4)
    lr_div = st.spec.mup_width_scale if st.spec.mup_enabled else 1.0
    for rank in range(4):
        opt = _opt(st, 4, rank, weight_decay=0.1)
        for b, segs in zip(opt.buckets, opt.segments):
            s_lo, s_hi = b.shard_range(rank, 4)
            assert segs[-1][0] == s_hi - s_lo and all(a[0] < c[0] for a, c in zip(segs[:-1], segs[1:]))
            for end, wd, lrm, name in segs:
                ps = st.by_name[name]
                assert wd == (0.1 if ps.has_weight_decay else 0.0)
                assert lrm == pytest.approx(1.0 / lr_div if ps.mup_lr_scaled else 1.0)
                p_lo = b.start + b.param_offsets[name]
                assert p_lo < s_lo + end <= p_lo + b.param_sizes[name]   # the segment ends inside it


def test_norm_weights_get_no_weight_decay_and_full_learning_rate():
    st = _store()
    opt = _opt(st, weight_decay=0.1)
    seen = {name: (wd, lrm) for segs in opt.segments for _, wd, lrm, name in segs}
    for ps in st.specs:
        if ps.is_norm:
            assert seen[ps.name] == (0.0, 1.0)


def test_step_counts_and_bias_corrections_advance():
    st = _store()
    opt = _opt(st)
    st.flat_grads.normal_()
    for t in (1, 2, 3):
        opt.compute_clip(st.flat_grads.pow(2).sum().reshape(1))
        opt.step(1e-3)
        assert opt.step_count == t
        assert float(opt.hyper_host[4]) == pytest.approx(1 - 0.9 ** t)
        assert float(opt.hyper_host[5]) == pytest.approx(1 - 0.95 ** t)


def test_parameters_are_the_rounded_master_weights_after_a_step():
    spec = load_model_spec("tiny", tie_embeddings=False)
    st = ParamStore(spec, "cpu", torch.bfloat16)
    st.init_random(0)
    opt = _opt(st)
    st.flat_grads.normal_()
    opt.compute_clip(st.flat_grads.pow(2).sum().reshape(1))
    opt.step(1e-2)
    for i, b in enumerate(opt.buckets):
        assert torch.equal(st.flat_params[b.start:b.start + b.size], opt.master_view(i).to(torch.bfloat16))


def test_clip_coefficient_follows_the_global_norm():
    st = _store()
    opt = _opt(st, max_grad_norm=1.0)
    opt.compute_clip(torch.tensor([25.0]))
    assert float(opt.grad_norm) == pytest.approx(5.0) and float(opt.hyper[6]) == pytest.approx(1 / (5 + 1e-6))
    opt.compute_clip(torch.tensor([0.25]))
    assert float(opt.hyper[6]) == 1.0
    opt2 = _opt(st, max_grad_norm=0.0)                    # clipping disabled
    opt2.compute_clip(torch.tensor([1e6]))
    assert float(opt2.hyper[6]) == 1.0


def test_buckets_are_updated_in_forward_consumption_order():
    """Embedding first, head last: the reverse of the flat-buffer (backward) order."""
    st = _store()
    opt = _opt(st, target=60_000)
    assert len(opt.buckets) >= 3
    order = []
    real = opt._update_bucket
    opt._update_bucket = lambda i, lr, t: (order.append(i), real(i, lr, t))
    st.flat_grads.normal_()
    opt.compute_clip(st.flat_grads.pow(2).sum().reshape(1))
    opt.step(1e-3)
    assert order == list(reversed(range(len(opt.buckets))))
    assert "tok_embeddings.weight" in opt.buckets[order[0]].params
    assert "output.weight" in opt.buckets[order[-1]].params


def test_state_round_trip_through_the_rank_count_independent_form():
    st = _store()
    opt = _opt(st)
    st.flat_grads.normal_()
    opt.compute_clip(st.flat_grads.pow(2).sum().reshape(1))
    opt.step(1e-2)
    state = opt.gather_full_state()
    assert set(state) == {"master_weights", "exp_avg", "exp_avg_sq"}
    assert set(state["exp_avg"]) == {ps.name for ps in st.specs}
    assert all(state["exp_avg"][n].shape == tuple(st.shapes[n]) for n in state["exp_avg"])
    st2 = _store()
    opt2 = _opt(st2, target=40_000)                      # another bucket layout
    opt2.load_full_state(state, opt.step_count)
    again = opt2.gather_full_state()
    for f in state:
        for n in state[f]:
            assert torch.equal(state[f][n], again[f][n]), (f, n)
    assert opt2.step_count == 1


# ------------------------------------------------------------------------------ gather events / gate
class _FakeEvent:
    waited = []

    def __init__(self, i):
        self.i = i


def test_wait_bucket_consumes_each_event_once(monkeypatch):
    st = _store()
    opt = _opt(st, target=60_000)
    waited = []

    class FakeStream:
        def wait_event(self, ev):
            waited.append(ev.i)
    monkeypatch.setattr(torch.cuda, "current_stream", lambda: FakeStream())
    opt.ag_events = [_FakeEvent(i) for i in range(len(opt.buckets))]
    opt.wait_bucket(1)
    opt.wait_bucket(1)                                    # second call: nothing left to wait for
    assert waited == [1] and opt.ag_events[1] is None
    opt.wait_all_gathers()
    assert sorted(waited) == list(range(len(opt.buckets))) and not any(opt.ag_events)


def test_forward_gate_waits_per_layer_for_the_buckets_that_hold_its_parameters():
    from forgetrain_b200.engine_config import from_spec
    from forgetrain_b200.parallel.topology import Topology
    from forgetrain_b200.trainer import Trainer
    spec = load_model_spec("tiny", tie_embeddings=False)
    cfg = from_spec(spec, dtype="fp32", comm="nccl", wgrad_bucket_target_elems=60_000, rs_buckets=0)
    tr = Trainer(spec, cfg, Topology(), seq_length=64, micro_batch_size=1, seed=0)
    assert tr.model.param_gate is None                    # CPU: no side stream, no gate
    calls = []
    tr.opt.wait_bucket = lambda i: calls.append(i)
    tr._install_param_gate()
    nb = len(tr.opt.buckets)
    assert nb >= 3
    tr.model.param_gate("tok_embeddings")
    assert calls == [tr.reducer.bucket_of["tok_embeddings.weight"]]
    calls.clear()
    tr.model.param_gate("layers.0")
    want = sorted({tr.reducer.bucket_of[ps.name] for ps in tr.store.specs if ps.name.startswith("layers.0.")})
    assert sorted(calls) == want
    calls.clear()
    tr.model.param_gate("output")
    assert calls == [tr.reducer.bucket_of["output.weight"]]
    # a whole forward touches every bucket, the embedding's first and the head's last
    calls.clear()
    tokens = torch.randint(0, spec.vocab_size, (1, 64))
    tr.model.forward(tokens)
    assert set(calls) == set(range(nb))
    assert calls[0] == tr.reducer.bucket_of["tok_embeddings.weight"]
    assert calls[-1] == tr.reducer.bucket_of["output.weight"]


# ------------------------------------------------------------------------------ micro-batches
def test_gradient_accumulation_reduces_once_after_the_last_micro_batch():
    from forgetrain_b200.engine_config import from_spec
    from forgetrain_b200.parallel.topology import Topology
    from forgetrain_b200.trainer import Trainer
    spec = load_model_spec("tiny", tie_embeddings=False)
    cfg = from_spec(spec, dtype="fp32", comm="nccl", wgrad_bucket_target_elems=60_000, rs_buckets=0,
                    warmup_iters=0, max_lr=1e-3)
    tr = Trainer(spec, cfg, Topology(), seq_length=64, micro_batch_size=1, seed=0)
    reported = []
    real = tr.reducer.on_grad_ready
    tr.reducer.on_grad_ready = lambda n: (reported.append(n), real(n))
    g = torch.Generator().manual_seed(0)
    mk = lambda: {"tokens": torch.randint(0, spec.vocab_size, (1, 64), generator=g),
                  "labels": torch.randint(0, spec.vocab_size, (1, 64), generator=g)}
    batches = [mk(), mk(), mk()]
    tr.train_step(batches)
    assert sorted(reported) == sorted(ps.name for ps in tr.store.specs)   # once each, not three times
    # and the accumulated gradient is the mean of the three single-batch gradients
    acc = tr.store.flat_grads.clone()
    tr2 = Trainer(spec, cfg, Topology(), seq_length=64, micro_batch_size=1, seed=0)
    want = torch.zeros_like(acc)
    for b in batches:
        tr2.model.forward_backward(b["tokens"], b["labels"], None, 1.0 / 3, accumulate=False)
        want += tr2.store.flat_grads
    assert torch.allclose(acc, want, atol=1e-6)
