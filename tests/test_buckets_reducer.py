import pytest
import torch

from forgetrain_b200.config import load_model_spec
from forgetrain_b200.models.params import ParamStore, flat_buffer_order
from forgetrain_b200.parallel.buckets import compute_grad_buckets
from forgetrain_b200.parallel.dp import BucketedGradReducer


def _entries(sizes):
    out, off = [], 0
    for i, n in enumerate(sizes):
        out.append((f"p{i}", off, n))
        off += n
    return out


def test_bucket_layout_greedy_close():
    b = compute_grad_buckets(_entries([8, 8, 16, 4, 4]), world=4, target=16)
    assert [x.params for x in b] == [["p0", "p1"], ["p2"], ["p3", "p4"]]
    assert [x.size for x in b] == [16, 16, 8]
    assert b[1].start == 16 and b[2].param_offsets == {"p3": 0, "p4": 4}
    assert b[0].shard_range(1, 4) == (4, 8)


def test_bucket_validation():
    with pytest.raises(ValueError):
        compute_grad_buckets(_entries([8]), world=0, target=8)
    with pytest.raises(ValueError):
        compute_grad_buckets(_entries([8]), world=2, target=0)
    with pytest.raises(ValueError):
        compute_grad_buckets([], world=2, target=8)
    with pytest.raises(ValueError):   # a bucket that cannot be split evenly
        compute_grad_buckets(_entries([6]), world=4, target=8)
    with pytest.raises(ValueError):   # hole in the flat buffer
        compute_grad_buckets([("a", 0, 8), ("b", 16, 8)], world=2, target=8)


def test_flat_order_is_reverse_registration():
    spec = load_model_spec("tiny", tie_embeddings=False)
    names = [p.name for p in flat_buffer_order(spec)]
    assert names[0] == "output.weight" and names[1] == "norm.weight"
    assert names[2] == "layers.3.feed_forward.w2.weight"
    assert names[2:8] == [f"layers.3.{s}" for s in ("feed_forward.w2.weight", "feed_forward.wfc1.weight",
                                                   "ffn_norm.weight", "attention.wqkv.weight",
                                                   "attention_norm.weight", "attention.wo.weight")]
    assert names[-1] == "tok_embeddings.weight"


def test_param_never_straddles_buckets_but_may_straddle_shards():
    spec = load_model_spec("tiny", tie_embeddings=False)
    store = ParamStore(spec, "cpu", torch.float32, pad_to=128 * 8, align=128 * 8)
    buckets = compute_grad_buckets(store.entries(), 8, 300_000)
    seen = set()
    for b in buckets:
        assert b.size % 8 == 0
        for n in b.params:
            assert n not in seen
            seen.add(n)
            assert 0 <= b.param_offsets[n] and b.param_offsets[n] + b.param_sizes[n] <= b.size
    assert seen == set(store.offsets)
    big = max(buckets, key=lambda b: b.size)
    assert any(b.param_sizes[n] > big.shard_size(8) for b in buckets for n in b.params)


def _reducer(world=1, rank=0, target=20000):
    spec = load_model_spec("tiny", num_layers=1, vocab_size=128, hidden_size=128, ffn_hidden_size=256,
                           num_attention_heads=4, num_query_groups=2, head_dim=32, tie_embeddings=False)
    store = ParamStore(spec, "cpu", torch.float32, pad_to=128 * world, align=128 * world)
    red = BucketedGradReducer(store.flat_grads, store.entries(), world, rank, None, target)
    return store, red


def test_reducer_lifecycle_and_errors():
    store, red = _reducer()
    with pytest.raises(RuntimeError):
        red.on_grad_ready("norm.weight")          # outside a step
    red.start_step()
    with pytest.raises(KeyError):
        red.on_grad_ready("nope")
    red.on_grad_ready("norm.weight")
    with pytest.raises(RuntimeError):
        red.on_grad_ready("norm.weight")          # duplicate
    with pytest.raises(RuntimeError):
        red.wait_all()                            # buckets still pending


def test_reducer_norm_over_all_grads_single_rank():
    store, red = _reducer()
    store.flat_grads.normal_()
    for name, off, n in store.entries():          # padding stays zero
        store.flat_grads[off + store.numel(name):off + n] = 0
    red.start_step()
    for ps in store.order:
        red.on_grad_ready(ps.name)
    red.wait_all()
    want = sum(store.grads[p.name].pow(2).sum() for p in store.order)
    assert torch.allclose(red.local_sumsq()[0], want, rtol=1e-5)


def test_reducer_norm_exclusion():
    store, red = _reducer()
    o = store.offsets["norm.weight"]
    red.norm_exclude = [(o, o + store.numel("norm.weight"))]
    store.flat_grads.fill_(0)
    store.grads["norm.weight"].fill_(2.0)
    store.grads["output.weight"].fill_(1.0)
    red.start_step()
    for ps in store.order:
        red.on_grad_ready(ps.name)
    red.wait_all()
    assert float(red.local_sumsq()) == float(store.grads["output.weight"].numel())


# ---------------------------------------------------------------------------------------------
# layout invariants for arbitrary parameter lists (property-based)
# ---------------------------------------------------------------------------------------------
from hypothesis import given, settings, strategies as hst


@settings(max_examples=200, deadline=None, derandomize=True)
@given(world=hst.integers(1, 16), units=hst.lists(hst.integers(1, 40), min_size=1, max_size=30),
       target_units=hst.integers(1, 120))
def test_bucket_layout_invariants(world, units, target_units):
    sizes = [u * world for u in units]               # the store pads every parameter like this
    entries = _entries(sizes)
    target = target_units * world
    buckets = compute_grad_buckets(entries, world, target)
    # buckets tile the flat buffer in order, without holes or overlap
    assert buckets[0].start == 0
    for a, b in zip(buckets, buckets[1:]):
        assert b.start == a.start + a.size and b.index == a.index + 1
    assert buckets[-1].start + buckets[-1].size == sum(sizes)
    # whole parameters, in flat order, each in exactly one bucket
    assert [n for b in buckets for n in b.params] == [e[0] for e in entries]
    for b in buckets:
        assert b.size == sum(b.param_sizes.values()) and b.size % world == 0
        off = 0
        for n in b.params:
            assert b.param_offsets[n] == off
            off += b.param_sizes[n]
        # greedy close: a bucket reaches the target only with its last parameter
        if b is not buckets[-1]:
            assert b.size >= target and b.size - b.param_sizes[b.params[-1]] < target
        # rank shards partition the bucket
        r = [b.shard_range(k, world) for k in range(world)]
        assert r[0][0] == b.start and r[-1][1] == b.start + b.size
        assert all(x[1] == y[0] for x, y in zip(r, r[1:]))
        assert all(hi - lo == b.shard_size(world) for lo, hi in r)


def test_reducer_runs_many_steps_and_resets_its_state():
    store, red = _reducer()
    for step in range(3):
        store.flat_grads.fill_(float(step + 1))
        for name, off, n in store.entries():
            store.flat_grads[off + store.numel(name):off + n] = 0
        red.start_step()
        for ps in reversed(store.order):              # any arrival order is fine
            red.on_grad_ready(ps.name)
        red.wait_all()
        real = sum(store.numel(p.name) for p in store.order)
        assert float(red.local_sumsq()) == pytest.approx(real * (step + 1) ** 2, rel=1e-6)
    red.wait_all()                                    # idempotent outside a step
    with pytest.raises(RuntimeError):
        red.on_grad_ready("norm.weight")


def test_single_rank_reduction_leaves_gradients_untouched():
    store, red = _reducer()
    store.flat_grads.normal_()
    before = store.flat_grads.clone()
    red.start_step()
    for ps in store.order:
        red.on_grad_ready(ps.name)
    red.wait_all()
    assert torch.equal(store.flat_grads, before)
