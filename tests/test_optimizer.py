import math

import pytest
import torch

from forgetrain_b200.config import load_model_spec
from forgetrain_b200.models.params import ParamStore
from forgetrain_b200.optim.adamw import ShardedAdamW
from forgetrain_b200.optim.lr import compute_lr
from forgetrain_b200.ops import reference as R
from forgetrain_b200.parallel.buckets import compute_grad_buckets


def test_wsd_schedule_shape():
    kw = dict(max_lr=1e-2, min_lr=1e-4, warmup_iters=10, lr_decay_iters=100, wsd_decay_iters=20)
    assert compute_lr(0, **kw) == 0.0
    assert math.isclose(compute_lr(5, **kw), 5e-3)
    assert compute_lr(10, **kw) == 1e-2 and compute_lr(80, **kw) == 1e-2
    mid = compute_lr(90, **kw)   # half of the decay window: min + (2*0.5^0.5 - 1)(max-min)
    assert math.isclose(mid, 1e-4 + (2 * 0.5 ** 0.5 - 1) * (1e-2 - 1e-4))
    assert math.isclose(compute_lr(100, **kw), 1e-4, rel_tol=1e-9)
    assert compute_lr(101, **kw) == 1e-4
    # warmup then constant (8B engine)
    assert compute_lr(50, 2e-4, 0.0, 10, 1000, 0) == 2e-4


def test_adamw_reference_matches_torch():
    torch.manual_seed(0)
    p = torch.randn(1000)
    g = [torch.randn(1000) for _ in range(5)]
    ref = p.clone().requires_grad_(True)
    opt = torch.optim.AdamW([ref], lr=1e-2, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1)
    m, v = torch.zeros(1000), torch.zeros(1000)
    for t, gi in enumerate(g, start=1):
        ref.grad = gi.clone()
        opt.step()
        R.adamw_step(p, m, v, gi, None, 1e-2, 0.9, 0.95, 1e-8, 0.1, t)
    assert torch.allclose(p, ref.detach(), atol=1e-6)


def _store():
    spec = load_model_spec("tiny", num_layers=2, vocab_size=256, hidden_size=128, ffn_hidden_size=256,
                           num_attention_heads=4, num_query_groups=2, head_dim=32, tie_embeddings=False)
    return spec, ParamStore(spec, "cpu", torch.float32, pad_to=128 * 4, align=128 * 4)


def test_sharded_step_equals_full_step_across_simulated_ranks():
    """Four simulated DP ranks, each updating only its shard, reproduce the unsharded update."""
    spec, store0 = _store()
    store0.init_random(0)
    torch.manual_seed(3)
    grads = torch.randn(store0.total)
    # unsharded reference
    buckets1 = compute_grad_buckets(store0.entries(), 1, 50_000)
    store0.flat_grads.copy_(grads)
    full = ShardedAdamW(store0, buckets1, 1, 0, None)
    full.hyper[6] = 1.0
    full.step(1e-2)
    want = store0.flat_params.clone()
    got = torch.zeros_like(want)
    for rank in range(4):
        _, st = _store()
        st.init_random(0)
        st.flat_grads.copy_(grads)
        b = compute_grad_buckets(st.entries(), 4, 50_000)
        opt = ShardedAdamW(st, b, 4, rank, None)
        opt.world = 4
        opt.hyper[6] = 1.0
        opt._all_gather_bucket = lambda i, bk: None   # no process group in this test
        opt.step(1e-2)
        for bk in b:
            lo, hi = bk.shard_range(rank, 4)
            got[lo:hi] = st.flat_params[lo:hi]
    assert torch.allclose(got, want, atol=1e-7)


def test_weight_decay_and_mup_lr_classes():
    spec, store = _store()
    store.init_random(0)
    b = compute_grad_buckets(store.entries(), 1, 10 ** 9)
    opt = ShardedAdamW(store, b, 1, 0, None, weight_decay=0.1)
    segs = {name: (wd, lrm) for (_, wd, lrm, name) in opt.segments[0]}
    assert segs["norm.weight"] == (0.0, 1.0)
    assert segs["tok_embeddings.weight"] == (0.1, 1.0)
    wd, lrm = segs["layers.0.attention.wqkv.weight"]
    assert wd == 0.1 and math.isclose(lrm, 1.0 / spec.mup_width_scale)


def test_clip_coefficient():
    spec, store = _store()
    store.init_random(0)
    b = compute_grad_buckets(store.entries(), 1, 10 ** 9)
    opt = ShardedAdamW(store, b, 1, 0, None, max_grad_norm=1.0)
    opt.compute_clip(torch.tensor([16.0]))
    assert math.isclose(float(opt.grad_norm), 4.0)
    assert math.isclose(float(opt.hyper[6]), 1.0 / (4.0 + 1e-6), rel_tol=1e-6)
    opt.compute_clip(torch.tensor([0.25]))
    assert float(opt.hyper[6]) == 1.0


def test_optimizer_state_roundtrip():
    spec, store = _store()
    store.init_random(0)
    b = compute_grad_buckets(store.entries(), 1, 50_000)
    opt = ShardedAdamW(store, b, 1, 0, None)
    store.flat_grads.normal_()
    opt.hyper[6] = 1.0
    opt.step(1e-3)
    state = opt.gather_full_state()
    assert set(state) == {"master_weights", "exp_avg", "exp_avg_sq"}
    assert state["exp_avg"]["norm.weight"].shape == (spec.hidden_size,)
    spec2, store2 = _store()
    store2.init_random(1)
    opt2 = ShardedAdamW(store2, compute_grad_buckets(store2.entries(), 1, 50_000), 1, 0, None)
    opt2.load_full_state(state, 1)
    assert opt2.step_count == 1
    for name in state["exp_avg"]:
        st2 = opt2.gather_full_state()
        assert torch.equal(st2["exp_avg_sq"][name], state["exp_avg_sq"][name])
        break
