"""The host C++ reference ops against the PyTorch oracle (two independent statements of the
same math), in fp32 and with bf16 storage rounding."""
import math

import pytest
import torch

from forgetrain_b200.ops import ref_cpu as C
from forgetrain_b200.ops import reference as R


def rel(a, b):
    return ((a.float() - b.float()).norm() / b.float().norm().clamp_min(1e-12)).item()


@pytest.fixture(autouse=True)
def _seed():
    torch.manual_seed(0)


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 1e-5), (torch.bfloat16, 6e-3)])
def test_linear_three_ways(dtype, tol):
    x = torch.randn(48, 40).to(dtype)
    w = (torch.randn(24, 40) * 0.1).to(dtype)
    dy = torch.randn(48, 24).to(dtype)
    assert rel(C.linear_fwd(x, w, 0.5), R.linear_fwd(x, w, 0.5)) < tol
    assert rel(C.linear_dgrad(dy, w), R.linear_dgrad(dy, w)) < tol
    ref = R.linear_wgrad(dy, x, torch.zeros(24, 40), False)
    assert rel(C.linear_wgrad(dy, x), ref) < 1e-5
    acc = ref.clone()
    assert rel(C.linear_wgrad(dy, x, out=acc, accumulate=True), 2 * ref) < 1e-5


def test_embedding_fwd_bwd_with_vocab_shard():
    w = torch.randn(32, 16)
    ids = torch.randint(0, 64, (3, 7))
    inside = (ids >= 16) & (ids < 48)
    got = C.embedding_fwd(ids, w, 12.0, vocab_start=16)
    want = torch.where(inside.reshape(-1, 1), w[(ids.reshape(-1) - 16).clamp(0, 31)] * 12.0,
                       torch.zeros(1))
    assert rel(got, want) < 1e-6
    dy = torch.randn(21, 16)
    a, b = torch.zeros(32, 16), torch.zeros(32, 16)
    C.embedding_bwd(ids, dy, 12.0, a, vocab_start=16)
    R.embedding_bwd(ids, dy, 12.0, b, vocab_start=16)
    assert rel(a, b) < 1e-6


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 1e-5), (torch.bfloat16, 8e-3)])
def test_rmsnorm_fwd_bwd(dtype, tol):
    res, x = torch.randn(33, 64).to(dtype), torch.randn(33, 64).to(dtype)
    w = (1 + 0.1 * torch.randn(64)).to(dtype)
    h, y, rs = C.add_rmsnorm_fwd(res, x, w, 1e-6)
    rh, ry, rrs = R.add_rmsnorm_fwd(res, x, w, 1e-6)
    assert rel(h, rh) < tol and rel(y, ry) < tol and rel(rs, rrs) < 1e-5
    _, y2, _ = C.add_rmsnorm_fwd(None, x, w, 1e-6)
    assert rel(y2, R.add_rmsnorm_fwd(None, x, w, 1e-6)[1]) < tol
    dy, dres = torch.randn(33, 64).to(dtype), torch.randn(33, 64).to(dtype)
    dwa, dwb = torch.ones(64), torch.ones(64)
    dx = C.rmsnorm_bwd(dy, rh, w, rrs, dres, dwa, True)
    rdx = R.rmsnorm_bwd(dy, rh, w, rrs, dres, dwb, True)
    assert rel(dx, rdx) < tol and rel(dwa, dwb) < 1e-5


def test_rope_forward_inverse_and_positions():
    B, S, G, g, D = 2, 8, 2, 3, 16
    qkv = torch.randn(B * S, G * (g + 2) * D)
    cos, sin = R.rope_tables(32, D, 10000.0)
    a = C.rope_(qkv.clone(), cos, sin, B, G, g, D)
    b = R.rope_(qkv.clone(), cos, sin, B, G, g, D)
    assert rel(a, b) < 1e-6
    assert rel(C.rope_(a.clone(), cos, sin, B, G, g, D, inverse=True), qkv) < 1e-5
    pos = torch.randint(0, 32, (B * S,))
    assert rel(C.rope_(qkv.clone(), cos, sin, B, G, g, D, position_ids=pos),
               R.rope_(qkv.clone(), cos, sin, B, G, g, D, position_ids=pos)) < 1e-6


def test_swiglu_fwd_bwd():
    y1, da = torch.randn(9, 64), torch.randn(9, 32)
    assert rel(C.swiglu_fwd(y1), R.swiglu_fwd(y1)) < 1e-6
    assert rel(C.swiglu_bwd(da, y1), R.swiglu_bwd(da, y1)) < 1e-6


def test_cross_entropy_masked_and_sharded():
    lg = torch.randn(17, 50) * 3
    lab = torch.randint(0, 50, (17,))
    mask = (torch.rand(17) > 0.3).float()
    la, da = C.cross_entropy_fwd_bwd(lg, lab, mask, 0.5)
    lb, db = R.cross_entropy_fwd_bwd(lg, lab, mask, 0.5)
    assert abs(float(la) - float(lb)) < 1e-5 and rel(da, db) < 1e-5
    # loss against the textbook formula
    want = (torch.nn.functional.cross_entropy(lg, lab, reduction="none") * mask).sum() / mask.sum()
    assert abs(float(la) - float(want)) < 1e-5


@pytest.mark.parametrize("B,S,G,g,D", [(1, 24, 1, 1, 16), (2, 33, 2, 3, 8)])
def test_attention_fwd_bwd(B, S, G, g, D):
    qkv = torch.randn(B * S, G * (g + 2) * D)
    o, lse = C.attention_fwd(qkv, B, G, g, D)
    ro, rlse = R.attention_fwd(qkv, B, G, g, D)
    assert rel(o, ro) < 1e-5 and rel(lse, rlse) < 1e-5
    do = torch.randn_like(ro)
    assert rel(C.attention_bwd(do, qkv, ro, rlse, B, G, g, D),
               R.attention_bwd(do, qkv, ro, rlse, B, G, g, D)) < 1e-5


def test_adamw_and_sumsq():
    p, g = torch.randn(1000), torch.randn(1000)
    pa, ma, va = p.clone(), torch.zeros(1000), torch.zeros(1000)
    pb, mb, vb = p.clone(), torch.zeros(1000), torch.zeros(1000)
    oa, ob = torch.empty(1000, dtype=torch.bfloat16), torch.empty(1000, dtype=torch.bfloat16)
    for t in (1, 2, 3):
        C.adamw_step(pa, ma, va, g, oa, 1e-2, 0.9, 0.95, 1e-8, 0.1, t, clip=0.7)
        R.adamw_step(pb, mb, vb, g, ob, 1e-2, 0.9, 0.95, 1e-8, 0.1, t, clip=0.7)
    assert rel(pa, pb) < 1e-6 and rel(va, vb) < 1e-6 and rel(oa, ob) < 1e-3
    assert math.isclose(float(C.sumsq(g)), float(R.sumsq(g)), rel_tol=1e-5)


def test_fused_fc1_swiglu_reference_equals_the_two_op_composition():
    """The one-pass C++ statement of the fused FC1 epilogue gives bitwise what GEMM followed by
    SwiGLU gives (the activation is computed from the rounded FC1 output in both)."""
    torch.manual_seed(0)
    x = torch.randn(37, 48).to(torch.bfloat16)
    w = (torch.randn(2 * 24, 48) * 0.2).to(torch.bfloat16)
    y, act = C.linear_swiglu_fwd(x, w, 0.5)
    y2 = C.linear_fwd(x, w, 0.5)
    assert torch.equal(y, y2) and torch.equal(act, C.swiglu_fwd(y2))
    ry, ract = R.linear_swiglu_fwd(x, w, 0.5)
    assert rel(y, ry) < 1e-2 and rel(act, ract) < 2e-2
    yf, actf = C.linear_swiglu_fwd(x.float(), w.float())          # fp32 storage: no rounding
    assert rel(actf, torch.nn.functional.silu(yf[:, :24]) * yf[:, 24:]) < 1e-6


def test_fused_fc2_dgrad_swiglu_backward_reference_equals_the_two_op_composition():
    """The one-pass C++ statement of the fused FC2-dgrad epilogue gives bitwise what the dgrad GEMM
    followed by the SwiGLU backward gives (d act is rounded to the storage type in both)."""
    torch.manual_seed(0)
    dy = torch.randn(37, 48).to(torch.bfloat16)
    w2 = (torch.randn(48, 24) * 0.2).to(torch.bfloat16)
    y1 = torch.randn(37, 2 * 24).to(torch.bfloat16)
    got = C.linear_dgrad_swiglu_bwd(dy, w2, y1, 0.5)
    assert torch.equal(got, C.swiglu_bwd(C.linear_dgrad(dy, w2, 0.5), y1))
    assert rel(got, R.linear_dgrad_swiglu_bwd(dy, w2, y1, 0.5)) < 2e-2
    gf = C.linear_dgrad_swiglu_bwd(dy.float(), w2.float(), y1.float())      # fp32 storage
    da = dy.float() @ w2.float()
    g, u = y1.float()[:, :24], y1.float()[:, 24:]
    sig = torch.sigmoid(g)
    assert rel(gf, torch.cat([da * sig * (1 + g * (1 - sig)) * u, da * g * sig], dim=1)) < 1e-5


# ---------------------------------------------------------------------------------------------
# random shapes: the two statements agree wherever the kernels may be asked to run
# ---------------------------------------------------------------------------------------------
def test_attention_cross_entropy_and_gemm_agree_on_random_geometries():
    from hypothesis import given, settings, strategies as hst

    @settings(max_examples=25, deadline=None, derandomize=True)
    @given(batch=hst.integers(1, 3), seq=hst.integers(1, 40), groups=hst.integers(1, 3),
           per_group=hst.integers(1, 4), half_dim=hst.integers(1, 6), seed=hst.integers(0, 1000))
    def attention(batch, seq, groups, per_group, half_dim, seed):
        D = 2 * half_dim
        g = torch.Generator().manual_seed(seed)
        qkv = torch.randn(batch * seq, groups * (per_group + 2) * D, generator=g)
        out_c, lse_c = C.attention_fwd(qkv, batch, groups, per_group, D)
        out_r, lse_r = R.attention_fwd(qkv, batch, groups, per_group, D)
        assert rel(out_c, out_r) < 2e-5 and rel(lse_c, lse_r) < 2e-5
        dout = torch.randn(out_r.shape, generator=g)
        d_c = C.attention_bwd(dout, qkv, out_r, lse_r, batch, groups, per_group, D)
        d_r = R.attention_bwd(dout, qkv, out_r, lse_r, batch, groups, per_group, D)
        assert rel(d_c, d_r) < 5e-5

    @settings(max_examples=40, deadline=None, derandomize=True)
    @given(rows=hst.integers(1, 30), vocab=hst.integers(2, 90), start=hst.integers(0, 40),
           masked=hst.floats(0.0, 0.9), scale=hst.sampled_from([1.0, 0.25]), seed=hst.integers(0, 1000))
    def cross_entropy(rows, vocab, start, masked, scale, seed):
        g = torch.Generator().manual_seed(seed)
        logits = 3 * torch.randn(rows, vocab, generator=g)
        labels = torch.randint(0, vocab + 2 * start + 1, (rows,), generator=g)   # also outside the shard
        mask = (torch.rand(rows, generator=g) >= masked).float()
        lc, dc = C.cross_entropy_fwd_bwd(logits.clone(), labels, mask, scale, vocab_start=start)
        lr_, dr = R.cross_entropy_fwd_bwd(logits.clone(), labels, mask, scale, vocab_start=start)
        assert float(lc) == pytest.approx(float(lr_), rel=2e-5, abs=2e-6)
        assert (dc.float() - dr.float()).abs().max() < 2e-6

    @settings(max_examples=40, deadline=None, derandomize=True)
    @given(M=hst.integers(1, 50), N=hst.integers(1, 50), K=hst.integers(1, 70), alpha=hst.sampled_from([1.0, 0.7]),
           seed=hst.integers(0, 1000))
    def gemm(M, N, K, alpha, seed):
        g = torch.Generator().manual_seed(seed)
        x, w, dy = torch.randn(M, K, generator=g), torch.randn(N, K, generator=g), torch.randn(M, N, generator=g)
        # sums with cancellation: the error is bounded against the sum of the magnitudes, not
        # against a result that may be close to zero
        def close(got, want, bound):
            assert float((got.float() - want.float()).abs().max()) <= 1e-5 * float(bound.max()) + 1e-7

        close(C.linear_fwd(x, w, alpha), R.linear_fwd(x, w, alpha), x.abs() @ w.abs().t())
        close(C.linear_dgrad(dy, w, alpha), R.linear_dgrad(dy, w, alpha), dy.abs() @ w.abs())
        close(C.linear_wgrad(dy, x), R.linear_wgrad(dy, x, torch.zeros(N, K), False), dy.abs().t() @ x.abs())

    attention()
    cross_entropy()
    gemm()
