"""Numerics of every sm_100a kernel against the plain PyTorch fp32 statement of the same op."""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu

if torch.cuda.is_available():
    from forgetrain_b200.ops import _lib, cuda_ops as C, gemm, attention as A
from forgetrain_b200.ops import reference as R


def rel(a, b):
    return float((a.float() - b.float()).abs().max() / (b.float().abs().max() + 1e-9))


@pytest.fixture(autouse=True)
def _seed_and_status():
    torch.manual_seed(0)
    yield
    torch.cuda.synchronize()
    _lib.check_status()


# (1280, 4096, 512): 160 tiles of 128 x 256 = one full wave of 148 CTAs + 12 tiles that the
# scheduler cuts into halves; (16384, 1024, 256): 512 tiles = 3 waves + 68 split tiles;
# (640, 1160, 320): every tile is split and the split meets a partial last column tile
@pytest.mark.parametrize("T,N,K", [(128, 128, 64), (384, 200, 72), (1000, 1280, 1024), (512, 73448, 256),
                                   (4096, 1024, 4096), (1280, 4096, 512), (16384, 1024, 256),
                                   (640, 1160, 320)])
def test_gemm_fwd_dgrad_wgrad(T, N, K):
    x = torch.randn(T, K, device="cuda").to(torch.bfloat16)
    w = (torch.randn(N, K, device="cuda") * 0.05).to(torch.bfloat16)
    dy = torch.randn(T, N, device="cuda").to(torch.bfloat16)
    y = gemm.linear_fwd(x, w)
    assert rel(y, x.float() @ w.float().t()) < 0.01
    y2 = gemm.linear_fwd(x, w, alpha=0.25)
    assert rel(y2, 0.25 * (x.float() @ w.float().t())) < 0.01
    dx = gemm.linear_dgrad(dy, w)
    assert rel(dx, dy.float() @ w.float()) < 0.01
    ref = dy.float().t() @ x.float()
    dw = gemm.linear_wgrad(dy, x)
    assert rel(dw, ref) < 1e-3
    gemm.linear_wgrad(dy, x, out=dw, accumulate=True)
    assert rel(dw, 2 * ref) < 1e-3
    dw1 = gemm.linear_wgrad(dy, x, splitk=1)
    dw4 = gemm.linear_wgrad(dy, x, splitk=min(4, (T + 63) // 64))
    assert rel(dw1, ref) < 1e-3 and rel(dw4, ref) < 1e-3


@pytest.mark.parametrize("bn", [128, 256])
@pytest.mark.parametrize("T,N,K", [(256, 256, 64), (640, 1280, 320), (1000, 1032, 1024), (2048, 4096, 512)])
def test_gemm_tile_shapes(T, N, K, bn):
    """Both single-CTA tile shapes (128 x 128, 128 x 256) against fp32 matmul, for all three operand-major combinations and the reduce-add epilogue."""
    x = torch.randn(T, K, device="cuda").to(torch.bfloat16)
    w = (torch.randn(N, K, device="cuda") * 0.05).to(torch.bfloat16)
    dy = torch.randn(T, N, device="cuda").to(torch.bfloat16)
    assert rel(gemm.linear_fwd(x, w, bn=bn), x.float() @ w.float().t()) < 0.01
    assert rel(gemm.linear_dgrad(dy, w, bn=bn), dy.float() @ w.float()) < 0.01
    ref = dy.float().t() @ x.float()
    dw = gemm.linear_wgrad(dy, x, bn=bn)
    assert rel(dw, ref) < 1e-3
    gemm.linear_wgrad(dy, x, out=dw, accumulate=True, bn=bn, splitk=3)
    assert rel(dw, 2 * ref) < 1e-3


@pytest.mark.parametrize("T,F,K", [(128, 128, 64), (300, 256, 200), (1000, 1024, 256), (4096, 4096, 1024)])
def test_fc1_with_swiglu_in_the_epilogue(T, F, K):
    """One kernel writes y = x w^T and act = silu(gate) * up; both must be BITWISE what the plain
    GEMM followed by the SwiGLU kernel give, and close to the fp32 statement."""
    x = torch.randn(T, K, device="cuda").to(torch.bfloat16)
    w = (torch.randn(2 * F, K, device="cuda") * 0.08).to(torch.bfloat16)
    y, act = gemm.linear_swiglu_fwd(x, w)
    y_ref = gemm.linear_fwd(x, w)
    act_ref = C.swiglu_fwd(y_ref)
    assert torch.equal(y, y_ref)
    assert torch.equal(act, act_ref)
    yf = x.float() @ w.float().t()
    assert rel(y, yf) < 0.01
    assert rel(act, torch.nn.functional.silu(yf[:, :F]) * yf[:, F:]) < 0.02
    y2, act2 = gemm.linear_swiglu_fwd(x, w, alpha=0.5)
    assert torch.equal(y2, gemm.linear_fwd(x, w, alpha=0.5))
    assert torch.equal(act2, C.swiglu_fwd(y2))
    # a width that is not a multiple of 128 takes the two-kernel route through the same front end
    w3 = w[: 2 * 64].contiguous()
    y3, act3 = C.linear_swiglu_fwd(x, w3)
    assert torch.equal(act3, C.swiglu_fwd(gemm.linear_fwd(x, w3)))


@pytest.mark.parametrize("T,F,H", [(128, 64, 64), (300, 192, 200), (1000, 1024, 256), (4096, 4096, 1024)])
def test_fc2_dgrad_with_swiglu_backward_in_the_epilogue(T, F, H):
    """One kernel computes d act = dy w2 in its accumulator and writes (d gate, d up); BITWISE what
    the plain dgrad GEMM followed by the SwiGLU backward kernel give, and close to fp32. The last
    shape has a half-full last wave, so the 128 x 128 half tiles run too."""
    dy = torch.randn(T, H, device="cuda").to(torch.bfloat16)
    w2 = (torch.randn(H, F, device="cuda") * 0.08).to(torch.bfloat16)
    y1 = torch.randn(T, 2 * F, device="cuda").to(torch.bfloat16)
    for alpha in (1.0, 0.5):
        got = gemm.linear_dgrad_swiglu_bwd(dy, w2, y1, alpha=alpha)
        ref = C.swiglu_bwd(gemm.linear_dgrad(dy, w2, alpha=alpha), y1)
        assert torch.equal(got, ref)
    yf = y1.float()
    da = dy.float() @ w2.float()
    sig = torch.sigmoid(yf[:, :F])
    ref32 = torch.cat([da * sig * (1 + yf[:, :F] * (1 - sig)) * yf[:, F:], da * yf[:, :F] * sig], dim=1)
    assert rel(gemm.linear_dgrad_swiglu_bwd(dy, w2, y1), ref32) < 0.02
    # a width that is not a multiple of 64 takes the two-kernel route through the same front end
    w3, y3 = w2[:, :40].contiguous(), y1[:, :80].contiguous()
    assert torch.equal(C.linear_dgrad_swiglu_bwd(dy, w3, y3), C.swiglu_bwd(gemm.linear_dgrad(dy, w3), y3))


def test_gemm_strided_views():
    """Operands that are column slices of a wider buffer (row pitch != width)."""
    big = torch.randn(512, 3 * 256, device="cuda").to(torch.bfloat16)
    x = big[:, 256:512]
    w = (torch.randn(384, 256, device="cuda") * 0.05).to(torch.bfloat16)
    assert rel(gemm.linear_fwd(x, w), x.float() @ w.float().t()) < 0.01


@pytest.mark.parametrize("B,S,G,g,D", [(1, 256, 1, 1, 64), (2, 512, 2, 2, 64), (1, 1024, 2, 8, 64),
                                        (1, 512, 1, 2, 128), (2, 768, 2, 4, 128),
                                        (1, 4096, 1, 2, 64), (1, 4096, 1, 1, 128)])
def test_flash_attention_fwd_bwd(B, S, G, g, D):
    qkv = torch.randn(B * S, G * (g + 2) * D, device="cuda").to(torch.bfloat16)
    o, lse = A.attention_fwd(qkv, B, G, g, D)
    ro, rlse = R.attention_fwd(qkv, B, G, g, D)
    assert rel(o, ro) < 0.01 and rel(lse, rlse) < 1e-4
    do = torch.randn_like(o)
    rd = R.attention_bwd(do, qkv, ro, rlse, B, G, g, D).view(B * S, G, g + 2, D)
    for hpc in ([0, 1] if g > 1 else [0]):
        d = A.attention_bwd(do, qkv, o, lse, B, G, g, D, heads_per_cta=hpc).view(B * S, G, g + 2, D)
        assert rel(d[:, :, :g], rd[:, :, :g]) < 0.015
        assert rel(d[:, :, g], rd[:, :, g]) < 0.015
        assert rel(d[:, :, g + 1], rd[:, :, g + 1]) < 0.015


def test_attention_rejects_unsupported_shapes():
    qkv = torch.randn(200, 4 * 64, device="cuda").to(torch.bfloat16)
    with pytest.raises(ValueError):
        A.attention_fwd(qkv, 1, 1, 2, 64)          # 200 is not a multiple of 256


@pytest.mark.parametrize("T,H", [(512, 256), (1024, 1024), (777, 1024), (512, 4096), (300, 2048)])
def test_rmsnorm_fwd_bwd(T, H):
    x = torch.randn(T, H, device="cuda").to(torch.bfloat16)
    res = torch.randn(T, H, device="cuda").to(torch.bfloat16)
    w = (1 + 0.1 * torch.randn(H, device="cuda")).to(torch.bfloat16)
    h, y, rs = C.add_rmsnorm_fwd(res, x, w, 1e-6)
    rh, ry, rrs = R.add_rmsnorm_fwd(res, x, w, 1e-6)
    assert torch.equal(h, rh) and rel(y, ry) < 0.01 and rel(rs, rrs) < 1e-5
    _, y2, _ = C.add_rmsnorm_fwd(None, x, w, 1e-6)
    assert rel(y2, R.add_rmsnorm_fwd(None, x, w, 1e-6)[1]) < 0.01
    dy = torch.randn(T, H, device="cuda").to(torch.bfloat16)
    dres = torch.randn(T, H, device="cuda").to(torch.bfloat16)
    dw, rdw = torch.zeros(H, device="cuda"), torch.zeros(H, device="cuda")
    rdx = R.rmsnorm_bwd(dy, rh, w, rrs, dres.clone(), rdw, False)
    dx = C.rmsnorm_bwd(dy, rh, w, rrs, dres.clone(), dw, False)
    assert rel(dx, rdx) < 0.01 and rel(dw, rdw) < 1e-4
    C.rmsnorm_bwd(dy, rh, w, rrs, None, dw, True)
    assert rel(dw, 2 * rdw) < 1e-4


@pytest.mark.parametrize("B,S,G,g,D", [(2, 256, 2, 2, 64), (1, 512, 2, 8, 64), (2, 256, 1, 4, 128)])
def test_rope(B, S, G, g, D):
    qkv = torch.randn(B * S, G * (g + 2) * D, device="cuda").to(torch.bfloat16)
    cos, sin = R.rope_tables(S, D, 10000.0, device="cuda")
    a = C.rope_(qkv.clone(), cos, sin, B, G, g, D)
    b = R.rope_(qkv.clone(), cos, sin, B, G, g, D)
    assert rel(a, b) < 0.01
    back = C.rope_(a.clone(), cos, sin, B, G, g, D, inverse=True)
    assert rel(back, qkv) < 0.02
    pid = torch.randint(0, S, (B * S,), device="cuda")
    assert rel(C.rope_(qkv.clone(), cos, sin, B, G, g, D, position_ids=pid),
               R.rope_(qkv.clone(), cos, sin, B, G, g, D, position_ids=pid)) < 0.01


def test_swiglu():
    y1 = torch.randn(1000, 2 * 1024, device="cuda").to(torch.bfloat16)
    da = torch.randn(1000, 1024, device="cuda").to(torch.bfloat16)
    assert rel(C.swiglu_fwd(y1), R.swiglu_fwd(y1)) < 0.01
    assert rel(C.swiglu_bwd(da, y1), R.swiglu_bwd(da, y1)) < 0.01


def test_embedding():
    ids = torch.randint(0, 5000, (2048,), device="cuda")
    w = torch.randn(5000, 256, device="cuda").to(torch.bfloat16)
    assert rel(C.embedding_fwd(ids, w, 12.0), R.embedding_fwd(ids, w, 12.0)) < 1e-6
    dy = torch.randn(2048, 256, device="cuda").to(torch.bfloat16)
    dw, rdw = torch.zeros(5000, 256, device="cuda"), torch.zeros(5000, 256, device="cuda")
    C.embedding_bwd(ids, dy, 12.0, dw)
    R.embedding_bwd(ids, dy, 12.0, rdw)
    assert rel(dw, rdw) < 1e-5
    # vocab-parallel: only the local range contributes
    dw2 = torch.zeros(1000, 256, device="cuda")
    C.embedding_bwd(ids, dy, 1.0, dw2, vocab_start=2000)
    r2 = torch.zeros(1000, 256, device="cuda")
    R.embedding_bwd(ids, dy, 1.0, r2, vocab_start=2000)
    assert rel(dw2, r2) < 1e-5
    e = C.embedding_fwd(ids, w[2000:3000].contiguous(), 2.0, vocab_start=2000)
    outside = (ids < 2000) | (ids >= 3000)
    assert float(e[outside].abs().max()) == 0.0


@pytest.mark.parametrize("T,V", [(256, 4096), (300, 73448), (100, 8008)])
def test_cross_entropy(T, V):
    lg = (torch.randn(T, V, device="cuda") * 2).to(torch.bfloat16)
    lab = torch.randint(0, V, (T,), device="cuda")
    mask = (torch.rand(T, device="cuda") > 0.2).float()
    rl, rd = R.cross_entropy_fwd_bwd(lg.clone(), lab, mask, 0.5)
    l, d = C.cross_entropy_fwd_bwd(lg.clone(), lab, mask, 0.5)
    assert abs(float(l) - float(rl)) / abs(float(rl)) < 1e-4
    assert rel(d, rd) < 0.01


def test_vocab_parallel_cross_entropy_two_shards_on_one_device():
    """The three-phase form with the statistics of two vocabulary shards combined by hand."""
    T, V = 128, 4096
    lg = (torch.randn(T, V, device="cuda") * 2).to(torch.bfloat16)
    lab = torch.randint(0, V, (T,), device="cuda")
    rl, rd = R.cross_entropy_fwd_bwd(lg.clone(), lab, None, 1.0)
    half = V // 2
    shards = [lg[:, :half].contiguous(), lg[:, half:].contiguous()]
    # phase 1 on both shards through the reference's reducer protocol
    stats = []
    for i, sh in enumerate(shards):
        m = sh.float().max(dim=-1).values
        stats.append(m)
    gmax = torch.maximum(stats[0], stats[1])

    def make_reduce(i):
        other = shards[1 - i].float()
        lab_o = lab - (1 - i) * half

        def red(x, op):
            if op == "max":
                return gmax.clone()
            se_o = torch.exp(other - gmax[:, None]).sum(-1)
            ok = (lab_o >= 0) & (lab_o < half)
            tg_o = torch.where(ok, other.gather(1, lab_o.clamp(0, half - 1)[:, None])[:, 0],
                               torch.zeros_like(gmax))
            return x + torch.stack([se_o, tg_o])
        return red
    outs = []
    for i, sh in enumerate(shards):
        l, d = C.cross_entropy_fwd_bwd(sh.clone(), lab, None, 1.0, vocab_start=i * half,
                                       stats_reduce=make_reduce(i))
        outs.append(d)
        assert abs(float(l) - float(rl)) / abs(float(rl)) < 1e-4
    assert rel(torch.cat(outs, dim=1), rd) < 0.01


def test_adamw_segments_and_sumsq():
    n = 4096 * 33
    p32 = torch.randn(n, device="cuda")
    m, v = torch.zeros(n, device="cuda"), torch.zeros(n, device="cuda")
    g = torch.randn(n, device="cuda")
    pb = torch.empty(n, device="cuda", dtype=torch.bfloat16)
    rp, rm, rv, rpb = p32.clone(), m.clone(), v.clone(), pb.clone()
    hyper = torch.tensor([1e-2, 0.9, 0.95, 1e-8, 1 - 0.9, 1 - 0.95, 0.7, 0], device="cuda")
    se = torch.tensor([4000, n], device="cuda", dtype=torch.int64)
    sw = torch.tensor([0.0, 0.1], device="cuda")
    sl = torch.tensor([1.0, 0.25], device="cuda")
    C.adamw_flat(p32, m, v, g, pb, hyper, se, sw, sl)
    R.adamw_step(rp[:4000], rm[:4000], rv[:4000], g[:4000], rpb[:4000], 1e-2, 0.9, 0.95, 1e-8, 0.0, 1, 0.7)
    R.adamw_step(rp[4000:], rm[4000:], rv[4000:], g[4000:], rpb[4000:], 2.5e-3, 0.9, 0.95, 1e-8, 0.1, 1, 0.7)
    assert rel(p32, rp) < 1e-6 and rel(m, rm) < 1e-6 and rel(v, rv) < 1e-6 and torch.equal(pb, rpb)
    ss = torch.zeros(1, device="cuda")
    C.sumsq_into(g, ss)
    assert abs(float(ss) - float(g.pow(2).sum())) / float(g.pow(2).sum()) < 1e-5
    nrm = torch.zeros(1, device="cuda")
    C.clip_coef(ss, 1.0, hyper, nrm)
    assert float(hyper[6]) == pytest.approx(1.0 / (float(nrm) + 1e-6), rel=1e-5)


def test_native_library_is_the_cuda_path():
    """CUDA tensors never fall back to PyTorch: the op layer routes to the native library."""
    from forgetrain_b200 import ops
    before = _lib.launch_count()
    x = torch.randn(256, 256, device="cuda").to(torch.bfloat16)
    w = torch.randn(256, 256, device="cuda").to(torch.bfloat16)
    ops.linear_fwd(x, w)
    ops.swiglu_fwd(x)
    assert _lib.launch_count() == before + 2


def test_device_side_schedule_matches_host_schedule():
    """The one-thread schedule kernel (step counter, warmup - stable - decay learning rate, bias
    corrections) against the host formulas, across every region of the schedule."""
    from forgetrain_b200.optim.lr import compute_lr
    max_lr, min_lr, warm, decay, wsd = 3e-3, 1e-4, 5, 40, 12
    b1, b2, eps = 0.9, 0.95, 1e-8
    sched = torch.tensor([max_lr, min_lr, warm, decay, wsd, b1, b2, eps], device="cuda")
    step = torch.zeros(1, dtype=torch.int32, device="cuda")
    hyper = torch.zeros(8, device="cuda")
    hyper[6] = 0.5                                   # the clip slot belongs to another kernel
    for it in range(50):
        C.adam_hyper_step(step, sched, hyper)
        h = hyper.cpu().double()
        t = it + 1
        assert int(step) == t
        assert h[0] == pytest.approx(compute_lr(it, max_lr, min_lr, warm, decay, wsd), rel=1e-6, abs=1e-12)
        assert h[1] == pytest.approx(b1, rel=1e-7) and h[2] == pytest.approx(b2, rel=1e-7)
        assert h[4] == pytest.approx(1 - b1 ** t, rel=1e-5) and h[5] == pytest.approx(1 - b2 ** t, rel=1e-5)
        assert h[6] == 0.5
    # warmup-then-constant (the 8B engine's schedule): wsd == 0
    sched[4] = 0
    step.zero_()
    for it in range(8):
        C.adam_hyper_step(step, sched, hyper)
        assert float(hyper[0]) == pytest.approx(compute_lr(it, max_lr, min_lr, warm, decay, 0), rel=1e-6)


@pytest.mark.parametrize("B,S,G,g,D", [(2, 512, 2, 2, 64), (1, 512, 1, 2, 128)])
def test_attention_backward_with_the_rope_backward_fused(B, S, G, g, D):
    """The last kernel of the attention backward can apply the transposed rotation to the q / k
    gradients; same result as the stand-alone RoPE kernel run on the unfused output (up to the
    one bf16 rounding the fusion saves), with and without explicit position ids."""
    from forgetrain_b200 import ops
    qkv = torch.randn(B * S, G * (g + 2) * D, device="cuda").to(torch.bfloat16)
    o, lse = A.attention_fwd(qkv, B, G, g, D)
    do = torch.randn_like(o)
    cos, sin = ops.rope_tables(S, D, 10000.0, device="cuda")
    pos = torch.randint(0, S, (B, S), device="cuda")
    for p in (None, pos):
        plain = A.attention_bwd(do, qkv, o, lse, B, G, g, D)
        want = ops.rope_(plain.clone(), cos, sin, B, G, g, D, inverse=True, position_ids=p)
        got = A.attention_bwd(do, qkv, o, lse, B, G, g, D, rope=(cos, sin, p))
        assert rel(got, want) < 0.01
        v = got.view(B * S, G, g + 2, D)[:, :, g + 1]
        assert torch.equal(v, plain.view(B * S, G, g + 2, D)[:, :, g + 1])   # v is not rotated
