"""Every CUDA kernel against the host C++ reference ops (``csrc/ref_cpu``) on small shapes."""
import pytest
import torch

pytestmark = pytest.mark.gpu

if torch.cuda.is_available():
    from forgetrain_b200.ops import _lib, attention as A, cuda_ops as K, gemm
from forgetrain_b200.ops import ref_cpu as C
from forgetrain_b200.ops import reference as R


def rel(a, b):
    return ((a.float().cpu() - b.float().cpu()).norm() / b.float().cpu().norm().clamp_min(1e-12)).item()


@pytest.fixture(autouse=True)
def _seed_and_status():
    torch.manual_seed(0)
    yield
    torch.cuda.synchronize()
    _lib.check_status()


def bf(*shape, scale=1.0):
    return (torch.randn(*shape, device="cuda") * scale).to(torch.bfloat16)


@pytest.mark.parametrize("bn", [128, 256])
def test_gemm_against_cpp(bn):
    x, w, dy = bf(384, 192), bf(320, 192, scale=0.05), bf(384, 320)
    assert rel(gemm.linear_fwd(x, w, alpha=0.5, bn=bn), C.linear_fwd(x, w, 0.5)) < 0.01
    assert rel(gemm.linear_dgrad(dy, w, bn=bn), C.linear_dgrad(dy, w)) < 0.01
    assert rel(gemm.linear_wgrad(dy, x, bn=bn), C.linear_wgrad(dy, x)) < 1e-3


def test_fc1_swiglu_epilogue_against_cpp():
    x, w = bf(384, 192), bf(2 * 256, 192, scale=0.08)
    y, act = gemm.linear_swiglu_fwd(x, w)
    cy = C.linear_fwd(x, w, 1.0)
    assert rel(y, cy) < 0.01
    assert rel(act, C.swiglu_fwd(cy)) < 0.02


def test_fc2_dgrad_swiglu_backward_epilogue_against_cpp():
    dy, w2, y1 = bf(384, 192), bf(192, 256, scale=0.08), bf(384, 2 * 256)
    got = gemm.linear_dgrad_swiglu_bwd(dy, w2, y1, alpha=0.5)
    assert rel(got, C.linear_dgrad_swiglu_bwd(dy, w2, y1, 0.5)) < 0.02


def test_embedding_norm_rope_swiglu_against_cpp():
    w = bf(512, 256)
    ids = torch.randint(0, 512, (300,), device="cuda")
    assert rel(K.embedding_fwd(ids, w, 12.0), C.embedding_fwd(ids, w, 12.0)) < 1e-3
    dy = bf(300, 256)
    dw, dwc = torch.zeros(512, 256, device="cuda"), torch.zeros(512, 256)
    K.embedding_bwd(ids, dy, 12.0, dw)
    C.embedding_bwd(ids, dy, 12.0, dwc)
    assert rel(dw, dwc) < 1e-5

    res, x, g = bf(300, 1024), bf(300, 1024), (1 + 0.1 * torch.randn(1024, device="cuda")).to(torch.bfloat16)
    h, y, rs = K.add_rmsnorm_fwd(res, x, g, 1e-6)
    ch, cy, crs = C.add_rmsnorm_fwd(res, x, g, 1e-6)
    assert rel(h, ch) < 1e-3 and rel(y, cy) < 5e-3 and rel(rs, crs) < 1e-4
    dyn, dres = bf(300, 1024), bf(300, 1024)
    gw, gwc = torch.zeros(1024, device="cuda"), torch.zeros(1024)
    dx = K.rmsnorm_bwd(dyn, h, g, rs, dres.clone(), gw, False)
    cdx = C.rmsnorm_bwd(dyn, h, g, rs, dres, gwc, False)
    assert rel(dx, cdx) < 5e-3 and rel(gw, gwc) < 1e-3

    qkv = bf(2 * 256, 2 * 4 * 64)
    cos, sin = R.rope_tables(256, 64, 10000.0, device="cuda")
    want = C.rope_(qkv.clone(), cos, sin, 2, 2, 2, 64)
    assert rel(K.rope_(qkv.clone(), cos, sin, 2, 2, 2, 64), want) < 5e-3

    y1, da = bf(300, 512), bf(300, 256)
    assert rel(K.swiglu_fwd(y1), C.swiglu_fwd(y1)) < 5e-3
    assert rel(K.swiglu_bwd(da, y1), C.swiglu_bwd(da, y1)) < 5e-3


def test_cross_entropy_and_adamw_against_cpp():
    lg = bf(200, 3000, scale=2.0)
    lab = torch.randint(0, 3000, (200,), device="cuda")
    mask = (torch.rand(200, device="cuda") > 0.2).float()
    closs, cd = C.cross_entropy_fwd_bwd(lg, lab, mask, 1.0)
    loss, d = K.cross_entropy_fwd_bwd(lg.clone(), lab, mask, 1.0)
    assert abs(float(loss) - float(closs)) < 1e-3 and rel(d, cd) < 0.01

    n = 5000
    p, g = torch.randn(n, device="cuda"), torch.randn(n, device="cuda")
    m, v = torch.zeros(n, device="cuda"), torch.zeros(n, device="cuda")
    pc, mc, vc = p.clone(), m.clone(), v.clone()
    out, outc = torch.empty(n, device="cuda", dtype=torch.bfloat16), torch.empty(n, dtype=torch.bfloat16)
    hyper = torch.tensor([1e-2, 0.9, 0.95, 1e-8, 1 - 0.9, 1 - 0.95, 0.7, 0], device="cuda")
    K.adamw_flat(p, m, v, g, out, hyper, torch.tensor([n], device="cuda", dtype=torch.int64),
                 torch.tensor([0.1], device="cuda"), torch.tensor([1.0], device="cuda"))
    C.adamw_step(pc, mc, vc, g, outc, 1e-2, 0.9, 0.95, 1e-8, 0.1, 1, clip=0.7)
    assert rel(p, pc) < 1e-5 and rel(v, vc) < 1e-5 and rel(out, outc) < 1e-3


@pytest.mark.parametrize("B,S,G,g,D", [(1, 256, 1, 2, 64), (1, 256, 1, 1, 128)])
def test_attention_against_cpp(B, S, G, g, D):
    qkv = bf(B * S, G * (g + 2) * D)
    o, lse = A.attention_fwd(qkv, B, G, g, D)
    co, clse = C.attention_fwd(qkv, B, G, g, D)
    assert rel(o, co) < 0.01 and rel(lse, clse) < 1e-4
    do = torch.randn_like(o)
    d = A.attention_bwd(do, qkv, o, lse, B, G, g, D)
    cd = C.attention_bwd(do, qkv, co, clse, B, G, g, D)
    assert rel(d, cd) < 0.015
