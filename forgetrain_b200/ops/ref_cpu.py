"""ctypes front end of the host C++ reference ops (``csrc/ref_cpu/ref_ops.cpp``).

Same signatures as :mod:`forgetrain_b200.ops.reference` for the ops it covers; inputs may live
on any device and in any dtype, the math runs on the host in fp32 / fp64 and the results come
back on the input's device in the storage dtype (rounded to bf16 inside the C++ code at the
points where the device kernels round). The library is built on first use with g++.
"""
from __future__ import annotations

import ctypes
import math

import torch

_LIB = None
c_int, c_float, c_long = ctypes.c_int, ctypes.c_float, ctypes.c_int64


def lib():
    global _LIB
    if _LIB is None:
        from .. import build
        L = ctypes.CDLL(str(build.build_ref_cpu()))
        L.ftref_cross_entropy.restype = ctypes.c_float
        L.ftref_sumsq.restype = ctypes.c_double
        _LIB = L
    return _LIB


def _f(t: torch.Tensor | None):
    """fp32 contiguous host copy (kept alive by the caller) or None."""
    return None if t is None else t.detach().to("cpu", torch.float32).contiguous()


def _p(t: torch.Tensor | None):
    return ctypes.c_void_p(None if t is None else t.data_ptr())


def _rnd(t: torch.Tensor) -> int:
    return int(t.dtype == torch.bfloat16)


def _back(host: torch.Tensor, like: torch.Tensor, dtype=None) -> torch.Tensor:
    return host.to(device=like.device, dtype=dtype or like.dtype)


def gemm(a, b, M, N, K, a_mn, b_mn, alpha=1.0, out=None, accumulate=False, out_dtype=None):
    A, B = _f(a), _f(b)
    od = out_dtype or (out.dtype if out is not None else a.dtype)
    D = _f(out) if (out is not None and accumulate) else torch.zeros(M, N)
    lib().ftref_gemm(_p(A), _p(B), _p(D), c_int(M), c_int(N), c_int(K), c_int(A.stride(0)),
                     c_int(B.stride(0)), c_int(N), c_int(int(a_mn)), c_int(int(b_mn)),
                     c_float(alpha), c_int(int(accumulate)), c_int(int(od == torch.bfloat16)))
    return D.to(device=a.device, dtype=od)


def linear_fwd(x, w, alpha=1.0):
    return gemm(x, w, x.shape[0], w.shape[0], x.shape[1], 0, 0, alpha)


def linear_dgrad(dy, w, alpha=1.0):
    return gemm(dy, w, dy.shape[0], w.shape[1], dy.shape[1], 0, 1, alpha)


def linear_wgrad(dy, x, out=None, accumulate=False, alpha=1.0):
    return gemm(dy, x, dy.shape[1], x.shape[1], dy.shape[0], 1, 1, alpha, out=out,
                accumulate=accumulate, out_dtype=torch.float32)


def embedding_fwd(ids, w, scale, vocab_start=0):
    I = ids.reshape(-1).to("cpu", torch.int64).contiguous()
    W = _f(w)
    out = torch.empty(I.numel(), W.shape[1])
    lib().ftref_embedding_fwd(_p(I), _p(W), _p(out), c_int(I.numel()), c_int(W.shape[1]),
                              c_float(scale), c_int(vocab_start), c_int(W.shape[0]), c_int(_rnd(w)))
    return _back(out, w)


def embedding_bwd(ids, dy, scale, dw, vocab_start=0):
    I = ids.reshape(-1).to("cpu", torch.int64).contiguous()
    DY, DW = _f(dy), _f(dw)
    lib().ftref_embedding_bwd(_p(I), _p(DY), _p(DW), c_int(I.numel()), c_int(DY.shape[1]),
                              c_float(scale), c_int(vocab_start), c_int(DW.shape[0]))
    dw.copy_(DW)


def add_rmsnorm_fwd(res, x, w, eps):
    R, X, W = _f(res), _f(x), _f(w)
    T, H = X.shape
    h, y, rstd = torch.empty(T, H), torch.empty(T, H), torch.empty(T)
    lib().ftref_add_rmsnorm_fwd(_p(R), _p(X), _p(W), _p(h), _p(y), _p(rstd), c_int(T), c_int(H),
                                c_float(eps), c_int(_rnd(x)))
    return _back(h, x), _back(y, x), _back(rstd, x, torch.float32)


def rmsnorm_bwd(dy, h, w, rstd, dres, dw, accumulate):
    DY, Hh, W, RS, DR, DW = _f(dy), _f(h), _f(w), _f(rstd), _f(dres), _f(dw)
    T, H = DY.shape
    dx = torch.empty(T, H)
    lib().ftref_rmsnorm_bwd(_p(DY), _p(Hh), _p(W), _p(RS), _p(DR), _p(dx), _p(DW),
                            c_int(int(accumulate)), c_int(T), c_int(H), c_int(_rnd(h)))
    dw.copy_(DW)
    return _back(dx, h)


def rope_(qkv, cos, sin, batch, n_groups, heads_per_group, head_dim, inverse=False,
          position_ids=None):
    Q, C, S_ = _f(qkv), _f(cos), _f(sin)
    T = Q.shape[0]
    pos = None if position_ids is None else position_ids.reshape(-1).to("cpu", torch.int32).contiguous()
    lib().ftref_rope(_p(Q), _p(C), _p(S_), _p(pos), c_int(T), c_int(T // batch), c_int(n_groups),
                     c_int(heads_per_group), c_int(head_dim), c_int(int(inverse)), c_int(_rnd(qkv)))
    qkv.copy_(Q)
    return qkv


def swiglu_fwd(y1):
    Y = _f(y1)
    T, F2 = Y.shape
    act = torch.empty(T, F2 // 2)
    lib().ftref_swiglu_fwd(_p(Y), _p(act), c_int(T), c_int(F2 // 2), c_int(_rnd(y1)))
    return _back(act, y1)


def linear_swiglu_fwd(x, w, alpha=1.0):
    """``(y, act)`` of FC1 with the activation folded in (one pass per row, no intermediate)."""
    X, W = _f(x), _f(w)
    T, K = X.shape
    F = W.shape[0] // 2
    y, act = torch.empty(T, 2 * F), torch.empty(T, F)
    lib().ftref_linear_swiglu(_p(X), _p(W), _p(y), _p(act), c_int(T), c_int(F), c_int(K),
                              c_int(X.stride(0)), c_int(W.stride(0)), c_float(alpha), c_int(_rnd(x)))
    return _back(y, x), _back(act, x)


def linear_dgrad_swiglu_bwd(dy, w2, y1, alpha=1.0):
    """``swiglu_bwd(alpha * dy @ w2, y1)`` in one pass per row (no ``[T, F]`` intermediate)."""
    DY, W, Y = _f(dy), _f(w2), _f(y1)
    T, K = DY.shape
    F = W.shape[1]
    dy1 = torch.empty(T, 2 * F)
    lib().ftref_linear_dgrad_swiglu_bwd(_p(DY), _p(W), _p(Y), _p(dy1), c_int(T), c_int(F), c_int(K),
                                        c_int(DY.stride(0)), c_int(W.stride(0)), c_float(alpha),
                                        c_int(_rnd(dy)))
    return _back(dy1, dy)


def swiglu_bwd(dact, y1):
    D, Y = _f(dact), _f(y1)
    T, F2 = Y.shape
    dy1 = torch.empty(T, F2)
    lib().ftref_swiglu_bwd(_p(D), _p(Y), _p(dy1), c_int(T), c_int(F2 // 2), c_int(_rnd(y1)))
    return _back(dy1, y1)


def cross_entropy_fwd_bwd(logits, labels, mask, loss_scale, valid=None, vocab_start=0):
    Lg = _f(logits)
    T, V = Lg.shape
    lab = labels.reshape(-1).to("cpu", torch.int64).contiguous()
    M = None if mask is None else _f(mask.reshape(-1))
    if valid is None:
        valid = float(T) if M is None else max(float(M.sum()), 1.0)
    d = torch.empty(T, V)
    loss = lib().ftref_cross_entropy(_p(Lg), _p(lab), _p(M), c_float(float(valid)), _p(d), c_int(T),
                                     c_int(V), c_int(vocab_start), c_float(loss_scale),
                                     c_int(_rnd(logits)))
    return torch.tensor(loss, dtype=torch.float32, device=logits.device), _back(d, logits)


def attention_fwd(qkv, batch, n_groups, heads_per_group, head_dim, scale=None):
    Q = _f(qkv)
    T = Q.shape[0]
    S = T // batch
    Hq = n_groups * heads_per_group
    scale = 1.0 / math.sqrt(head_dim) if scale is None else scale
    out, lse = torch.empty(T, Hq * head_dim), torch.empty(batch, Hq, S)
    lib().ftref_attention_fwd(_p(Q), _p(out), _p(lse), c_int(batch), c_int(S), c_int(n_groups),
                              c_int(heads_per_group), c_int(head_dim), c_float(scale),
                              c_int(_rnd(qkv)))
    return _back(out, qkv), _back(lse, qkv, torch.float32)


def attention_bwd(dout, qkv, out, lse, batch, n_groups, heads_per_group, head_dim, scale=None):
    DO, Q, O, L = _f(dout), _f(qkv), _f(out), _f(lse)
    T = Q.shape[0]
    scale = 1.0 / math.sqrt(head_dim) if scale is None else scale
    d = torch.empty_like(Q)
    lib().ftref_attention_bwd(_p(DO), _p(Q), _p(O), _p(L), _p(d), c_int(batch), c_int(T // batch),
                              c_int(n_groups), c_int(heads_per_group), c_int(head_dim),
                              c_float(scale), c_int(_rnd(qkv)))
    return _back(d, qkv)


def adamw_step(p32, m, v, g, p_out, lr, beta1, beta2, eps, weight_decay, step, clip=1.0):
    P, M, V, G = _f(p32), _f(m), _f(v), _f(g)
    out = None if p_out is None else torch.empty_like(P)
    lib().ftref_adamw(_p(P), _p(M), _p(V), _p(G), _p(out), c_long(P.numel()), c_float(lr),
                      c_float(beta1), c_float(beta2), c_float(eps), c_float(weight_decay),
                      c_int(step), c_float(clip), c_int(0 if p_out is None else _rnd(p_out)))
    p32.copy_(P), m.copy_(M), v.copy_(V)
    if p_out is not None:
        p_out.copy_(out)


def sumsq(x):
    X = _f(x)
    return torch.tensor(lib().ftref_sumsq(_p(X), c_long(X.numel())), dtype=torch.float32,
                        device=x.device)
