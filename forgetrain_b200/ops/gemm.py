"""bf16 GEMMs on the tcgen05 kernel (``csrc/gemm_sm100.cu``).

Three entry points cover what a linear layer needs, all on the same kernel with different
operand majors, so no transposed copies are made:

* :func:`linear_fwd`   ``y = alpha * x @ w.T``            (bf16 out)
* :func:`linear_dgrad` ``dx = alpha * dy @ w``            (bf16 out)
* :func:`linear_wgrad` ``dw (+)= dy.T @ x``               (fp32 out, optional accumulate)
* :func:`linear_swiglu_fwd` FC1 forward with ``silu(gate) * up`` computed in the epilogue
* :func:`linear_dgrad_swiglu_bwd` FC2 dgrad with the SwiGLU backward computed in the epilogue

Plays the role of the reference's ``custom_gemm_<op>_{fwd,dgrad,wgrad}`` shims
(exports/train_engine_8b/src/training_engine_tensor/custom_gemm.py:81-225) for all five
projections at once.
"""
from __future__ import annotations

import torch

from . import _lib

c_int, c_float = _lib.c_int, _lib.c_float


def _check2d(t: torch.Tensor, name: str, dtype) -> None:
    if t.dim() != 2 or t.dtype != dtype or not t.is_cuda:
        raise ValueError(f"{name}: expected a 2-D CUDA {dtype} tensor, got {tuple(t.shape)} {t.dtype}")
    if t.stride(1) != 1:
        raise ValueError(f"{name}: innermost dimension must be contiguous")
    esz = t.element_size()
    if t.data_ptr() % 16 or (t.stride(0) * esz) % 16:
        raise ValueError(f"{name}: base and row pitch must be 16-byte aligned")


def gemm_raw(a, b, d, M, N, K, a_mn, b_mn, *, accumulate=False, alpha=1.0, splitk=0, bn=0,
             max_ctas=0) -> None:
    """Low-level launch; see ``ft_gemm_bf16`` in csrc/gemm_sm100.cu for the conventions."""
    L = _lib.lib()
    out_dtype = 0 if d.dtype == torch.bfloat16 else 1
    rc = L.ft_gemm_bf16(_lib.ptr(a), _lib.ptr(b), _lib.ptr(d), c_int(M), c_int(N), c_int(K),
                        c_int(a.stride(0)), c_int(b.stride(0)), c_int(d.stride(0)),
                        c_int(int(a_mn)), c_int(int(b_mn)), c_int(out_dtype),
                        c_int(int(accumulate)), c_float(alpha), c_int(splitk), c_int(bn),
                        c_int(max_ctas), _lib.ptr(_lib.status_word(a.device)), _lib.stream())
    _lib.check_rc(rc, "ft_gemm_bf16")


def linear_fwd(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor | None = None,
               alpha: float = 1.0, **kw) -> torch.Tensor:
    """``out[T,N] = alpha * x[T,K] @ w[N,K].T`` (bf16)."""
    _check2d(x, "x", torch.bfloat16)
    _check2d(w, "w", torch.bfloat16)
    T, K = x.shape
    N = w.shape[0]
    assert w.shape[1] == K
    if out is None:
        out = torch.empty(T, N, dtype=torch.bfloat16, device=x.device)
    _check2d(out, "out", torch.bfloat16)
    gemm_raw(x, w, out, T, N, K, 0, 0, alpha=alpha, **kw)
    return out


def linear_swiglu_fwd(x: torch.Tensor, w: torch.Tensor, alpha: float = 1.0,
                      max_ctas: int = 0) -> tuple[torch.Tensor, torch.Tensor]:
    """FC1 with the activation in the GEMM epilogue: ``y = alpha * x @ w.T`` with
    ``w = [gate rows ; up rows]`` (``[2F, K]``) and ``act = silu(y[:, :F]) * y[:, F:]``, one kernel.
    ``act`` is bitwise what ``swiglu_fwd(y)`` returns. ``F`` must be a multiple of 128."""
    _check2d(x, "x", torch.bfloat16)
    _check2d(w, "w", torch.bfloat16)
    T, K = x.shape
    F = w.shape[0] // 2
    assert w.shape[1] == K and w.shape[0] == 2 * F and F % 128 == 0
    y = torch.empty(T, 2 * F, dtype=torch.bfloat16, device=x.device)
    act = torch.empty(T, F, dtype=torch.bfloat16, device=x.device)
    rc = _lib.lib().ft_gemm_swiglu_bf16(
        _lib.ptr(x), _lib.ptr(w), _lib.ptr(y), _lib.ptr(act), c_int(T), c_int(F), c_int(K),
        c_int(x.stride(0)), c_int(w.stride(0)), c_int(y.stride(0)), c_int(act.stride(0)),
        c_float(alpha), c_int(max_ctas), _lib.ptr(_lib.status_word(x.device)), _lib.stream())
    _lib.check_rc(rc, "ft_gemm_swiglu_bf16")
    return y, act


def linear_dgrad(dy: torch.Tensor, w: torch.Tensor, out: torch.Tensor | None = None,
                 alpha: float = 1.0, **kw) -> torch.Tensor:
    """``out[T,K] = alpha * dy[T,N] @ w[N,K]`` (bf16)."""
    _check2d(dy, "dy", torch.bfloat16)
    _check2d(w, "w", torch.bfloat16)
    T, N = dy.shape
    K = w.shape[1]
    assert w.shape[0] == N
    if out is None:
        out = torch.empty(T, K, dtype=torch.bfloat16, device=dy.device)
    _check2d(out, "out", torch.bfloat16)
    gemm_raw(dy, w, out, T, K, N, 0, 1, alpha=alpha, **kw)
    return out


def linear_dgrad_swiglu_bwd(dy: torch.Tensor, w2: torch.Tensor, y1: torch.Tensor,
                            alpha: float = 1.0, max_ctas: int = 0) -> torch.Tensor:
    """``dy1[T,2F] = swiglu_bwd(alpha * dy[T,H] @ w2[H,F], y1[T,2F])`` in one kernel: the gradient of
    the activation stays in the accumulator. Bitwise what ``linear_dgrad`` followed by
    ``swiglu_bwd`` returns. ``F`` must be a multiple of 64."""
    _check2d(dy, "dy", torch.bfloat16)
    _check2d(w2, "w2", torch.bfloat16)
    _check2d(y1, "y1", torch.bfloat16)
    T, H = dy.shape
    F = w2.shape[1]
    assert w2.shape[0] == H and y1.shape == (T, 2 * F) and F % 64 == 0
    dy1 = torch.empty(T, 2 * F, dtype=torch.bfloat16, device=dy.device)
    rc = _lib.lib().ft_gemm_swiglu_bwd_bf16(
        _lib.ptr(dy), _lib.ptr(w2), _lib.ptr(y1), _lib.ptr(dy1), c_int(T), c_int(F), c_int(H),
        c_int(dy.stride(0)), c_int(w2.stride(0)), c_int(y1.stride(0)), c_int(dy1.stride(0)),
        c_float(alpha), c_int(max_ctas), _lib.ptr(_lib.status_word(dy.device)), _lib.stream())
    _lib.check_rc(rc, "ft_gemm_swiglu_bwd_bf16")
    return dy1


def linear_wgrad(dy: torch.Tensor, x: torch.Tensor, out: torch.Tensor | None = None,
                 accumulate: bool = False, alpha: float = 1.0, **kw) -> torch.Tensor:
    """``out[N,K] (+)= alpha * dy[T,N].T @ x[T,K]`` with fp32 output."""
    _check2d(dy, "dy", torch.bfloat16)
    _check2d(x, "x", torch.bfloat16)
    T, N = dy.shape
    K = x.shape[1]
    assert x.shape[0] == T
    if out is None:
        assert not accumulate
        out = torch.empty(N, K, dtype=torch.float32, device=dy.device)
    _check2d(out, "out", torch.float32)
    gemm_raw(dy, x, out, N, K, T, 1, 1, accumulate=accumulate, alpha=alpha, **kw)
    return out
