"""The allocation-free RMSNorm-backward entry point (``ft_rmsnorm_bwd_noalloc``).

Some users of the library cannot allocate device memory at the point of the call: code running
inside a CUDA-graph capture, hosts that gave the whole GPU to a fixed-size pool, C programs
without a tensor allocator. For them the library carries its own scratch for this kernel. The
test calls the exported C symbol directly (no Python wrapper in between) twice in a row and
compares both results with the regular entry point, which takes its scratch from the caller.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _ptr(t):
    return ctypes.c_void_p(0 if t is None else t.data_ptr())


# H = 8192 fills the scratch rows to their full width (FT_NOALLOC_MAX_HIDDEN)
@pytest.mark.parametrize("T,H", [(1000, 1024), (4096, 4096), (300, 256), (2048, 8192)])
def test_noalloc_entry_point_matches_regular_entry_point(T, H):
    from forgetrain_b200.ops import _lib
    lib = ctypes.CDLL(str(_lib.LIB_PATH))          # the raw exported symbols
    lib.ft_rmsnorm_bwd_noalloc.restype = ctypes.c_int
    lib.ft_rmsnorm_bwd.restype = ctypes.c_int
    lib.ft_rmsnorm_bwd_partials.restype = ctypes.c_int
    torch.manual_seed(0)
    dev = "cuda"
    st = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    w = (1 + 0.1 * torch.randn(H, device=dev)).to(torch.bfloat16)
    nparts = lib.ft_rmsnorm_bwd_partials(ctypes.c_int(T), ctypes.c_int(H))
    partial = torch.empty(nparts, H, dtype=torch.float32, device=dev)
    for call in range(2):                           # two calls in a row share the scratch array
        dy = torch.randn(T, H, device=dev).to(torch.bfloat16)
        h = torch.randn(T, H, device=dev).to(torch.bfloat16)
        rstd = torch.rsqrt(h.float().pow(2).mean(-1) + 1e-6)
        dres = torch.randn(T, H, device=dev).to(torch.bfloat16)
        dx_ref, dx_new = torch.empty_like(dy), torch.empty_like(dy)
        dw_ref = torch.full((H,), 3.0, device=dev)
        dw_new = torch.full((H,), 3.0, device=dev)
        acc = ctypes.c_int(call)                    # second call also checks accumulate
        rc = lib.ft_rmsnorm_bwd(_ptr(dy), _ptr(h), _ptr(w), _ptr(rstd), _ptr(dres), _ptr(dx_ref),
                                _ptr(partial), _ptr(dw_ref), acc, ctypes.c_int(T), ctypes.c_int(H), st)
        assert rc == 0
        rc = lib.ft_rmsnorm_bwd_noalloc(_ptr(dy), _ptr(h), _ptr(w), _ptr(rstd), _ptr(dres),
                                        _ptr(dx_new), _ptr(dw_new), acc, ctypes.c_int(T),
                                        ctypes.c_int(H), st)
        assert rc == 0
        torch.cuda.synchronize()
        assert torch.equal(dx_new, dx_ref)
        err = float((dw_new - dw_ref).abs().max() / (dw_ref.abs().max() + 1e-9))
        assert err < 1e-4, err


def test_noalloc_entry_point_rejects_sizes_beyond_its_scratch():
    from forgetrain_b200.ops import _lib
    lib = ctypes.CDLL(str(_lib.LIB_PATH))
    lib.ft_rmsnorm_bwd_noalloc.restype = ctypes.c_int
    z = ctypes.c_void_p(0)
    st = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    assert lib.ft_rmsnorm_bwd_noalloc(z, z, z, z, z, z, z, ctypes.c_int(0), ctypes.c_int(8),
                                      ctypes.c_int(16384), st) == -2
    assert lib.ft_rmsnorm_bwd_noalloc(z, z, z, z, z, z, z, ctypes.c_int(0), ctypes.c_int(8),
                                      ctypes.c_int(1000), st) == -1
