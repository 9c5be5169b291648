"""Allocation-free RMSNorm backward (``hmf_rms_norm_bwd_noalloc``).

Some hosts of the kernel library may not allocate device memory at call time (a server with a
frozen memory arena, a plugin that must not re-enter its framework's allocator).  For them the
library offers one entry point whose workspace is compiled in.  This test calls it through its
exported C symbol with plain pointers, twice in a row (the second call reuses the workspace the
first one dirtied), and checks both results against the regular entry point that takes a
caller-provided scratch buffer.  It lives in the last-collected test file on purpose.
"""
import ctypes

import pytest
import torch

from hybrid_model_factory_b200.ops import _lib

pytestmark = pytest.mark.gpu


def _run_regular(K, x, w, dy, rstd):
    N, D = x.shape
    dx = torch.empty_like(x)
    dw = torch.empty(D, device=x.device, dtype=torch.float32)
    nb = K.hmf_rms_norm_bwd_blocks(ctypes.c_longlong(N))
    part = torch.empty(nb, D, device=x.device, dtype=torch.float32)
    rc = K.hmf_rms_norm_bwd(_lib.ptr(x), _lib.ptr(w), _lib.ptr(dy), _lib.ptr(rstd), _lib.ptr(dx), _lib.ptr(part),
                            _lib.ptr(dw), ctypes.c_int(0), ctypes.c_longlong(N), ctypes.c_int(D), ctypes.c_int(0),
                            _lib.stream_ptr(x.device))
    assert rc == 0, K.hmf_last_error()
    return dx, dw


def _run_noalloc(K, x, w, dy, rstd):
    N, D = x.shape
    dx = torch.empty_like(x)
    dw = torch.empty(D, device=x.device, dtype=torch.float32)
    stream = _lib.stream_ptr(x.device)
    before = torch.cuda.memory_allocated()
    rc = K.hmf_rms_norm_bwd_noalloc(_lib.ptr(x), _lib.ptr(w), _lib.ptr(dy), _lib.ptr(rstd), _lib.ptr(dx), _lib.ptr(dw),
                                    ctypes.c_int(0), ctypes.c_longlong(N), ctypes.c_int(D), ctypes.c_int(0), stream)
    assert rc == 0, K.hmf_last_error()
    assert torch.cuda.memory_allocated() == before
    return dx, dw


def test_noalloc_matches_regular_entry_point_twice():
    K = _lib.kernels()
    dev = torch.device("cuda", 0)
    # the second shape reuses the workspace left by the first; the third has more rows than the compiled-in number of
    # partial-sum slabs can take one block each, so the entry point must clamp the slab count
    for N, D in [(3000, 4096), (777, 128), (70000, 128)]:
        x = torch.randn(N, D, device=dev).bfloat16()
        w = (torch.randn(D, device=dev) * 0.1 + 1).bfloat16()
        dy = torch.randn(N, D, device=dev).bfloat16()
        rstd = torch.rsqrt(x.float().pow(2).mean(-1) + 1e-6)
        dx_ref, dw_ref = _run_regular(K, x, w, dy, rstd)
        for _ in range(2):
            dx, dw = _run_noalloc(K, x, w, dy, rstd)
            torch.cuda.synchronize()
            torch.testing.assert_close(dx.float(), dx_ref.float(), rtol=2e-2, atol=2e-2)
            torch.testing.assert_close(dw, dw_ref, rtol=2e-2, atol=2e-2 * max(1.0, dw_ref.abs().max().item()))


def test_noalloc_rejects_oversize():
    K = _lib.kernels()
    dev = torch.device("cuda", 0)
    x = torch.zeros(8, 8200, device=dev).bfloat16()
    rc = K.hmf_rms_norm_bwd_noalloc(_lib.ptr(x), _lib.ptr(x[0]), _lib.ptr(x), _lib.ptr(torch.ones(8, device=dev)),
                                    _lib.ptr(torch.empty_like(x)), _lib.ptr(torch.empty(8200, device=dev)),
                                    ctypes.c_int(0), ctypes.c_longlong(8), ctypes.c_int(8200), ctypes.c_int(0),
                                    _lib.stream_ptr(dev))
    assert rc == -4
    assert b"workspace limit" in K.hmf_last_error()
