"""bf16 GEMM on tcgen05 tensor cores (``csrc/kernels/gemm_bf16.cu``).

``gemm(a, b, a_mn_major=False, b_mn_major=False)`` computes ``op(a) @ op(b).T`` with fp32
accumulation in tensor memory:

* ``a`` stored ``[M, K]`` (K-major) or ``[K, M]`` (``a_mn_major``)
* ``b`` stored ``[N, K]`` (K-major, the ``nn.Linear`` weight layout) or ``[K, N]``

so the three GEMMs of a linear layer (forward, input gradient, weight gradient) read their
operands where they already are, without transpose passes.  On CPU tensors the same contract
is evaluated with ``torch.matmul`` in fp32 (reference).
"""
from __future__ import annotations

import ctypes

import torch

from . import _lib

_OUT_MODES = {"bf16": 0, "f32": 1, "f32_accumulate": 2}


def gemm(a: torch.Tensor, b: torch.Tensor, *, a_mn_major: bool = False, b_mn_major: bool = False,
         bias: torch.Tensor | None = None, out: torch.Tensor | None = None,
         out_mode: str = "bf16") -> torch.Tensor:
    assert a.dim() == 2 and b.dim() == 2
    M, K = (a.shape[1], a.shape[0]) if a_mn_major else a.shape
    N, Kb = (b.shape[1], b.shape[0]) if b_mn_major else b.shape
    assert K == Kb, f"contraction mismatch {K} vs {Kb}"
    if not _lib.use_cuda_kernels(a, b):
        am = a.float().t() if a_mn_major else a.float()
        bm = b.float() if b_mn_major else b.float().t()
        res = am @ bm
        if bias is not None:
            res = res + bias.float()
        if out_mode == "f32_accumulate":
            out.add_(res)
            return out
        res = res.to(torch.bfloat16 if out_mode == "bf16" else torch.float32)
        if out is not None:
            out.copy_(res)
            return out
        return res
    assert a.dtype == torch.bfloat16 and b.dtype == torch.bfloat16
    assert a.stride(1) == 1 and b.stride(1) == 1, "operands must be row-major (unit inner stride)"
    if out is None:
        assert out_mode != "f32_accumulate", "accumulate needs an existing output"
        out = torch.empty(M, N, device=a.device,
                          dtype=torch.bfloat16 if out_mode == "bf16" else torch.float32)
    assert out.stride(1) == 1
    if bias is not None:
        bias = bias.float().contiguous()
    rc = _lib.kernels().hmf_gemm_bf16(
        _lib.ptr(a), _lib.ptr(b), _lib.ptr(out), _lib.ptr(bias),
        ctypes.c_int(M), ctypes.c_int(N), ctypes.c_int(K),
        ctypes.c_longlong(a.stride(0)), ctypes.c_longlong(b.stride(0)),
        ctypes.c_longlong(out.stride(0)),
        ctypes.c_int(int(a_mn_major)), ctypes.c_int(int(b_mn_major)),
        ctypes.c_int(_OUT_MODES[out_mode]), _lib.stream_ptr(a.device))
    _lib.check(rc, "hmf_gemm_bf16")
    return out
