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
import os
from typing import Optional

import torch
import torch.nn.functional as F

from . import _lib

_OUT_MODES = {"bf16": 0, "f32": 1, "f32_accumulate": 2}


def _use_pair_kernel(M: int, N: int, pair) -> bool:
    """The CTA-pair kernel (256 x 256 tiles on two SMs, ``gemm_bf16_2cta.cu``) takes problems with at least one full
    tile; ``HMF_GEMM_PAIR=0`` keeps everything on the single-CTA kernel."""
    if pair is not None:
        return bool(pair)
    return M >= 256 and N >= 256 and os.environ.get("HMF_GEMM_PAIR", "1") != "0"


def gemm(a: torch.Tensor, b: torch.Tensor, *, a_mn_major: bool = False, b_mn_major: bool = False,
         bias: torch.Tensor | None = None, out: torch.Tensor | None = None,
         out_mode: str = "bf16", pair: bool | None = None) -> torch.Tensor:
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
    K_ = _lib.kernels()
    fn = K_.hmf_gemm_bf16_2cta if _use_pair_kernel(M, N, pair) else K_.hmf_gemm_bf16
    rc = fn(
        _lib.ptr(a), _lib.ptr(b), _lib.ptr(out), _lib.ptr(bias),
        ctypes.c_int(M), ctypes.c_int(N), ctypes.c_int(K),
        ctypes.c_longlong(a.stride(0)), ctypes.c_longlong(b.stride(0)),
        ctypes.c_longlong(out.stride(0)),
        ctypes.c_int(int(a_mn_major)), ctypes.c_int(int(b_mn_major)),
        ctypes.c_int(_OUT_MODES[out_mode]), _lib.stream_ptr(a.device))
    _lib.check(rc, "hmf_gemm_bf16")
    return out


# ------------------------------------------------------------------------------------------------------
# nn.Linear on the kernel above
# ------------------------------------------------------------------------------------------------------
# Below this many rows (decode steps) a 128-row tile is mostly padding and the weight read dominates: those calls go
# to the swap-AB kernel (weight rows on the MMA M axis, the few activation rows on N, K split over more SMs when the
# weight has few 128-row tiles), ``csrc/kernels/gemm_allreduce.cu`` on one rank.
MIN_ROWS = 128
_skinny_state = {}


def _skinny_ok(x2: torch.Tensor, w: torch.Tensor) -> bool:
    return (x2.is_cuda and x2.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and w.dim() == 2 and x2.dim() == 2
            and 1 <= x2.shape[0] <= 256 and w.shape[0] % 128 == 0 and w.shape[1] % 64 == 0
            and x2.shape[1] == w.shape[1] and w.stride(1) == 1 and w.stride(0) % 8 == 0 and w.data_ptr() % 16 == 0
            and _lib.kernels_available() and os.environ.get("HMF_LINEAR", "own") == "own")


def skinny_gemm(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``y [M, N] = x [M, K] w [N, K]^T + bias`` for ``M <= 256`` (decode batches) on the swap-AB tcgen05 kernel."""
    from .fused_comm import PeerGemmAllReduce
    x2 = _rows(x)
    M, K = x2.shape
    N = w.shape[0]
    dev = x2.device
    st = _skinny_state.get(dev.index)
    if st is None:      # partial / flag scratch of the K-split reduction (unused when one split covers K)
        st = _skinny_state[dev.index] = PeerGemmAllReduce(None, 256, 16384, dev)     # fp32 partials: half the capacity
    # K splits put more CTAs on the weight stream when the weight has few 128-row tiles; two CTAs fit on an SM, so
    # up to 296 are resident at once.  The splits of a tile form one cluster and meet in shared memory.
    splits, tiles = 1, N // 128
    if N <= st.max_n // 2:
        while (splits < st.MAX_SPLIT and tiles * splits * 2 <= 296 and K % (splits * 2 * 64) == 0
               and K // (splits * 2) >= 256):
            splits *= 2
    y = torch.empty(M, N, device=dev, dtype=torch.bfloat16)
    c_int, c_ll = ctypes.c_int, ctypes.c_longlong
    _lib.check(_lib.kernels().hmf_gemm_skinny(
        _lib.ptr(x2), _lib.ptr(w), _lib.ptr(bias), _lib.ptr(y), c_int(M), c_int(N), c_int(K), c_ll(x2.stride(0)),
        c_ll(w.stride(0)), st.part_ptrs, st.flag_ptrs, _lib.ptr(st.sync), c_ll(st.part_stride), c_int(st.max_tiles),
        c_int(splits), _lib.stream_ptr(dev)), "gemm_skinny")
    return y


def _own_linear_ok(x: torch.Tensor, w: torch.Tensor) -> bool:
    return (x.is_cuda and x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and w.dim() == 2
            and w.shape[0] % 8 == 0 and w.shape[1] % 8 == 0 and w.is_contiguous() and x.shape[-1] == w.shape[1]
            and x.numel() >= MIN_ROWS * x.shape[-1] and w.data_ptr() % 16 == 0 and _lib.kernels_available()
            and os.environ.get("HMF_LINEAR", "own") == "own")


def _rows(x: torch.Tensor) -> torch.Tensor:
    """``[..., K] -> [M, K]`` with unit inner stride, a row stride that is a multiple of 8 and a 16-byte aligned
    base (what a TMA descriptor needs); a copy only if the view does not qualify."""
    x2 = x.reshape(-1, x.shape[-1])
    if x2.stride(1) != 1 or x2.stride(0) % 8 != 0 or x2.data_ptr() % 16 != 0:
        x2 = x2.contiguous()
    return x2


class _Linear(torch.autograd.Function):
    """``y = x W^T + b`` with all three GEMMs (forward, input gradient, weight gradient) on the tcgen05 kernel; the
    operands are read in the layout they already have (no transposes)."""

    @staticmethod
    def forward(ctx, x, w, b):
        x2 = _rows(x)
        y = gemm(x2, w, bias=b)
        ctx.save_for_backward(x2, w)
        ctx.has_bias, ctx.x_shape = b is not None, x.shape
        return y.view(*x.shape[:-1], w.shape[0])

    @staticmethod
    def backward(ctx, dy):
        x2, w = ctx.saved_tensors
        dy2 = _rows(dy)
        dx = dw = db = None
        if ctx.needs_input_grad[0]:
            dx = gemm(dy2, w, b_mn_major=True).view(ctx.x_shape)             # [M, N] x [N, K]
        if ctx.needs_input_grad[1]:
            dw = gemm(dy2, x2, a_mn_major=True, b_mn_major=True)             # [N, M] x [M, K]
        if ctx.has_bias and ctx.needs_input_grad[2]:
            db = dy2.float().sum(0).to(dy.dtype)
        return dx, dw, db


def linear(x: torch.Tensor, w: torch.Tensor, b: torch.Tensor | None = None) -> torch.Tensor:
    """Drop-in for ``F.linear``: bf16 CUDA operands run on the library's own GEMM (set ``HMF_LINEAR=cublas`` to
    compare against the vendor library), everything else takes ``F.linear``."""
    if not _own_linear_ok(x, w):
        if (x.is_cuda and x.dtype == torch.bfloat16 and x.numel() < MIN_ROWS * x.shape[-1] and x.numel() > 0
                and not (torch.is_grad_enabled() and (x.requires_grad or w.requires_grad))
                and (b is None or b.dtype == torch.bfloat16) and _skinny_ok(x.reshape(-1, x.shape[-1]), w)):
            return skinny_gemm(x, w, b).view(*x.shape[:-1], w.shape[0])
        return F.linear(x, w, b)
    if torch.is_grad_enabled() and (x.requires_grad or w.requires_grad or (b is not None and b.requires_grad)):
        return _Linear.apply(x, w, b)
    return gemm(_rows(x), w, bias=b).view(*x.shape[:-1], w.shape[0])


class Linear(torch.nn.Linear):
    """``nn.Linear`` whose forward and backward run on the library's GEMM.  Same parameters, same state-dict keys."""

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return linear(x, self.weight, self.bias)


def use_own_linear(model: torch.nn.Module) -> int:
    """Re-classes every plain ``nn.Linear`` of ``model`` in place (parameters and names untouched); returns how many."""
    n = 0
    for m in model.modules():
        if type(m) is torch.nn.Linear:
            m.__class__ = Linear
            n += 1
    return n
