"""Float8 linear layers for ``fp8: true`` training: row-wise scaled e4m3 / e5m2 operands, fp32 accumulation on the
CTA-pair tcgen05 GEMM (``csrc/kernels/gemm_bf16_2cta.cu``, ``kind::f8f6f4``), scales applied in the GEMM epilogue.

The recipe is the reference's default (torchao ``Float8LinearConfig.from_recipe_name("rowwise")`` behind
``train/fp8_utils.py:29-106``): every GEMM operand carries one scale per row *of that GEMM*, i.e. per token for
activations and gradients, per output feature for the weight in the forward pass, and per input feature / per feature
when the same tensor is contracted over its other axis in the two backward GEMMs:

    y  = q_rows(x)     . q_rows(W)^T          x [M, K],  W [N, K]
    dx = q_rows(dy)    . q_cols_t(W)^T        dy [M, N], W^T quantised per input feature
    dW = q_cols_t(dy)  . q_cols_t(x)^T        both quantised per feature and written transposed ([N, M], [K, M])

Gradients are quantised to e5m2 (range), activations and weights to e4m3 (precision).  Embeddings, the LM head and
layers whose dimensions are not multiples of 16 stay in bf16, as in the reference's module filter.  On tensors that
are not bf16 CUDA tensors the same quantise / de-quantise arithmetic runs in PyTorch (the numerical reference of the
kernels, and the CPU path of the tests).
"""
from __future__ import annotations

import ctypes
from typing import Optional, Tuple

import torch
import torch.nn.functional as F

from . import _lib

E4M3, E5M2 = 0, 1
_FMAX = {E4M3: 448.0, E5M2: 57344.0}
_TORCH_DT = {E4M3: torch.float8_e4m3fn, E5M2: torch.float8_e5m2}
c_int, c_ll = ctypes.c_int, ctypes.c_longlong


def _on_gpu(x: torch.Tensor) -> bool:
    return x.is_cuda and x.dtype == torch.bfloat16 and _lib.kernels_available()


def quant_rows(x: torch.Tensor, fmt: int = E4M3) -> Tuple[torch.Tensor, torch.Tensor]:
    """``x [R, C]`` -> ``(q [R, C] uint8 holding fp8 bits, scale [R] fp32)`` with ``x ~ q * scale[:, None]``."""
    R, C = x.shape
    if _on_gpu(x) and C % 16 == 0:
        x = x if (x.stride(1) == 1 and x.stride(0) % 8 == 0) else x.contiguous()
        q = torch.empty(R, C, device=x.device, dtype=torch.uint8)
        scale = torch.empty(R, device=x.device, dtype=torch.float32)
        _lib.check(_lib.kernels().hmf_fp8_quant_rows(_lib.ptr(x), c_ll(x.stride(0)), _lib.ptr(q), c_ll(C), _lib.ptr(scale),
                                                     c_ll(R), c_int(C), c_int(fmt), _lib.stream_ptr(x.device)), "fp8_quant_rows")
        return q, scale
    amax = x.float().abs().amax(-1)
    scale = torch.where(amax > 0, amax / _FMAX[fmt], torch.ones_like(amax))
    q = (x.float() / scale[:, None]).clamp(-_FMAX[fmt], _FMAX[fmt]).to(_TORCH_DT[fmt]).view(torch.uint8)
    return q, scale


def quant_cols_t(x: torch.Tensor, fmt: int = E4M3) -> Tuple[torch.Tensor, torch.Tensor]:
    """``x [R, C]`` -> ``(q_t [C, R] uint8, scale [C] fp32)``: quantised per column of ``x`` and transposed."""
    R, C = x.shape
    if _on_gpu(x) and R % 16 == 0:
        x = x if x.stride(1) == 1 else x.contiguous()
        qt = torch.empty(C, R, device=x.device, dtype=torch.uint8)
        scale = torch.empty(C, device=x.device, dtype=torch.float32)
        amax = torch.empty(C, device=x.device, dtype=torch.float32)
        _lib.check(_lib.kernels().hmf_fp8_quant_cols_t(_lib.ptr(x), c_ll(x.stride(0)), _lib.ptr(qt), c_ll(R), _lib.ptr(scale),
                                                       _lib.ptr(amax), c_ll(R), c_int(C), c_int(fmt),
                                                       _lib.stream_ptr(x.device)), "fp8_quant_cols_t")
        _lib.add_launches(1)
        return qt, scale
    q, scale = quant_rows(x.t().contiguous(), fmt)
    return q, scale


def dequant(q: torch.Tensor, scale: torch.Tensor, fmt: int = E4M3) -> torch.Tensor:
    return q.view(_TORCH_DT[fmt]).float() * scale[:, None]


def gemm_fp8(aq: torch.Tensor, sa: torch.Tensor, bq: torch.Tensor, sb: torch.Tensor, fmt_a: int = E4M3,
             fmt_b: int = E4M3, bias: Optional[torch.Tensor] = None, out_dtype=torch.bfloat16) -> torch.Tensor:
    """``(aq [M, K] * sa[:, None]) @ (bq [N, K] * sb[:, None]).T`` with fp32 accumulation."""
    M, K = aq.shape
    N = bq.shape[0]
    if aq.is_cuda and _lib.kernels_available() and K % 16 == 0:
        out = torch.empty(M, N, device=aq.device, dtype=out_dtype)
        if bias is not None:
            bias = bias.float().contiguous()
        _lib.check(_lib.kernels().hmf_gemm_fp8_2cta(
            _lib.ptr(aq), _lib.ptr(bq), _lib.ptr(out), _lib.ptr(sa), _lib.ptr(sb), _lib.ptr(bias), c_int(M), c_int(N),
            c_int(K), c_ll(aq.stride(0)), c_ll(bq.stride(0)), c_ll(out.stride(0)), c_int(fmt_a), c_int(fmt_b),
            c_int(0 if out_dtype == torch.bfloat16 else 1), _lib.stream_ptr(aq.device)), "gemm_fp8")
        return out
    res = dequant(aq, sa, fmt_a) @ dequant(bq, sb, fmt_b).t()
    if bias is not None:
        res = res + bias.float()
    return res.to(out_dtype)


class _Fp8Linear(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, b):
        x2 = x.reshape(-1, x.shape[-1])
        xq, sx = quant_rows(x2, E4M3)
        wq, sw = quant_rows(w, E4M3)
        y = gemm_fp8(xq, sx, wq, sw, E4M3, E4M3, bias=b, out_dtype=x.dtype)
        ctx.save_for_backward(x2, w)
        ctx.has_bias, ctx.x_shape = b is not None, x.shape
        return y.view(*x.shape[:-1], w.shape[0])

    @staticmethod
    def backward(ctx, dy):
        x2, w = ctx.saved_tensors
        dy2 = dy.reshape(-1, dy.shape[-1])
        dx = dw = db = None
        if ctx.needs_input_grad[0]:
            dyq, sdy = quant_rows(dy2, E5M2)                 # [M, N] per token
            wtq, swt = quant_cols_t(w, E4M3)                 # [K, N] per input feature
            dx = gemm_fp8(dyq, sdy, wtq, swt, E5M2, E4M3, out_dtype=dy.dtype).view(ctx.x_shape)
        if ctx.needs_input_grad[1]:
            dytq, sdyt = quant_cols_t(dy2, E5M2)             # [N, M] per output feature
            xtq, sxt = quant_cols_t(x2, E4M3)                # [K, M] per input feature
            dw = gemm_fp8(dytq, sdyt, xtq, sxt, E5M2, E4M3, out_dtype=w.dtype)
        if ctx.has_bias and ctx.needs_input_grad[2]:
            db = dy2.float().sum(0).to(dy.dtype)
        return dx, dw, db


def fp8_linear(x: torch.Tensor, w: torch.Tensor, b: Optional[torch.Tensor] = None) -> torch.Tensor:
    if x.shape[-1] % 16 or w.shape[0] % 16 or x.numel() == 0:
        return F.linear(x, w, b)
    return _Fp8Linear.apply(x, w, b)


class Fp8Linear(torch.nn.Linear):
    """``nn.Linear`` whose three GEMMs run in row-wise scaled float8.  Same parameters and state-dict keys."""

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return fp8_linear(x, self.weight, self.bias)


SKIP_NAMES = ("embed", "lm_head", "output", "classifier", "score", "v_head", "router", "gate.")


def use_fp8_linear(model: torch.nn.Module, skip=SKIP_NAMES) -> int:
    """Re-classes the eligible linear layers of ``model`` in place (``fp8: true``); returns how many.  Skipped: names
    containing one of ``skip`` (embeddings, heads, routers) and layers with a dimension that is not a multiple of 16
    (reference: ``train/fp8_utils.py::module_filter_func``)."""
    n = 0
    for name, m in model.named_modules():
        if not isinstance(m, torch.nn.Linear) or isinstance(m, Fp8Linear):
            continue
        if type(m).__name__ not in ("Linear",):               # adapters and other subclasses keep their own forward
            continue
        low = (name + ".").lower()
        if any(s in low for s in skip) or m.in_features % 16 or m.out_features % 16:
            continue
        m.__class__ = Fp8Linear
        n += 1
    return n
