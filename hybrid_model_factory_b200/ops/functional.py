"""Public functional API of the op library.

Every function takes tensors on either device:

* CUDA tensors run the hand-written sm_100a kernels of ``csrc/kernels`` (bound in
  ``ops/cuda_ops.py``) wrapped in ``torch.autograd.Function``s whose backward is a kernel too;
* CPU tensors run the differentiable PyTorch reference of ``ops/reference.py``.

There is no silent fallback on a GPU: if the kernel library is missing the call raises.
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch

from . import _lib
from . import reference as R

Tensor = torch.Tensor


def _cuda(*ts) -> bool:
    return _lib.use_cuda_kernels(*[t for t in ts if isinstance(t, torch.Tensor)])


def _ck():
    from . import cuda_ops
    return cuda_ops


# -- normalisation / elementwise ------------------------------------------------------------
def rms_norm(x: Tensor, weight: Optional[Tensor], eps: float = 1e-6, zero_centered: bool = False) -> Tensor:
    if _cuda(x):
        return _ck().rms_norm(x, weight, eps, zero_centered)
    return R.rms_norm(x, weight, eps, zero_centered)


def fused_add_rms_norm(x: Tensor, residual: Tensor, weight: Tensor, eps: float = 1e-6) -> Tuple[Tensor, Tensor]:
    if _cuda(x, residual):
        return _ck().fused_add_rms_norm(x, residual, weight, eps)
    return R.fused_add_rms_norm(x, residual, weight, eps)


def gated_rms_norm(x: Tensor, gate: Tensor, weight: Tensor, eps: float = 1e-5, norm_before_gate: bool = True) -> Tensor:
    if _cuda(x, gate):
        return _ck().gated_rms_norm(x, gate, weight, eps, norm_before_gate)
    return R.gated_rms_norm(x, gate, weight, eps, norm_before_gate)


def swiglu(gate: Tensor, up: Tensor) -> Tensor:
    if _cuda(gate, up):
        return _ck().swiglu(gate, up)
    return R.swiglu(gate, up)


def apply_rope(x: Tensor, cos: Tensor, sin: Tensor) -> Tensor:
    if _cuda(x):
        return _ck().apply_rope(x, cos, sin)
    return R.apply_rope(x, cos, sin)


def l2_norm(x: Tensor, eps: float = 1e-6) -> Tensor:
    return R.l2_norm(x, eps)


def gka_prepare(q: Tensor, k: Tensor, v: Tensor, beta: Optional[Tensor] = None, eps: float = 1e-6):
    """Gated KalmaNet inputs: unit-norm ``q``, ``k`` scaled by ``beta + eps`` after normalisation, ``v`` scaled by
    ``beta + eps`` (one fused kernel each way on the GPU)."""
    if _cuda(q, k, v):
        return _ck().gka_prepare(q, k, v, beta, eps)
    return R.gka_prepare(q, k, v, beta, eps)


def gdn_gating(a: Tensor, b: Tensor, A_log: Tensor, dt_bias: Tensor, beta_scale: float = 1.0) -> Tuple[Tensor, Tensor]:
    if _cuda(a, b):
        return _ck().gdn_gating(a, b, A_log, dt_bias, beta_scale)
    return R.gdn_gating(a, b, A_log, dt_bias, beta_scale)


def causal_conv1d(x: Tensor, weight: Tensor, bias: Optional[Tensor] = None, activation: Optional[str] = "silu",
                  initial_state: Optional[Tensor] = None, return_final_state: bool = False):
    if _cuda(x):
        return _ck().causal_conv1d(x, weight, bias, activation, initial_state, return_final_state)
    return R.causal_conv1d(x, weight, bias, activation, initial_state, return_final_state)


def causal_conv1d_update(x: Tensor, conv_state: Tensor, weight: Tensor, bias: Optional[Tensor] = None,
                         activation: Optional[str] = "silu") -> Tuple[Tensor, Tensor]:
    if _cuda(x):
        return _ck().causal_conv1d_update(x, conv_state, weight, bias, activation)
    return R.causal_conv1d_update(x, conv_state, weight, bias, activation)


# -- linear / loss ----------------------------------------------------------------------------
def linear(x: Tensor, weight: Tensor, bias: Optional[Tensor] = None) -> Tensor:
    """``x @ weight.T + bias``.  Plain projections use the vendor GEMM through PyTorch; the
    tcgen05 GEMM of this library (``ops.gemm``) backs the fused paths."""
    return torch.nn.functional.linear(x, weight, bias)


def linear_cross_entropy(hidden: Tensor, weight: Tensor, labels: Tensor, ignore_index: int = -100,
                         chunk: int = 8192) -> Tuple[Tensor, Tensor]:
    """Sum of token cross entropies of ``hidden @ weight.T`` and the number of valid labels,
    without materialising the full logit matrix."""
    if _cuda(hidden, weight):
        return _ck().linear_cross_entropy(hidden, weight, labels, ignore_index, chunk)
    return R.linear_cross_entropy(hidden, weight, labels, ignore_index, "sum", chunk)


# -- attention --------------------------------------------------------------------------------
def attention(q: Tensor, k: Tensor, v: Tensor, *, scale: Optional[float] = None, causal: bool = True,
              window: Optional[int] = None, hollow: Optional[int] = None, q_pos: Optional[Tensor] = None,
              k_pos: Optional[Tensor] = None, return_lse: bool = False):
    if _cuda(q, k, v):
        return _ck().attention(q, k, v, scale=scale, causal=causal, window=window, hollow=hollow, q_pos=q_pos,
                               k_pos=k_pos, return_lse=return_lse)
    return R.attention(q, k, v, scale=scale, causal=causal, window=window, hollow=hollow, q_pos=q_pos, k_pos=k_pos,
                       return_lse=return_lse)


def merge_attention_states(o1, lse1, o2, lse2):
    return R.merge_attention_states(o1, lse1, o2, lse2)


def qsparse_attention(q: Tensor, k: Tensor, v: Tensor, q_index: Tensor, *, scale: Optional[float] = None) -> Tensor:
    if _cuda(q, k, v):
        return _ck().qsparse_attention(q, k, v, q_index, scale)
    return R.qsparse_attention(q, k, v, q_index, scale=scale)
