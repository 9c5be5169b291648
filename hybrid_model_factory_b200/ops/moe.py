"""Mixture-of-experts ops: softmax top-k router and routed SwiGLU experts.

``experts_forward`` sorts the (token, expert) assignments by expert, runs every expert on its
contiguous token group and scatters the weighted results back (a grouped GEMM; the reference
project loops over hit experts with two ``F.linear`` calls and ``index_add_``,
``models/hybrid_qwen3_moe/modeling_hybrid_qwen3_moe.py:329-365``).  With an expert-parallel
context the experts are sharded over ranks and tokens are exchanged by all-to-all
(``parallel/ep.py``).
"""
from __future__ import annotations

from typing import Tuple

import torch
import torch.nn.functional as F

from . import _lib
from . import reference as R

Tensor = torch.Tensor


def router(logits: Tensor, top_k: int, norm_topk_prob: bool = True) -> Tuple[Tensor, Tensor]:
    return R.moe_router(logits, top_k, norm_topk_prob)


def grouped_swiglu_experts(x_sorted: Tensor, counts: Tensor, w_gate_up: Tensor, w_down: Tensor) -> Tensor:
    """``x_sorted [N, Dm]`` holds the tokens of expert 0, then expert 1, ... (``counts [E]``).
    Returns ``down_e(silu(gate_e x) * up_e x)`` for each row."""
    if _lib.use_cuda_kernels(x_sorted, w_gate_up) and hasattr(_lib.kernels(), "hmf_grouped_gemm_bf16"):
        from . import cuda_ops
        return cuda_ops.grouped_swiglu_experts(x_sorted, counts, w_gate_up, w_down)
    out = torch.empty(x_sorted.shape[0], w_down.shape[1], dtype=x_sorted.dtype, device=x_sorted.device)
    start = 0
    for e, n in enumerate(counts.tolist()):
        if n == 0:
            continue
        xs = x_sorted[start:start + n]
        h = F.linear(xs, w_gate_up[e])
        g, u = h.chunk(2, dim=-1)
        out[start:start + n] = F.linear(F.silu(g) * u, w_down[e])
        start += n
    return out


def experts_forward(x: Tensor, w_gate_up: Tensor, w_down: Tensor, weights: Tensor, indices: Tensor,
                    ep=None, fused=None) -> Tensor:
    """``x [T, Dm]``, routing ``weights, indices [T, k]`` -> ``[T, Dm]``.  ``fused`` (a
    ``parallel.ep_fused.FusedExpertParallel``) runs the tcgen05 grouped GEMMs, with the expert-parallel all-to-all
    folded into them, whenever no gradient is needed."""
    if (fused is not None and not torch.is_grad_enabled() and x.is_cuda and x.dtype == torch.bfloat16
            and indices.numel() <= fused.max_send):
        return fused.forward(x, weights, indices, w_gate_up, w_down)
    if ep is not None and ep.size > 1:
        from ..parallel.ep import ep_experts_forward
        return ep_experts_forward(x, w_gate_up, w_down, weights, indices, ep)
    T, k = indices.shape
    E = w_gate_up.shape[0]
    flat_e = indices.reshape(-1)
    order = torch.argsort(flat_e, stable=True)
    token_of = order // k
    counts = torch.bincount(flat_e, minlength=E)
    y = grouped_swiglu_experts(x[token_of], counts, w_gate_up, w_down)
    y = y * weights.reshape(-1)[order][:, None].to(y.dtype)
    out = torch.zeros_like(x)
    out.index_add_(0, token_of, y)
    return out
