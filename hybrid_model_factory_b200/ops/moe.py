"""Mixture-of-experts ops: softmax top-k router and routed SwiGLU experts.

``experts_forward`` sorts the (token, expert) assignments by expert and scatters the weighted results back.  On
the GPU (bf16) every expert's rows are padded to whole 128-row tiles and all experts run in ONE grouped tcgen05 GEMM
per projection, forward and backward (``csrc/kernels/gemm_bf16.cu``, grouped modes); the reference project loops over
hit experts with two ``F.linear`` calls and ``index_add_``
(``models/hybrid_qwen3_moe/modeling_hybrid_qwen3_moe.py:329-365``), which is the formulation kept for CPU / fp32.  With an expert-parallel
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


TILE = 128      # rows per GEMM tile: every expert's group of rows is padded to a whole number of tiles


def padded_layout(flat_expert: Tensor, num_experts: int):
    """Row layout of the grouped GEMMs for assignments ``flat_expert [A]`` (expert of every (token, slot) pair).

    The pairs are sorted by expert and every expert's group is padded to whole 128-row tiles, so that a GEMM tile
    never straddles two experts.  Everything is computed on the device with static shapes (no host synchronisation):
    the row count is the upper bound ``R = roundup(A, 128) + 128 * E`` and unused tiles are marked ``-1``.

    Returns ``(order [A], dst_rows [A], mtile_group [R/128] int32, k_offsets [E+1] int32, R)``: pair ``order[i]``
    goes to row ``dst_rows[i]``."""
    A = flat_expert.numel()
    E = num_experts
    R = (A + TILE - 1) // TILE * TILE + TILE * E
    order = torch.argsort(flat_expert, stable=True)
    sorted_e = flat_expert[order]
    # (not torch.bincount: on the GPU it reads the largest value back to the host to size its result)
    counts = torch.zeros(E, dtype=torch.long, device=flat_expert.device).scatter_add_(
        0, flat_expert.long(), torch.ones_like(flat_expert, dtype=torch.long))
    padded = (counts + TILE - 1) // TILE * TILE
    pad_end = torch.cumsum(padded, 0)
    pad_start = pad_end - padded
    start = torch.cumsum(counts, 0) - counts
    dst_rows = pad_start[sorted_e] + (torch.arange(A, device=flat_expert.device) - start[sorted_e])
    tiles = torch.arange(R // TILE, device=flat_expert.device)
    group = torch.searchsorted(pad_end // TILE, tiles, right=True)
    mtile_group = torch.where(tiles < pad_end[-1] // TILE, group, torch.full_like(group, -1)).to(torch.int32)
    k_offsets = torch.cat([pad_start[:1] * 0, pad_end]).to(torch.int32)
    return order, dst_rows, mtile_group, k_offsets, R


def _grouped_gemm(a: Tensor, w: Tensor, mtile_group: Tensor, b_mn_major: bool = False) -> Tensor:
    """``a [R, K]`` times the stacked expert matrices ``w`` (``[E, N, K]``, or ``[E, K, N]`` with ``b_mn_major``)."""
    import ctypes
    R, K = a.shape
    E = w.shape[0]
    N = w.shape[2] if b_mn_major else w.shape[1]
    out = torch.zeros(R, N, device=a.device, dtype=a.dtype)     # rows of unused tiles stay zero
    w2 = w.reshape(E * w.shape[1], w.shape[2])
    _lib.check(_lib.kernels().hmf_grouped_gemm_bf16(
        _lib.ptr(a), _lib.ptr(w2), _lib.ptr(out), _lib.ptr(mtile_group), ctypes.c_int(R), ctypes.c_int(N),
        ctypes.c_int(K), ctypes.c_int(E), ctypes.c_longlong(a.stride(0)), ctypes.c_longlong(w2.stride(0)),
        ctypes.c_longlong(out.stride(0)), ctypes.c_int(int(b_mn_major)), _lib.stream_ptr(a.device)), "grouped_gemm")
    return out


def _grouped_wgrad(dy: Tensor, a: Tensor, k_offsets: Tensor, E: int) -> Tensor:
    """``dW[e] = dy[rows of e]^T a[rows of e]`` for every expert: ``[E, N, K]``."""
    import ctypes
    R, N = dy.shape
    K = a.shape[1]
    out = torch.empty(E, N, K, device=a.device, dtype=a.dtype)
    _lib.check(_lib.kernels().hmf_grouped_gemm_wgrad_bf16(
        _lib.ptr(dy), _lib.ptr(a), _lib.ptr(out), _lib.ptr(k_offsets), ctypes.c_int(R), ctypes.c_int(N),
        ctypes.c_int(K), ctypes.c_int(E), ctypes.c_longlong(dy.stride(0)), ctypes.c_longlong(a.stride(0)),
        ctypes.c_longlong(K), _lib.stream_ptr(a.device)), "grouped_gemm_wgrad")
    return out


class _GroupedSwiGLUExperts(torch.autograd.Function):
    """``down_e(silu(gate_e x) * up_e x)`` over rows grouped by expert: two grouped tcgen05 GEMMs forward, two
    grouped input-gradient GEMMs and two grouped weight-gradient GEMMs backward (one launch each for all experts)."""

    @staticmethod
    def forward(ctx, x_pad, w_gate_up, w_down, mtile_group, k_offsets):
        from . import cuda_ops
        h = _grouped_gemm(x_pad, w_gate_up, mtile_group)                       # [R, 2F]
        F_ = h.shape[1] // 2
        act = cuda_ops.swiglu(h[:, :F_], h[:, F_:])                            # [R, F]
        y = _grouped_gemm(act, w_down, mtile_group)                            # [R, Dm]
        ctx.save_for_backward(x_pad, h, act, w_gate_up, w_down, mtile_group, k_offsets)
        return y

    @staticmethod
    def backward(ctx, dy):
        from . import cuda_ops
        x_pad, h, act, w_gate_up, w_down, mtile_group, k_offsets = ctx.saved_tensors
        E = w_down.shape[0]
        dy = dy.contiguous()
        F_ = h.shape[1] // 2
        d_act = _grouped_gemm(dy, w_down, mtile_group, b_mn_major=True)        # [R, F]  (w_down is [E, Dm, F])
        d_wd = _grouped_wgrad(dy, act, k_offsets, E) if ctx.needs_input_grad[2] else None
        dg, du = cuda_ops.swiglu_backward(h[:, :F_], h[:, F_:], d_act)
        dh = torch.cat([dg, du], dim=1)
        dx = _grouped_gemm(dh, w_gate_up, mtile_group, b_mn_major=True) if ctx.needs_input_grad[0] else None
        d_wgu = _grouped_wgrad(dh, x_pad, k_offsets, E) if ctx.needs_input_grad[1] else None
        return dx, d_wgu, d_wd, None, None


def grouped_experts_available(x: Tensor, w_gate_up: Tensor, w_down: Tensor) -> bool:
    Dm, F2 = w_gate_up.shape[2], w_gate_up.shape[1]
    return (_lib.use_cuda_kernels(x, w_gate_up) and x.dtype == torch.bfloat16 and w_gate_up.dtype == torch.bfloat16
            and Dm % 64 == 0 and F2 % 128 == 0 and w_gate_up.is_contiguous() and w_down.is_contiguous())


def grouped_swiglu_experts(x_sorted: Tensor, counts: Tensor, w_gate_up: Tensor, w_down: Tensor) -> Tensor:
    """Reference formulation (CPU, fp32, odd sizes): ``x_sorted [N, Dm]`` holds the tokens of expert 0, then expert
    1, ... (``counts [E]``); one pair of matrix products per expert that has tokens."""
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


def experts_rows(rows: Tensor, expert_of_row: Tensor, w_gate_up: Tensor, w_down: Tensor) -> Tensor:
    """``rows [A, Dm]``, each to be processed by expert ``expert_of_row [A]``: returns the expert outputs in the same
    row order."""
    E = w_gate_up.shape[0]
    if grouped_experts_available(rows, w_gate_up, w_down):
        # bf16 on the GPU: grouped GEMMs over a padded row layout, no per-expert loop and no host synchronisation
        order, dst_rows, mtile_group, k_offsets, R = padded_layout(expert_of_row, E)
        x_pad = torch.zeros(R, rows.shape[1], device=rows.device, dtype=rows.dtype).index_copy(0, dst_rows, rows[order])
        y_pad = _GroupedSwiGLUExperts.apply(x_pad, w_gate_up, w_down, mtile_group, k_offsets)
        return torch.empty_like(rows).index_copy(0, order, y_pad[dst_rows])
    order = torch.argsort(expert_of_row, stable=True)
    counts = torch.bincount(expert_of_row, minlength=E)
    y = grouped_swiglu_experts(rows[order], counts, w_gate_up, w_down)
    return torch.empty_like(y).index_copy(0, order, y)


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
    y = experts_rows(x.repeat_interleave(k, dim=0), indices.reshape(-1), w_gate_up, w_down)
    return (y.view(T, k, -1) * weights[..., None].to(y.dtype)).sum(1)
