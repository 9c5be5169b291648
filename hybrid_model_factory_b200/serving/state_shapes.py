"""Shapes and dtypes of the per-request recurrent state of every mixer type, for a given tensor-parallel size
(used to size the slot pool and by external cache managers).  Reference: ``primed_vllm/layers/primed_utils.py:14-256``.
"""
from __future__ import annotations

from typing import Dict, Tuple

import torch


def _div(n: int, tp: int, what: str) -> int:
    assert n % tp == 0, f"{what}={n} does not divide by the tensor-parallel size {tp}"
    return n // tp


def gdn_state_shapes(num_q_heads: int, num_k_heads: int, num_v_heads: int, head_dim: int, conv_size: int = 4,
                     tp: int = 1) -> Dict[str, Tuple[tuple, torch.dtype]]:
    H = _div(max(num_q_heads, num_k_heads, num_v_heads), tp, "heads")
    conv_dim = (_div(num_q_heads, tp, "q heads") + _div(num_k_heads, tp, "k heads") + _div(num_v_heads, tp, "v heads")) * head_dim
    return {"conv": ((conv_size - 1, conv_dim), torch.bfloat16), "recurrent": ((H, head_dim, head_dim), torch.float32)}


def gka_state_shapes(num_q_heads: int, num_k_heads: int, num_v_heads: int, head_dim: int, conv_size: int = 4,
                     use_v_conv: bool = True, tp: int = 1) -> Dict[str, Tuple[tuple, torch.dtype]]:
    H = _div(max(num_q_heads, num_k_heads, num_v_heads), tp, "heads")
    conv_dim = (_div(num_q_heads, tp, "q heads") + _div(num_k_heads, tp, "k heads")
                + (_div(num_v_heads, tp, "v heads") if use_v_conv else 0)) * head_dim
    return {"conv": ((conv_size - 1, conv_dim), torch.bfloat16), "h_kk": ((H, head_dim, head_dim), torch.float32),
            "h_kv": ((H, head_dim, head_dim), torch.float32)}


def mamba2_state_shapes(d_inner: int, d_xb: int, d_state: int, d_conv: int = 4, tp: int = 1):
    headdim = d_state
    nheads = _div(d_inner // headdim, tp, "heads")
    conv_dim = _div(d_inner, tp, "d_inner") + 2 * _div(d_xb, tp, "d_xb")
    return {"conv": ((d_conv - 1, conv_dim), torch.bfloat16), "ssm": ((nheads, headdim, d_state), torch.float32)}


def attention_kv_shape(num_kv_heads: int, head_dim: int, block_size: int, tp: int = 1):
    return {"k": ((block_size, _div(num_kv_heads, tp, "kv heads"), head_dim), torch.bfloat16),
            "v": ((block_size, _div(num_kv_heads, tp, "kv heads"), head_dim), torch.bfloat16)}


def bytes_per_request(shapes: Dict[str, Tuple[tuple, torch.dtype]]) -> int:
    total = 0
    for shape, dtype in shapes.values():
        n = 1
        for s in shape:
            n *= s
        total += n * torch.empty((), dtype=dtype).element_size()
    return total
