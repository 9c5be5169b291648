"""Building blocks shared by all decoder families: RMSNorm, SwiGLU MLP, rotary tables,
low-rank linear.  Parameter names follow the HF checkpoints the reference project reads and
writes (``models/hybrid_qwen3/modeling_hybrid_qwen3.py:85-216``)."""
from __future__ import annotations

import math
from typing import Optional, Tuple

import torch
import torch.nn as nn

from ..ops import functional as F_ops
from ..ops import reference as R


class RMSNorm(nn.Module):
    def __init__(self, hidden_size: int, eps: float = 1e-6, zero_centered: bool = False):
        super().__init__()
        self.weight = nn.Parameter(torch.zeros(hidden_size) if zero_centered else torch.ones(hidden_size))
        self.variance_epsilon = eps
        self.zero_centered = zero_centered

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return F_ops.rms_norm(x, self.weight, self.variance_epsilon, self.zero_centered)

    def extra_repr(self):
        return f"{tuple(self.weight.shape)}, eps={self.variance_epsilon}"


class GatedRMSNorm(nn.Module):
    """Per-head RMSNorm fused with a SiLU gate (``rmsnorm(x) * w * silu(g)`` or, for Mamba2,
    ``rmsnorm(x * silu(g)) * w``)."""

    def __init__(self, dim: int, eps: float = 1e-5, norm_before_gate: bool = True):
        super().__init__()
        self.weight = nn.Parameter(torch.ones(dim))
        self.eps = eps
        self.norm_before_gate = norm_before_gate

    def forward(self, x: torch.Tensor, gate: Optional[torch.Tensor] = None) -> torch.Tensor:
        if gate is None:
            return F_ops.rms_norm(x, self.weight, self.eps)
        return F_ops.gated_rms_norm(x, gate, self.weight, self.eps, self.norm_before_gate)


class MLP(nn.Module):
    """SwiGLU feed-forward: ``down(silu(gate(x)) * up(x))``."""

    def __init__(self, hidden_size: int, intermediate_size: int, bias: bool = False):
        super().__init__()
        self.hidden_size, self.intermediate_size = hidden_size, intermediate_size
        self.gate_proj = nn.Linear(hidden_size, intermediate_size, bias=bias)
        self.up_proj = nn.Linear(hidden_size, intermediate_size, bias=bias)
        self.down_proj = nn.Linear(intermediate_size, hidden_size, bias=bias)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return self.down_proj(F_ops.swiglu(self.gate_proj(x), self.up_proj(x)))


class RotaryEmbedding(nn.Module):
    """cos/sin tables from explicit position ids (so zig-zag sharded sequences rotate by their
    true positions).  Supports the default and linear / dynamic-NTK scaling types."""

    def __init__(self, dim: int, theta: float = 1e6, scaling: Optional[dict] = None, max_position: int = 0):
        super().__init__()
        self.dim, self.theta, self.scaling, self.max_position = dim, theta, scaling or {}, max_position
        inv = 1.0 / (theta ** (torch.arange(0, dim, 2, dtype=torch.float32) / dim))
        kind = self.scaling.get("rope_type", self.scaling.get("type", "default"))
        factor = float(self.scaling.get("factor", 1.0))
        if kind == "linear":
            inv = inv / factor
        elif kind in ("dynamic", "ntk") and factor > 1.0:
            base = theta * factor ** (dim / max(dim - 2, 1))
            inv = 1.0 / (base ** (torch.arange(0, dim, 2, dtype=torch.float32) / dim))
        self.register_buffer("inv_freq", inv, persistent=False)

    @torch.no_grad()
    def forward(self, position_ids: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
        freqs = position_ids.float()[..., None] * self.inv_freq.float().to(position_ids.device)
        emb = torch.cat([freqs, freqs], dim=-1)
        return emb.cos(), emb.sin()


class LinearLowRank(nn.Module):
    """``B(act(A x))`` with ``B`` zero-initialised: a residual low-rank map used to expand K/V heads
    on top of a plain repeat (reference: ``layers/low_rank_linear.py:8-57``)."""

    def __init__(self, in_features: int, out_features: int, rank: int, act_fn: Optional[nn.Module] = None):
        super().__init__()
        self.A = nn.Linear(in_features, rank, bias=False)
        self.B = nn.Linear(rank, out_features, bias=False)
        self.act_fn = act_fn
        nn.init.zeros_(self.B.weight)
        self.B._keep_init = True  # survives the model-wide normal_ initialisation

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        h = self.A(x)
        if self.act_fn is not None:
            h = self.act_fn(h)
        return self.B(h)


class ShortConvolution(nn.Module):
    """Depthwise causal conv1d (kernel ``K``) + SiLU with cache / halo support.  ``weight`` has
    the HF layout ``[C, 1, K]`` so checkpoints of the reference project load unchanged."""

    def __init__(self, hidden_size: int, kernel_size: int = 4, bias: bool = False, activation: Optional[str] = "silu"):
        super().__init__()
        self.hidden_size, self.kernel_size, self.activation = hidden_size, kernel_size, activation
        self.weight = nn.Parameter(torch.empty(hidden_size, 1, kernel_size))
        self.bias = nn.Parameter(torch.zeros(hidden_size)) if bias else None
        bound = 1.0 / math.sqrt(kernel_size)
        nn.init.uniform_(self.weight, -bound, bound)

    def forward(self, x: torch.Tensor, cache: Optional[torch.Tensor] = None, output_final_state: bool = False):
        """``x [B, T, C]``; ``cache [B, K-1, C]`` holds the tokens preceding ``x``."""
        w = self.weight.squeeze(1)
        if x.shape[1] == 1 and cache is not None and not self.training:
            y, new = F_ops.causal_conv1d_update(x[:, 0], cache, w, self.bias, self.activation)
            return y[:, None], new
        res = F_ops.causal_conv1d(x, w, self.bias, self.activation, cache, output_final_state)
        if output_final_state:
            return res
        return res, None


def repeat_heads(x: torch.Tensor, n_rep: int) -> torch.Tensor:
    """``[B, T, H, D] -> [B, T, H*n_rep, D]`` with each head repeated consecutively."""
    if n_rep == 1:
        return x
    B, T, H, D = x.shape
    return x[:, :, :, None, :].expand(B, T, H, n_rep, D).reshape(B, T, H * n_rep, D)


def init_dt_bias(n: int, dt_min: float = 0.001, dt_max: float = 0.1, floor: float = 1e-4) -> torch.Tensor:
    dt = torch.exp(torch.rand(n) * (math.log(dt_max) - math.log(dt_min)) + math.log(dt_min)).clamp(min=floor)
    return dt + torch.log(-torch.expm1(-dt))
