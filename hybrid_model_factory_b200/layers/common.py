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


def rope_inverse_frequencies(dim: int, theta: float, scaling: Optional[dict], max_position: int = 0):
    """``(inv_freq [dim/2], attention_factor)`` for the RoPE variants of the HF configuration format
    (``rope_scaling`` / ``rope_parameters`` with ``rope_type`` in default | linear | dynamic | yarn | llama3 | longrope;
    the same formulas as ``transformers.modeling_rope_utils.ROPE_INIT_FUNCTIONS``, which the reference's rotary module
    dispatches to, ``modeling_hybrid_qwen3.py:121-183``)."""
    import math
    scaling = scaling or {}
    kind = scaling.get("rope_type", scaling.get("type", "default"))
    factor = float(scaling.get("factor", 1.0))
    exps = torch.arange(0, dim, 2, dtype=torch.float32) / dim
    inv = 1.0 / (theta ** exps)
    att = 1.0
    if kind == "linear":
        inv = inv / factor
    elif kind in ("dynamic", "ntk") and factor > 1.0:
        inv = 1.0 / ((theta * factor ** (dim / max(dim - 2, 1))) ** exps)
    elif kind == "llama3":
        lo = float(scaling.get("low_freq_factor", 1.0))
        hi = float(scaling.get("high_freq_factor", 4.0))
        old = float(scaling.get("original_max_position_embeddings", max_position or 8192))
        wavelen = 2 * math.pi / inv
        smooth = ((old / wavelen) - lo) / max(hi - lo, 1e-9)
        mid = (1 - smooth) * inv / factor + smooth * inv
        inv = torch.where(wavelen > old / lo, inv / factor, torch.where(wavelen < old / hi, inv, mid))
    elif kind == "yarn":
        old = float(scaling.get("original_max_position_embeddings", max_position or 4096))
        beta_fast, beta_slow = float(scaling.get("beta_fast", 32)), float(scaling.get("beta_slow", 1))

        def correction_dim(rotations):
            return dim * math.log(old / (rotations * 2 * math.pi)) / (2 * math.log(theta))
        low, high = correction_dim(beta_fast), correction_dim(beta_slow)
        if scaling.get("truncate", True):
            low, high = math.floor(low), math.ceil(high)
        low, high = max(low, 0), min(high, dim - 1)
        ramp = ((torch.arange(dim // 2, dtype=torch.float32) - low) / max(high - low, 1e-3)).clamp(0, 1)
        extrapolation = 1 - ramp
        inv = inv / factor * (1 - extrapolation) + inv * extrapolation

        def mscale(weight=1.0):
            return 1.0 if factor <= 1 else 0.1 * weight * math.log(factor) + 1.0
        if scaling.get("attention_factor"):
            att = float(scaling["attention_factor"])
        elif scaling.get("mscale") and scaling.get("mscale_all_dim"):      # ratio of the two magnitude corrections
            att = mscale(float(scaling["mscale"])) / mscale(float(scaling["mscale_all_dim"]))
        else:
            att = mscale()
    elif kind == "longrope":
        old = float(scaling.get("original_max_position_embeddings", max_position or 4096))
        ext = torch.tensor(scaling.get("long_factor" if max_position > old else "short_factor"), dtype=torch.float32)
        inv = 1.0 / (ext * theta ** exps)
        f = max(max_position / old, 1.0)
        att = float(scaling.get("attention_factor") or (math.sqrt(1 + math.log(f) / math.log(old)) if f > 1 else 1.0))
    elif kind not in ("default", "mrope"):
        raise ValueError(f"unknown rope_type {kind!r}")
    return inv, att


class RotaryEmbedding(nn.Module):
    """cos/sin tables from explicit position ids (so zig-zag sharded sequences rotate by their
    true positions).  Scaling types: default, linear, dynamic-NTK, llama3, yarn, longrope."""

    def __init__(self, dim: int, theta: float = 1e6, scaling: Optional[dict] = None, max_position: int = 0):
        super().__init__()
        self.dim, self.theta, self.scaling, self.max_position = dim, theta, scaling or {}, max_position
        inv, self.attention_factor = rope_inverse_frequencies(dim, theta, self.scaling, max_position)
        self.register_buffer("inv_freq", inv, persistent=False)

    def _apply(self, fn, recurse=True):
        """The frequencies stay fp32 whatever the model is cast to (rounded to bf16 they are off by up to 0.4 %, which
        at a distance of a few thousand tokens is a phase error of several radians against the trained model), and
        they are recomputed rather than moved, so a model built on the meta device gets them too."""
        super()._apply(fn, recurse)
        inv, _ = rope_inverse_frequencies(self.dim, self.theta, self.scaling, self.max_position)
        self.inv_freq = inv.to(self.inv_freq.device)
        return self

    @torch.no_grad()
    def forward(self, position_ids: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
        freqs = position_ids.float()[..., None] * self.inv_freq.float().to(position_ids.device)
        emb = torch.cat([freqs, freqs], dim=-1)
        if self.attention_factor != 1.0:                      # yarn / longrope scale the rotated vectors
            return emb.cos() * self.attention_factor, emb.sin() * self.attention_factor
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


def input_proj(module: nn.Module, name: str, x: torch.Tensor, kw: Optional[dict]) -> torch.Tensor:
    """Projection ``name`` of a mixer applied to the layer input ``x``, or its precomputed result when the caller
    (a packed prefill: ``models/modeling_hybrid.py::DecoderLayer``) already applied it to the whole packed row and
    passes this sample's slice in ``kw["pre_proj"]``."""
    pre = None if kw is None else kw.get("pre_proj")
    if pre is not None and name in pre:
        return pre[name]
    return getattr(module, name)(x)


def output_proj(module: nn.Module, name: str, y: torch.Tensor, kw: Optional[dict]) -> torch.Tensor:
    """Output projection of a mixer, left to the caller when ``kw["defer_out_proj"]`` is set (one GEMM over the
    packed row instead of one per sample)."""
    if kw is not None and kw.get("defer_out_proj"):
        return y
    return getattr(module, name)(y)


def repeat_heads(x: torch.Tensor, n_rep: int) -> torch.Tensor:
    """``[B, T, H, D] -> [B, T, H*n_rep, D]`` with each head repeated consecutively."""
    if n_rep == 1:
        return x
    B, T, H, D = x.shape
    return x[:, :, :, None, :].expand(B, T, H, n_rep, D).reshape(B, T, H * n_rep, D)


def init_dt_bias(n: int, dt_min: float = 0.001, dt_max: float = 0.1, floor: float = 1e-4) -> torch.Tensor:
    dt = torch.exp(torch.rand(n) * (math.log(dt_max) - math.log(dt_min)) + math.log(dt_min)).clamp(min=floor)
    return dt + torch.log(-torch.expm1(-dt))
