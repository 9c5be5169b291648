"""Gated KalmaNet mixer (ridge-regression memory with a Chebyshev solver).

``q, k`` = conv+SiLU then ``x / (||x|| + 1e-6)``; ``beta = sigmoid(W_b x + b)`` scales ``k`` and
``v`` by ``beta + 1e-6``; ``alpha = sigmoid(W_alpha x + b)``; ``g`` as in GDN and ``gk = g`` when
``use_forgetting_gate_kk``.  The core solves ``(H_t + lambda_t I) x_t = q_t`` with
``H_t = sum e^{G_t - G_i} k_i k_i^T`` and ``lambda_t = ridge * ||H_t||_F`` by ``num_iter`` Chebyshev
steps, mixes ``q' = q + alpha (x - q)`` and runs simple GLA with ``q'``; gated RMSNorm; ``o_proj``.
Two recurrent states ``h_kk`` and ``h_kv`` (both ``[H, D, D]``, fp32).
Reference: ``layers/gated_kalmanet/gka.py:77-686``.
"""
from __future__ import annotations

from dataclasses import asdict, dataclass
from typing import Optional

import torch
import torch.nn as nn

from ..ops import functional as F_ops
from ..ops import mixers
from ..parallel.sp import merge_segments, segments_with_halo
from .common import GatedRMSNorm, LinearLowRank, RMSNorm, ShortConvolution, init_dt_bias, input_proj, output_proj, repeat_heads


@dataclass
class GKAConfig:
    hidden_size: int
    head_dim: int
    num_q_heads: int
    num_k_heads: int
    num_v_heads: int
    use_alpha_connection: bool = True
    use_v_conv: bool = True
    use_forgetting_gate: bool = True
    gla_rescale: bool = True
    solver_type: str = "chebyshev"
    bp_lambda: bool = True
    num_iter: int = 30
    ridge_strength: float = 0.02
    use_gate: bool = True
    conv_size: int = 4
    norm_eps: float = 1e-6
    use_forgetting_gate_kk: bool = True
    use_beta_gate: bool = True
    chunk_size: int = 64
    kv_proj_rank: Optional[int] = None
    kv_learnable_residual: bool = False

    def to_dict(self):
        return asdict(self)

    @classmethod
    def from_dict(cls, d):
        if isinstance(d, cls):
            return d
        fields = cls.__dataclass_fields__
        return cls(**{k: v for k, v in dict(d).items() if k in fields})


def construct_gka_config(config, user: Optional[dict] = None) -> GKAConfig:
    """Head counts from the Transformer config (or Qwen3-Next ``linear_*`` fields) + user knobs
    (reference: ``layers/gated_kalmanet/gka_config.py:97-194``)."""
    user = user.to_dict() if hasattr(user, "to_dict") else dict(user or {})
    if getattr(config, "linear_num_value_heads", None) is not None:
        base = dict(hidden_size=config.hidden_size, head_dim=config.linear_key_head_dim,
                    num_q_heads=config.linear_num_key_heads, num_k_heads=config.linear_num_key_heads,
                    num_v_heads=config.linear_num_value_heads)
    else:
        nh = config.num_attention_heads
        base = dict(hidden_size=config.hidden_size,
                    head_dim=getattr(config, "head_dim", None) or config.hidden_size // nh, num_q_heads=nh,
                    num_k_heads=getattr(config, "num_key_value_heads", nh),
                    num_v_heads=getattr(config, "num_key_value_heads", nh))
    for k in GKAConfig.__dataclass_fields__:
        if k in user and user[k] is not None and k not in base:
            base[k] = user[k]
    return GKAConfig(**base)


class GatedKalmaNet(nn.Module):
    def __init__(self, hidden_size: int = 2048, head_dim: int = 128, num_q_heads: int = 16,
                 num_k_heads: Optional[int] = None, num_v_heads: Optional[int] = None, use_alpha_connection: bool = True,
                 use_v_conv: bool = True, use_forgetting_gate: bool = True, gla_rescale: bool = True,
                 solver_type: str = "chebyshev", bp_lambda: bool = True, num_iter: int = 30,
                 ridge_strength: float = 0.02, use_gate: bool = True, conv_size: int = 4, norm_eps: float = 1e-6,
                 use_forgetting_gate_kk: bool = True, use_beta_gate: bool = True, chunk_size: int = 64,
                 kv_proj_rank: Optional[int] = None, kv_learnable_residual: bool = False,
                 layer_idx: Optional[int] = None, **_):
        super().__init__()
        assert solver_type == "chebyshev", f"unknown GKA solver type {solver_type}"
        self.hidden_size, self.head_dim, self.layer_idx = hidden_size, head_dim, layer_idx
        self.num_q_heads = num_q_heads
        self.num_k_heads = num_k_heads if num_k_heads is not None else num_q_heads
        self.num_v_heads = num_v_heads if num_v_heads is not None else num_q_heads
        self.expanded_num_heads = H = max(self.num_q_heads, self.num_k_heads, self.num_v_heads)
        self.num_q_groups, self.num_k_groups = H // self.num_q_heads, H // self.num_k_heads
        self.num_v_groups = H // self.num_v_heads
        self.query_dim, self.key_dim = self.num_q_heads * head_dim, self.num_k_heads * head_dim
        self.value_dim, self.expanded_dim = self.num_v_heads * head_dim, H * head_dim
        self.use_alpha_connection, self.use_v_conv = use_alpha_connection, use_v_conv
        self.use_forgetting_gate, self.use_forgetting_gate_kk = use_forgetting_gate, use_forgetting_gate_kk
        self.use_beta_gate, self.use_gate = use_beta_gate, use_gate
        self.num_iter, self.ridge_strength, self.bp_lambda = num_iter, ridge_strength, bp_lambda
        self.chunk_size, self.conv_size = chunk_size, conv_size
        self.gla_scale = head_dim ** -0.5 if gla_rescale else 1.0
        self.sequence_parallel_group = None

        self.q_proj = nn.Linear(hidden_size, self.query_dim, bias=False)
        self.k_proj = nn.Linear(hidden_size, self.key_dim, bias=False)
        self.v_proj = nn.Linear(hidden_size, self.value_dim, bias=False)
        self.a_proj = nn.Linear(hidden_size, H, bias=False)
        if use_beta_gate:
            self.b_proj = nn.Linear(hidden_size, H, bias=True)
        if use_alpha_connection:
            self.alpha_proj = nn.Linear(hidden_size, H, bias=True)
        self.A_log = nn.Parameter(torch.log(torch.empty(H, dtype=torch.float32).uniform_(0, 16).clamp(min=1e-4)))
        self.A_log._no_weight_decay = True
        self.dt_bias = nn.Parameter(init_dt_bias(H))
        self.dt_bias._no_weight_decay = True
        self.q_conv1d = ShortConvolution(self.query_dim, conv_size)
        self.k_conv1d = ShortConvolution(self.key_dim, conv_size)
        if use_v_conv:
            self.v_conv1d = ShortConvolution(self.value_dim, conv_size)
        if use_gate:
            self.g_proj = nn.Linear(hidden_size, self.expanded_dim, bias=False)
            self.o_norm = GatedRMSNorm(head_dim, eps=norm_eps)
        else:
            self.o_norm = RMSNorm(head_dim, eps=norm_eps)
        self.o_proj = nn.Linear(self.expanded_dim, hidden_size, bias=False)
        self.kv_proj_rank, self.kv_learnable_residual = kv_proj_rank, kv_learnable_residual
        if kv_proj_rank is not None:
            self.proj_k = LinearLowRank(self.key_dim, self.expanded_dim, kv_proj_rank, nn.SiLU())
            self.proj_v = LinearLowRank(self.value_dim, self.expanded_dim, kv_proj_rank, nn.SiLU())
            if kv_learnable_residual:
                self.k_rep = nn.Parameter(torch.kron(torch.eye(self.num_k_heads), torch.ones(self.num_k_groups, 1)))
                self.v_rep = nn.Parameter(torch.kron(torch.eye(self.num_v_heads), torch.ones(self.num_v_groups, 1)))

    _expand_kv = None  # assigned below (shared with GatedDeltaNet)

    INPUT_PROJECTIONS = ("q_proj", "k_proj", "v_proj", "a_proj", "b_proj", "alpha_proj", "g_proj")
    OUTPUT_PROJECTION = "o_proj"

    def forward(self, hidden_states: torch.Tensor, past_key_values=None, use_cache: bool = False, **kwargs):
        sp = self.sequence_parallel_group
        B, T, _ = hidden_states.shape
        last = past_key_values.get_ssm(self.layer_idx) if past_key_values is not None else None
        q, k, v = (input_proj(self, n, hidden_states, kwargs) for n in ("q_proj", "k_proj", "v_proj"))
        new_conv = None
        if sp is not None and sp.size > 1:
            parts, convs = [q, k], [self.q_conv1d, self.k_conv1d]
            if self.use_v_conv:
                parts.append(v)
                convs.append(self.v_conv1d)
            x = torch.cat(parts, dim=-1)
            seg, halo = segments_with_halo(x, sp, self.conv_size - 1)
            w = torch.cat([c.weight for c in convs], dim=0).squeeze(1)
            x = merge_segments(F_ops.causal_conv1d(seg, w, None, "silu", halo), sp)
            outs = torch.split(x, [p.shape[-1] for p in parts], dim=-1)
            q, k = outs[0], outs[1]
            if self.use_v_conv:
                v = outs[2]
        else:
            cq, ck, cv = last["conv_state"] if last is not None else (None, None, None)
            want = use_cache or past_key_values is not None
            q, cq = self.q_conv1d(q, cq, want)
            k, ck = self.k_conv1d(k, ck, want)
            if self.use_v_conv:
                v, cv = self.v_conv1d(v, cv, want)
            new_conv = (cq, ck, cv)
        q = repeat_heads(q.reshape(B, T, self.num_q_heads, self.head_dim), self.num_q_groups)
        k, v = self._expand_kv(k, v)
        # unit-norm q and k, beta gate on k and v: one pass over the three tensors (`ops/cuda_ops.py::gka_prepare`)
        beta = torch.sigmoid(input_proj(self, "b_proj", hidden_states, kwargs)) if self.use_beta_gate else None
        q, k, v = F_ops.gka_prepare(q, k, v, beta, 1e-6)
        alpha = (torch.sigmoid(input_proj(self, "alpha_proj", hidden_states, kwargs))
                 if self.use_alpha_connection else None)
        if self.use_forgetting_gate:
            g = -self.A_log.float().exp() * torch.nn.functional.softplus(
                input_proj(self, "a_proj", hidden_states, kwargs).float() + self.dt_bias.float())
        else:
            g = torch.zeros(B, T, self.expanded_num_heads, device=q.device, dtype=torch.float32)
        gk = g if (self.use_forgetting_gate and self.use_forgetting_gate_kk) else None
        state0 = last["recurrent_state"] if last is not None else None
        num_iter = int(kwargs.get("num_iter", self.num_iter))
        o, state = mixers.gka(q, k, v, alpha, g, gk, scale=self.gla_scale, ridge_ratio=self.ridge_strength,
                              num_iter=num_iter, initial_state=state0, sp=sp, chunk_size=self.chunk_size,
                              recurrent=(T == 1 and not self.training))
        if past_key_values is not None:
            past_key_values.update_ssm(self.layer_idx, recurrent_state=state, conv_state=new_conv, offset=T)
        if self.use_gate:
            gate = input_proj(self, "g_proj", hidden_states, kwargs).view(B, T, self.expanded_num_heads, self.head_dim)
            o = self.o_norm(o.to(hidden_states.dtype), gate)
        else:
            o = self.o_norm(o.to(hidden_states.dtype))
        return output_proj(self, "o_proj", o.reshape(B, T, self.expanded_dim), kwargs), None, past_key_values


from .gdn import GatedDeltaNet as _GDN  # noqa: E402

GatedKalmaNet._expand_kv = _GDN._expand_kv


class GatedKalmaNetLayer(GatedKalmaNet):
    """Builds the mixer from ``config.gka_config`` (reference: ``layers/gated_kalmanet/modules.py:22-96``)."""

    def __init__(self, config, layer_idx: int):
        cfg = getattr(config, "gka_config", None)
        cfg = GKAConfig.from_dict(cfg) if cfg else construct_gka_config(config)
        super().__init__(layer_idx=layer_idx, **cfg.to_dict())
        overrides = getattr(config, "gka_overrides", None) or {}
        if "num_iter" in overrides:
            self.num_iter = int(overrides["num_iter"])
