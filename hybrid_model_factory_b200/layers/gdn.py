"""Gated DeltaNet mixer.

``q, k, v = silu(conv1d_4(W x))``; K/V heads expanded to ``H = max(Hq, Hk, Hv)``;
``beta = sigmoid(W_b x)`` (x2 with ``allow_neg_eigval``); ``g = -exp(A_log) softplus(W_gk x + dt_bias)``;
chunked gated delta rule with L2-normalised q, k; gated per-head RMSNorm; ``o_proj``.
Parameter names and shapes match the reference layer (``layers/gated_deltanet/gdn.py:58-236``)
so its checkpoints load unchanged.

Sequence parallelism: projections run on local tokens only; the convolution gets a 3-token
halo of the pre-convolution activations and the recurrence receives its incoming state through
``ops.scan.ssm_scan`` (the reference gathers the whole sequence on every rank instead,
``gdn.py:369-386``).
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
class GDNConfig:
    hidden_size: int
    head_dim: int
    num_q_heads: int
    num_k_heads: int
    num_v_heads: int
    use_gate: bool = True
    use_short_conv: bool = True
    allow_neg_eigval: bool = False
    conv_size: int = 4
    conv_bias: bool = False
    norm_eps: float = 1e-5
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


def construct_gdn_config(config, user: Optional[dict] = None) -> GDNConfig:
    """Derives head counts from a Transformer config (attention -> GDN) or from Qwen3-Next style
    ``linear_*`` fields (reference: ``layers/gated_deltanet/gdn_config.py:71-149``)."""
    user = dict(user or {})
    if hasattr(user, "to_dict"):
        user = user.to_dict()
    if getattr(config, "linear_num_value_heads", None) is not None:
        base = dict(hidden_size=config.hidden_size, head_dim=config.linear_key_head_dim,
                    num_q_heads=config.linear_num_key_heads, num_k_heads=config.linear_num_key_heads,
                    num_v_heads=config.linear_num_value_heads,
                    conv_size=getattr(config, "linear_conv_kernel_dim", 4),
                    # released Gated-DeltaNet checkpoints norm their head outputs with the model's own epsilon
                    norm_eps=float(getattr(config, "rms_norm_eps", 1e-6)))
    else:
        nh = config.num_attention_heads
        base = dict(hidden_size=config.hidden_size,
                    head_dim=getattr(config, "head_dim", None) or config.hidden_size // nh,
                    num_q_heads=nh, num_k_heads=getattr(config, "num_key_value_heads", nh),
                    num_v_heads=getattr(config, "num_key_value_heads", nh))
    for k in ("use_gate", "use_short_conv", "allow_neg_eigval", "conv_size", "conv_bias", "norm_eps", "kv_proj_rank",
              "kv_learnable_residual"):
        if k in user and user[k] is not None:
            base[k] = user[k]
    return GDNConfig(**base)


class GatedDeltaNet(nn.Module):
    def __init__(self, hidden_size: int = 2048, head_dim: int = 128, num_q_heads: int = 16,
                 num_k_heads: Optional[int] = None, num_v_heads: Optional[int] = None, use_gate: bool = True,
                 use_short_conv: bool = True, allow_neg_eigval: bool = False, conv_size: int = 4, conv_bias: bool = False,
                 layer_idx: Optional[int] = None, norm_eps: float = 1e-5, kv_proj_rank: Optional[int] = None,
                 kv_learnable_residual: bool = False, chunk_size: int = 64, **_):
        super().__init__()
        self.hidden_size, self.head_dim, self.layer_idx = hidden_size, head_dim, layer_idx
        self.num_q_heads = num_q_heads
        self.num_k_heads = num_k_heads if num_k_heads is not None else num_q_heads
        self.num_v_heads = num_v_heads if num_v_heads is not None else num_q_heads
        self.expanded_num_heads = max(self.num_q_heads, self.num_k_heads, self.num_v_heads)
        self.num_q_groups = self.expanded_num_heads // self.num_q_heads
        self.num_k_groups = self.expanded_num_heads // self.num_k_heads
        self.num_v_groups = self.expanded_num_heads // self.num_v_heads
        self.query_dim = self.num_q_heads * head_dim
        self.key_dim = self.num_k_heads * head_dim
        self.value_dim = self.num_v_heads * head_dim
        self.expanded_dim = self.expanded_num_heads * head_dim
        self.use_gate, self.use_short_conv, self.allow_neg_eigval = use_gate, use_short_conv, allow_neg_eigval
        self.conv_size, self.conv_bias, self.chunk_size = conv_size, conv_bias, chunk_size
        self.sequence_parallel_group = None
        H = self.expanded_num_heads

        self.q_proj = nn.Linear(hidden_size, self.query_dim, bias=False)
        self.k_proj = nn.Linear(hidden_size, self.key_dim, bias=False)
        self.v_proj = nn.Linear(hidden_size, self.value_dim, bias=False)
        self.b_proj = nn.Linear(hidden_size, H, bias=False)
        self.gk_proj = nn.Linear(hidden_size, H, bias=False)
        self.A_log = nn.Parameter(torch.log(torch.empty(H, dtype=torch.float32).uniform_(0, 16).clamp(min=1e-4)))
        self.A_log._no_weight_decay = True
        self.dt_bias = nn.Parameter(init_dt_bias(H))
        self.dt_bias._no_weight_decay = True
        if use_short_conv:
            self.q_conv1d = ShortConvolution(self.query_dim, conv_size, conv_bias)
            self.k_conv1d = ShortConvolution(self.key_dim, conv_size, conv_bias)
            self.v_conv1d = ShortConvolution(self.value_dim, conv_size, conv_bias)
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

    # ------------------------------------------------------------------------------
    def _expand_kv(self, k: torch.Tensor, v: torch.Tensor):
        """``[B,T,Hk*D] -> [B,T,H,D]``: plain repeat, or repeat / learnable mix plus a low-rank term
        (reference: ``gdn.py:240-300``)."""
        B, T, _ = k.shape
        D, H = self.head_dim, self.expanded_num_heads
        kh, vh = k.view(B, T, self.num_k_heads, D), v.view(B, T, self.num_v_heads, D)
        if self.kv_proj_rank is None:
            return repeat_heads(kh, self.num_k_groups), repeat_heads(vh, self.num_v_groups)
        if self.kv_learnable_residual:
            k_res = torch.einsum("eh,bthd->bted", self.k_rep.to(k.dtype), kh)
            v_res = torch.einsum("eh,bthd->bted", self.v_rep.to(v.dtype), vh)
        else:
            k_res, v_res = repeat_heads(kh, self.num_k_groups), repeat_heads(vh, self.num_v_groups)
        return k_res + self.proj_k(k).view(B, T, H, D), v_res + self.proj_v(v).view(B, T, H, D)

    INPUT_PROJECTIONS, OUTPUT_PROJECTION = ("q_proj", "k_proj", "v_proj", "gk_proj", "b_proj", "g_proj"), "o_proj"

    def forward(self, hidden_states: torch.Tensor, past_key_values=None, use_cache: bool = False, **kwargs):
        sp = self.sequence_parallel_group
        B, T, _ = hidden_states.shape
        last = past_key_values.get_ssm(self.layer_idx) if past_key_values is not None else None
        q, k, v = (input_proj(self, n, hidden_states, kwargs) for n in ("q_proj", "k_proj", "v_proj"))
        new_conv = None
        if self.use_short_conv:
            if sp is not None and sp.size > 1:
                qkv = torch.cat([q, k, v], dim=-1)
                seg, halo = segments_with_halo(qkv, sp, self.conv_size - 1)
                w = torch.cat([self.q_conv1d.weight, self.k_conv1d.weight, self.v_conv1d.weight], dim=0).squeeze(1)
                bias = None
                if self.conv_bias:
                    bias = torch.cat([self.q_conv1d.bias, self.k_conv1d.bias, self.v_conv1d.bias])
                qkv = merge_segments(F_ops.causal_conv1d(seg, w, bias, "silu", halo), sp)
                q, k, v = torch.split(qkv, [self.query_dim, self.key_dim, self.value_dim], dim=-1)
            else:
                cq, ck, cv = last["conv_state"] if last is not None else (None, None, None)
                want = use_cache or past_key_values is not None
                q, cq = self.q_conv1d(q, cq, want)
                k, ck = self.k_conv1d(k, ck, want)
                v, cv = self.v_conv1d(v, cv, want)
                new_conv = (cq, ck, cv)
        q = q.reshape(B, T, self.num_q_heads, self.head_dim)
        k, v = self._expand_kv(k, v)
        q = repeat_heads(q, self.num_q_groups)
        g, beta = F_ops.gdn_gating(input_proj(self, "gk_proj", hidden_states, kwargs),
                                   input_proj(self, "b_proj", hidden_states, kwargs), self.A_log, self.dt_bias,
                                   2.0 if self.allow_neg_eigval else 1.0)
        state0 = last["recurrent_state"] if last is not None else None
        o, state = mixers.gated_delta_rule(q, k, v, g, beta, initial_state=state0, sp=sp, chunk_size=self.chunk_size,
                                           recurrent=(T == 1 and not self.training))
        if past_key_values is not None:
            transition = None
            if getattr(past_key_values, "cache_transitions", False):
                # the recurrence is affine in the state: with v = 0 and S_0 = I the final state is the transition
                eye = torch.eye(self.head_dim, device=q.device, dtype=torch.float32).expand(
                    B, self.expanded_num_heads, -1, -1).contiguous()
                _, transition = mixers.gated_delta_rule(q, k, torch.zeros_like(k), g, beta, initial_state=eye,
                                                        chunk_size=self.chunk_size, recurrent=(T == 1))
            extra = {} if transition is None else {"transition": transition}
            past_key_values.update_ssm(self.layer_idx, recurrent_state=state, conv_state=new_conv, offset=T, **extra)
        if self.use_gate:
            gate = input_proj(self, "g_proj", hidden_states, kwargs).view(B, T, self.expanded_num_heads, self.head_dim)
            o = self.o_norm(o.to(hidden_states.dtype), gate)
        else:
            o = self.o_norm(o.to(hidden_states.dtype))
        return output_proj(self, "o_proj", o.reshape(B, T, self.expanded_dim), kwargs), None, past_key_values


class GatedDeltaNetLayer(GatedDeltaNet):
    """Builds the mixer from ``config.gdn_config`` (reference: ``layers/gated_deltanet/modules.py:22-96``)."""

    def __init__(self, config, layer_idx: int):
        cfg = getattr(config, "gdn_config", None)
        cfg = GDNConfig.from_dict(cfg) if cfg else construct_gdn_config(config)
        super().__init__(layer_idx=layer_idx, **cfg.to_dict())
