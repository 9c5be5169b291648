"""Softmax attention layers: full GQA attention (Qwen3 / Qwen2 / Llama / Ministral flavours),
sliding-window attention (``SWA``) with sequence-parallel halo, and the gated attention of
Qwen3-Next (``q_proj`` emits ``[q, gate]``, output multiplied by ``sigmoid(gate)``, partial rotary).

Reference behaviour: ``models/hybrid_qwen3/modeling_hybrid_qwen3.py:257-421`` and
``models/qwen3_next_hmf/modeling_qwen3_next_hmf.py:233-310``.
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch
import torch.nn as nn

from ..ops import functional as F_ops
from ..parallel.cp_attention import cp_attention
from ..parallel.sp import halo_exchange
from .common import RMSNorm, input_proj, output_proj


class Attention(nn.Module):
    def __init__(self, config, layer_idx: int, *, sliding_window: Optional[int] = None, gated: bool = False):
        super().__init__()
        self.config, self.layer_idx = config, layer_idx
        self.hidden_size = config.hidden_size
        self.num_heads = config.num_attention_heads
        self.num_kv_heads = getattr(config, "num_key_value_heads", self.num_heads)
        self.head_dim = getattr(config, "head_dim", None) or self.hidden_size // self.num_heads
        self.scaling = self.head_dim ** -0.5
        self.sliding_window = sliding_window
        self.gated = gated
        self.sequence_parallel_group = None
        qkv_bias = bool(getattr(config, "attention_bias", False) or getattr(config, "qkv_bias", False))
        o_bias = bool(getattr(config, "attention_bias", False)) and not getattr(config, "qkv_bias", False)
        q_out = self.num_heads * self.head_dim * (2 if gated else 1)
        self.q_proj = nn.Linear(self.hidden_size, q_out, bias=qkv_bias)
        self.k_proj = nn.Linear(self.hidden_size, self.num_kv_heads * self.head_dim, bias=qkv_bias)
        self.v_proj = nn.Linear(self.hidden_size, self.num_kv_heads * self.head_dim, bias=qkv_bias)
        self.o_proj = nn.Linear(self.num_heads * self.head_dim, self.hidden_size, bias=o_bias)
        if getattr(config, "use_qk_norm", False):
            zc = bool(getattr(config, "zero_centered_norm", False))
            self.q_norm = RMSNorm(self.head_dim, eps=config.rms_norm_eps, zero_centered=zc)
            self.k_norm = RMSNorm(self.head_dim, eps=config.rms_norm_eps, zero_centered=zc)
        else:
            self.q_norm = self.k_norm = None

    INPUT_PROJECTIONS, OUTPUT_PROJECTION = ("q_proj", "k_proj", "v_proj"), "o_proj"

    def _qkv(self, hidden_states, position_embeddings, kw=None):
        B, T, _ = hidden_states.shape
        q = input_proj(self, "q_proj", hidden_states, kw)
        gate = None
        if self.gated:
            q = q.view(B, T, self.num_heads, 2 * self.head_dim)
            q, gate = q[..., : self.head_dim], q[..., self.head_dim:].reshape(B, T, -1)
        else:
            q = q.view(B, T, self.num_heads, self.head_dim)
        k = input_proj(self, "k_proj", hidden_states, kw).view(B, T, self.num_kv_heads, self.head_dim)
        v = input_proj(self, "v_proj", hidden_states, kw).view(B, T, self.num_kv_heads, self.head_dim)
        if not self.gated and q.is_cuda and (self.q_norm is not None or position_embeddings is not None):
            from ..ops import cuda_ops
            if cuda_ops.heads_norm_rope_ok(q, self.head_dim, position_embeddings):
                # inference: per-head norm + rotary of q and of k in one launch each
                qn, kn = self.q_norm, self.k_norm
                eps = 0.0 if qn is None else qn.variance_epsilon
                zc = False if qn is None else qn.zero_centered
                q = cuda_ops.heads_norm_rope(q.reshape(B, T, -1), 0, self.num_heads, 0, None if qn is None else qn.weight,
                                             None, eps, zc, position_embeddings).view(B, T, self.num_heads, self.head_dim)
                k = cuda_ops.heads_norm_rope(k.reshape(B, T, -1), 0, self.num_kv_heads, 0,
                                             None if kn is None else kn.weight, None, eps, zc,
                                             position_embeddings).view(B, T, self.num_kv_heads, self.head_dim)
                return q, k, v, gate
        if self.q_norm is not None:
            q, k = self.q_norm(q), self.k_norm(k)
        if position_embeddings is not None:
            cos, sin = position_embeddings
            q, k = F_ops.apply_rope(q, cos, sin), F_ops.apply_rope(k, cos, sin)
        return q, k, v, gate

    def forward(self, hidden_states: torch.Tensor, position_embeddings=None, past_key_values=None,
                position_ids: Optional[torch.Tensor] = None, **kwargs) -> Tuple[torch.Tensor, None, object]:
        B, T, _ = hidden_states.shape
        q, k, v, gate = self._qkv(hidden_states, position_embeddings, kwargs)
        beta = (getattr(self.config, "rope_scaling", None) or {}).get("llama_4_scaling_beta")
        if beta and position_ids is not None:
            # queries far beyond the original context get a logarithmically growing temperature (Ministral 3):
            # 1 + beta * log(1 + floor(position / original_max_position_embeddings)), which is 1 inside that context
            old = float(self.config.rope_scaling.get("original_max_position_embeddings") or 0) or float("inf")
            scale = 1.0 + float(beta) * torch.log1p(torch.floor(position_ids.to(torch.float32) / old))
            q = q * scale.reshape(scale.shape[0], T, 1, 1).to(q.dtype)
        sp = self.sequence_parallel_group
        if sp is not None and sp.size > 1:
            if getattr(sp, "mode", "zigzag") == "ulysses":
                from ..parallel.ulysses import ulysses_attention
                o = ulysses_attention(q, k, v, sp, scale=self.scaling, window=self.sliding_window)
            elif self.sliding_window is None:
                o = cp_attention(q, k, v, sp, scale=self.scaling)
            else:
                o = self._swa_sp(q, k, v, sp)
        else:
            if past_key_values is not None:
                k, v = past_key_values.update_attention(self.layer_idx, k, v, window=self.sliding_window)
            ratio = getattr(self, "shift_group_ratio", None)
            group = int(T * ratio) if (ratio and self.training and past_key_values is None) else 0
            if group >= 2 and T % group == 0 and q.shape[2] % 2 == 0:
                # LongLoRA: attention inside groups of `group` tokens, half of the heads on the half-shifted sequence
                from ..layers.common import repeat_heads
                from ..train.adapters import shift_attention
                rep = q.shape[2] // k.shape[2]
                o = shift_attention(q, repeat_heads(k, rep), repeat_heads(v, rep), group,
                                    lambda a, b, c: F_ops.attention(a, b, c, scale=self.scaling, causal=True))
            else:
                o = F_ops.attention(q, k, v, scale=self.scaling, causal=True, window=self.sliding_window)
        o = o.reshape(B, T, -1)
        if gate is not None:
            o = o * torch.sigmoid(gate)
        return output_proj(self, "o_proj", o, kwargs), None, past_key_values

    def _swa_sp(self, q, k, v, sp):
        """Sliding-window attention under zig-zag SP: each segment needs the ``window-1`` keys
        before it, fetched as a halo from the neighbouring rank
        (reference: ``layers/swa/sequence_parallel.py:29-223``)."""
        B, T = q.shape[0], q.shape[1]
        half = T // 2
        w = self.sliding_window
        halo = min(w - 1, half)
        assert w - 1 <= half, "sliding window larger than a sequence-parallel chunk is not supported"
        kv = torch.cat([k, v], dim=-1)
        h = halo_exchange(kv, sp, halo)  # [B, 2, halo, Hkv, 2D]
        outs = []
        for seg in range(2):
            ks = torch.cat([h[:, seg], kv[:, seg * half:(seg + 1) * half]], dim=1)
            k_s, v_s = ks[..., : self.head_dim], ks[..., self.head_dim:]
            first = (seg == 0 and sp.rank == 0)
            if first:
                # zeros before position 0 must not be attended: drop the halo
                k_s, v_s = k_s[:, halo:], v_s[:, halo:]
            outs.append(F_ops.attention(q[:, seg * half:(seg + 1) * half], k_s.contiguous(), v_s.contiguous(),
                                        scale=self.scaling, causal=True, window=w))
        return torch.cat(outs, dim=1)


class SlidingWindowAttention(Attention):
    """``SWA`` layer symbol: attention restricted to the last ``window_size`` tokens."""

    def __init__(self, config, layer_idx: int):
        swa = getattr(config, "swa_config", None) or {}
        window = swa.get("window_size") if isinstance(swa, dict) else getattr(swa, "window_size", None)
        window = window or getattr(config, "sliding_window", None) or 2048
        super().__init__(config, layer_idx, sliding_window=int(window))
