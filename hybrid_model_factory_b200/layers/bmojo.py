"""B'MOJO-F layer: an SSM mixer produces "fading tokens"; two sliding-window attention passes
run over (a) in-context keys/values projected from the layer input with window ``w`` and
(b) fading keys/values projected from the SSM output, visible through the *hollow* window
``[i-2w+1, i-w]``; both are merged with the exact log-sum-exp softmax combination.  With
``tie_attn_weights=False`` the fading stream has its own ``q/k/v_proj_`` (and q/k norms).
Reference: ``layers/bmojo_f/modules.py:31-211``, ``bmojo_attention.py:69-503``,
``bmojo_attention_utils.py:79-211`` and ``:409-426``.
"""
from __future__ import annotations


import torch
import torch.nn as nn

from ..ops import functional as F_ops
from ..parallel.sp import halo_exchange
from .common import RMSNorm
from .gdn import GatedDeltaNetLayer
from .gka import GatedKalmaNetLayer
from .mamba2 import Mamba2Layer


def _bmojo_cfg(config) -> dict:
    cfg = getattr(config, "bmojo_config", None) or {}
    cfg = cfg.to_dict() if hasattr(cfg, "to_dict") else dict(cfg)
    return {"window_size": int(cfg.get("window_size", 2048)), "tie_attn_weights": bool(cfg.get("tie_attn_weights", True)),
            "ssm_mixer": str(cfg.get("ssm_mixer", "mamba2"))}


class BMOJOAttention(nn.Module):
    def __init__(self, config, layer_idx: int):
        super().__init__()
        cfg = _bmojo_cfg(config)
        self.layer_idx = layer_idx
        self.window = cfg["window_size"]
        self.tie_attn_weights = cfg["tie_attn_weights"]
        self.hidden_size = config.hidden_size
        self.num_heads = config.num_attention_heads
        self.num_kv_heads = getattr(config, "num_key_value_heads", self.num_heads)
        self.head_dim = getattr(config, "head_dim", None) or self.hidden_size // self.num_heads
        self.scaling = self.head_dim ** -0.5
        self.sequence_parallel_group = None
        bias = bool(getattr(config, "attention_bias", False) or getattr(config, "qkv_bias", False))
        qd, kvd = self.num_heads * self.head_dim, self.num_kv_heads * self.head_dim
        self.q_proj = nn.Linear(self.hidden_size, qd, bias=bias)
        self.k_proj = nn.Linear(self.hidden_size, kvd, bias=bias)
        self.v_proj = nn.Linear(self.hidden_size, kvd, bias=bias)
        self.o_proj = nn.Linear(qd, self.hidden_size, bias=False)
        qk_norm = bool(getattr(config, "use_qk_norm", False))
        self.q_norm = RMSNorm(self.head_dim, config.rms_norm_eps) if qk_norm else None
        self.k_norm = RMSNorm(self.head_dim, config.rms_norm_eps) if qk_norm else None
        if not self.tie_attn_weights:
            self.q_proj_ = nn.Linear(self.hidden_size, qd, bias=bias)
            self.k_proj_ = nn.Linear(self.hidden_size, kvd, bias=bias)
            self.v_proj_ = nn.Linear(self.hidden_size, kvd, bias=bias)
            self.q_norm_ = RMSNorm(self.head_dim, config.rms_norm_eps) if qk_norm else None
            self.k_norm_ = RMSNorm(self.head_dim, config.rms_norm_eps) if qk_norm else None

    def _project(self, q_src, kv_src, in_context: bool, position_embeddings):
        B, T, _ = q_src.shape
        untied = (not self.tie_attn_weights) and (not in_context)
        qp, kp, vp = (self.q_proj_, self.k_proj_, self.v_proj_) if untied else (self.q_proj, self.k_proj, self.v_proj)
        qn, kn = (self.q_norm_, self.k_norm_) if untied else (self.q_norm, self.k_norm)
        q = qp(q_src).view(B, T, self.num_heads, self.head_dim)
        k = kp(kv_src).view(B, T, self.num_kv_heads, self.head_dim)
        v = vp(kv_src).view(B, T, self.num_kv_heads, self.head_dim)
        if qn is not None:
            q, k = qn(q), kn(k)
        if position_embeddings is not None:
            cos, sin = position_embeddings
            q, k = F_ops.apply_rope(q, cos, sin), F_ops.apply_rope(k, cos, sin)
        return q, k, v

    def forward(self, hidden_states, fading_tokens, position_embeddings=None, position_ids=None, past_key_values=None):
        B, T, _ = hidden_states.shape
        w = self.window
        q_s, k_s, v_s = self._project(hidden_states, hidden_states, True, position_embeddings)
        q_c, k_c, v_c = self._project(hidden_states, fading_tokens, False, position_embeddings)
        sp = self.sequence_parallel_group
        if position_ids is None:
            off = past_key_values.seqlen_offset if past_key_values is not None else 0
            position_ids = torch.arange(off, off + T, device=hidden_states.device).expand(B, T)
        if sp is not None and sp.size > 1:
            o = self._forward_sp(q_s, k_s, v_s, q_c, k_c, v_c, position_ids, sp)
        else:
            k_pos = position_ids
            if past_key_values is not None:
                k_s, v_s, k_c, v_c, k_pos = past_key_values.update_bmojo(self.layer_idx, k_s, v_s, k_c, v_c, position_ids,
                                                                         keep=2 * w - 1)
            o_s, l_s = F_ops.attention(q_s, k_s, v_s, scale=self.scaling, causal=True, window=w, q_pos=position_ids,
                                       k_pos=k_pos, return_lse=True)
            o_c, l_c = F_ops.attention(q_c, k_c, v_c, scale=self.scaling, causal=True, hollow=w, q_pos=position_ids,
                                       k_pos=k_pos, return_lse=True)
            o, _ = F_ops.merge_attention_states(o_s, l_s, o_c, l_c)
        return self.o_proj(o.reshape(B, T, -1))

    def _forward_sp(self, q_s, k_s, v_s, q_c, k_c, v_c, position_ids, sp):
        """Zig-zag SP: both streams need the ``2w-1`` tokens before each local segment."""
        B, T = q_s.shape[0], q_s.shape[1]
        half, w = T // 2, self.window
        halo = 2 * w - 1
        assert halo <= half, f"B'MOJO window {2 * w} larger than a sequence-parallel chunk {half} is not supported"
        kv = torch.cat([k_s, v_s, k_c, v_c], dim=-1)
        h = halo_exchange(kv, sp, halo)
        D = self.head_dim
        outs = []
        for seg in range(2):
            sl = slice(seg * half, (seg + 1) * half)
            kv_seg = torch.cat([h[:, seg], kv[:, sl]], dim=1)
            q_pos = position_ids[:, sl]
            k_pos = torch.cat([q_pos[:, :1] - halo + torch.arange(halo, device=q_pos.device)[None], q_pos], dim=1)
            ks, vs, kc, vc = (kv_seg[..., i * D:(i + 1) * D].contiguous() for i in range(4))
            # keys before position 0 (rank 0, first segment) have negative positions: mask them by
            # pushing them outside every window
            k_pos = torch.where(k_pos < 0, torch.full_like(k_pos, -(4 * w + 4 * half)), k_pos)
            o_s, l_s = F_ops.attention(q_s[:, sl], ks, vs, scale=self.scaling, causal=True, window=w, q_pos=q_pos,
                                       k_pos=k_pos, return_lse=True)
            o_c, l_c = F_ops.attention(q_c[:, sl], kc, vc, scale=self.scaling, causal=True, hollow=w, q_pos=q_pos,
                                       k_pos=k_pos, return_lse=True)
            outs.append(F_ops.merge_attention_states(o_s, l_s, o_c, l_c)[0])
        return torch.cat(outs, dim=1)


class BMojoLayer(nn.Module):
    def __init__(self, config, layer_idx: int):
        super().__init__()
        cfg = _bmojo_cfg(config)
        self.ssm_mixer_type = cfg["ssm_mixer"].lower()
        self.sequence_parallel_group = None
        if self.ssm_mixer_type == "mamba2":
            self.mamba = Mamba2Layer(config, layer_idx)
        elif self.ssm_mixer_type in ("gated_deltanet", "gdn"):
            self.gdn = GatedDeltaNetLayer(config, layer_idx)
        elif self.ssm_mixer_type in ("gated_kalmanet", "gka"):
            self.gka = GatedKalmaNetLayer(config, layer_idx)
        else:
            raise ValueError(f"{self.ssm_mixer_type} is not a valid fading-token mixer for B'MOJO "
                             "(expected mamba2, gdn or gka)")
        self.bmojo_attn = BMOJOAttention(config, layer_idx)

    @property
    def ssm_mixer(self):
        if self.ssm_mixer_type == "mamba2":
            return self.mamba
        if self.ssm_mixer_type in ("gated_deltanet", "gdn"):
            return self.gdn
        return self.gka

    def forward(self, hidden_states, position_embeddings=None, position_ids=None, past_key_values=None, **kwargs):
        fading, _, _ = self.ssm_mixer(hidden_states, past_key_values=past_key_values,
                                      position_embeddings=position_embeddings, **kwargs)
        out = self.bmojo_attn(hidden_states, fading, position_embeddings, position_ids, past_key_values)
        return out, None, past_key_values
