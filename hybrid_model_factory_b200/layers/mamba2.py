"""Mamba2 mixer mapped onto the attention dimensions of the base Transformer.

Correspondence ``x <-> V``, ``B <-> K``, ``C <-> Q``; ``headdim = d_state = head_dim``,
``ngroups = nheads = Hq``, ``d_xb = Hkv * head_dim``.  ``in_proj -> [z, x, B, C, dt]``; optional
per-head RMSNorm on B and C; optional RoPE on B and C; depthwise causal conv (k=4) + SiLU over
``[x, B, C]``; x and B repeated to ``H`` heads; SSD chunk scan; gated RMSNorm with ``z``
(``norm_before_gate=False``, group = head); ``out_proj``.
Reference: ``layers/mamba/mamba2.py:98-693`` and ``mamba2_config.py:58-122``.
"""
from __future__ import annotations

from dataclasses import asdict, dataclass, field
from typing import Optional

import torch
import torch.nn as nn
import torch.nn.functional as F

from ..ops import functional as F_ops
from ..ops import mixers
from ..parallel.sp import merge_segments, segments_with_halo
from .common import GatedRMSNorm, RMSNorm, init_dt_bias, input_proj, output_proj, repeat_heads


@dataclass
class Mamba2Config:
    d_model: int
    d_inner: int
    d_xb: int
    ssm_cfg: dict = field(default_factory=dict)
    use_qk_norm: bool = True
    use_pos_emb: bool = False
    d_conv: int = 4
    chunk_size: int = 256
    rms_norm_eps: float = 1e-6

    def to_dict(self):
        return asdict(self)

    @classmethod
    def from_dict(cls, d):
        if isinstance(d, cls):
            return d
        fields = cls.__dataclass_fields__
        return cls(**{k: v for k, v in dict(d).items() if k in fields})


def construct_mamba2_config(config, user: Optional[dict] = None) -> Mamba2Config:
    user = user.to_dict() if hasattr(user, "to_dict") else dict(user or {})
    nh = config.num_attention_heads
    head_dim = getattr(config, "head_dim", None) or config.hidden_size // nh
    nkv = getattr(config, "num_key_value_heads", nh)
    return Mamba2Config(d_model=config.hidden_size, d_inner=nh * head_dim, d_xb=nkv * head_dim,
                        ssm_cfg={"expand": 1, "ngroups": nh, "d_state": head_dim},
                        use_qk_norm=user.get("use_qk_norm", True), use_pos_emb=user.get("use_pos_emb", False),
                        rms_norm_eps=getattr(config, "rms_norm_eps", 1e-6))


class Mamba2(nn.Module):
    def __init__(self, d_model: int, d_inner: int, d_xb: int, d_state: int, ngroups: int, d_conv: int = 4,
                 chunk_size: int = 256, use_qk_norm: bool = True, use_pos_emb: bool = False, bias: bool = False,
                 conv_bias: bool = True, layer_idx: Optional[int] = None, dt_min: float = 0.001, dt_max: float = 0.1,
                 A_init_range=(1, 16), **_):
        super().__init__()
        self.d_model, self.d_inner, self.d_xb, self.d_state, self.ngroups = d_model, d_inner, d_xb, d_state, ngroups
        self.headdim = d_state
        self.nheads = d_inner // self.headdim
        self.num_kv_groups = d_inner // d_xb
        self.d_conv, self.chunk_size, self.layer_idx = d_conv, chunk_size, layer_idx
        self.use_pos_emb = use_pos_emb
        self.sequence_parallel_group = None
        assert d_inner == ngroups * d_state
        d_in_proj = d_inner + d_xb + d_xb + d_inner + self.nheads  # [z, x, B, C, dt]
        self.in_proj = nn.Linear(d_model, d_in_proj, bias=bias)
        self.in_proj_valid = d_in_proj      # tensor-parallel shards pad the weight with zero rows past this width
        self.conv_dim = d_inner + 2 * d_xb
        self.conv1d = nn.Conv1d(self.conv_dim, self.conv_dim, kernel_size=d_conv, groups=self.conv_dim,
                                padding=d_conv - 1, bias=conv_bias)
        self.dt_bias = nn.Parameter(init_dt_bias(self.nheads, dt_min, dt_max))
        self.dt_bias._no_weight_decay = True
        self.A_log = nn.Parameter(torch.log(torch.empty(self.nheads, dtype=torch.float32).uniform_(*A_init_range)))
        self.A_log._no_weight_decay = True
        self.D = nn.Parameter(torch.ones(self.nheads))
        self.D._no_weight_decay = True
        self.norm = GatedRMSNorm(self.headdim, eps=1e-5, norm_before_gate=False)
        # the gated norm weight spans d_inner in the checkpoint (one scale per channel)
        self.norm.weight = nn.Parameter(torch.ones(d_inner))
        self.out_proj = nn.Linear(d_inner, d_model, bias=bias)
        if use_qk_norm:
            self.C_norm = RMSNorm(self.headdim, 1e-6)
            self.B_norm = RMSNorm(self.headdim, 1e-6)
        else:
            self.C_norm = self.B_norm = None

    def _norm_rope(self, xBC, position_embeddings):
        Bsz, T, _ = xBC.shape
        pe = position_embeddings if self.use_pos_emb else None
        if xBC.is_cuda and self.headdim == 128 and self.d_xb % 128 == 0 and self.d_state == 128:
            from ..ops import cuda_ops
            if cuda_ops.heads_norm_rope_ok(xBC, self.headdim, pe):       # inference: one kernel for the whole method
                bn = self.B_norm
                return cuda_ops.heads_norm_rope(
                    xBC, self.d_xb // 128, self.d_xb // 128, self.d_inner // 128, None if bn is None else bn.weight,
                    None if bn is None else self.C_norm.weight, 0.0 if bn is None else bn.variance_epsilon,
                    False if bn is None else bn.zero_centered, pe)
        x, Bm, Cm = torch.split(xBC, [self.d_xb, self.d_xb, self.d_inner], dim=-1)
        Bm = Bm.reshape(Bsz, T, -1, self.headdim)
        Cm = Cm.reshape(Bsz, T, -1, self.headdim)
        if self.B_norm is not None:
            Bm, Cm = self.B_norm(Bm), self.C_norm(Cm)
        if self.use_pos_emb and position_embeddings is not None:
            cos, sin = position_embeddings
            Bm, Cm = F_ops.apply_rope(Bm, cos, sin), F_ops.apply_rope(Cm, cos, sin)
        return torch.cat([x, Bm.reshape(Bsz, T, -1), Cm.reshape(Bsz, T, -1)], dim=-1)

    INPUT_PROJECTIONS, OUTPUT_PROJECTION = ("in_proj",), "out_proj"

    def forward(self, hidden_states: torch.Tensor, past_key_values=None, position_embeddings=None,
                use_cache: bool = False, **kwargs):
        sp = self.sequence_parallel_group
        Bsz, T, _ = hidden_states.shape
        last = past_key_values.get_ssm(self.layer_idx) if past_key_values is not None else None
        zxbcdt = input_proj(self, "in_proj", hidden_states, kwargs)
        if zxbcdt.shape[-1] != self.in_proj_valid:
            zxbcdt = zxbcdt[..., :self.in_proj_valid]
        z, xBC, dt = torch.split(zxbcdt, [self.d_inner, self.conv_dim, self.nheads], dim=-1)
        xBC = self._norm_rope(xBC, position_embeddings)
        w = self.conv1d.weight.squeeze(1)
        new_conv = None
        if sp is not None and sp.size > 1:
            seg, halo = segments_with_halo(xBC, sp, self.d_conv - 1)
            xBC = merge_segments(F_ops.causal_conv1d(seg, w, self.conv1d.bias, "silu", halo), sp)
        else:
            cs = last["conv_state"] if last is not None else None
            want = use_cache or past_key_values is not None
            if T == 1 and cs is not None and not self.training:
                y1, new_conv = F_ops.causal_conv1d_update(xBC[:, 0], cs, w, self.conv1d.bias, "silu")
                xBC = y1[:, None]
            elif want:
                xBC, new_conv = F_ops.causal_conv1d(xBC, w, self.conv1d.bias, "silu", cs, True)
            else:
                xBC = F_ops.causal_conv1d(xBC, w, self.conv1d.bias, "silu", cs)
        x, Bm, Cm = torch.split(xBC, [self.d_xb, self.d_xb, self.d_inner], dim=-1)
        x = repeat_heads(x.reshape(Bsz, T, -1, self.headdim), self.num_kv_groups)
        Bm = repeat_heads(Bm.reshape(Bsz, T, -1, self.d_state), self.num_kv_groups)
        Cm = Cm.reshape(Bsz, T, self.ngroups, self.d_state)
        A = -torch.exp(self.A_log.float())
        dtp = F.softplus(dt.float() + self.dt_bias.float())
        state0 = last["recurrent_state"] if last is not None else None
        y, state = mixers.ssd(x, dtp, A, Bm, Cm, self.D, initial_state=state0, sp=sp, chunk_size=self.chunk_size,
                              recurrent=(T == 1 and not self.training))
        if past_key_values is not None:
            log_aprod = (dtp * A).sum(dim=1)  # [B, H] log of the cumulative decay (state composition)
            past_key_values.update_ssm(self.layer_idx, recurrent_state=state, conv_state=new_conv, offset=T,
                                       log_aprod=log_aprod)
        y = y.to(hidden_states.dtype)
        zg = z.reshape(Bsz, T, self.nheads, self.headdim)
        wn = self.norm.weight.view(self.nheads, self.headdim)
        y = F_ops.gated_rms_norm(y, zg, wn, self.norm.eps, norm_before_gate=False)
        return output_proj(self, "out_proj", y.reshape(Bsz, T, self.d_inner), kwargs), None, past_key_values


class Mamba2Layer(Mamba2):
    def __init__(self, config, layer_idx: int):
        cfg = getattr(config, "mamba2_config", None)
        cfg = Mamba2Config.from_dict(cfg) if cfg else construct_mamba2_config(config)
        super().__init__(d_model=cfg.d_model, d_inner=cfg.d_inner, d_xb=cfg.d_xb, d_state=cfg.ssm_cfg["d_state"],
                         ngroups=cfg.ssm_cfg["ngroups"], d_conv=cfg.d_conv, chunk_size=cfg.chunk_size,
                         use_qk_norm=cfg.use_qk_norm, use_pos_emb=cfg.use_pos_emb, layer_idx=layer_idx)
