"""L2A ("learn to attend") mixer: sliding-window attention for every token plus *conditional* global attention
for the tokens a router selects.

    s   = SWA(norm(x))                                    local stream, own q/k/v/o projections
    x1  = x + s
    d   = sigmoid(W_r norm_g(x1) / temperature)           router, one scalar per token
    m   = 1[d > threshold] + d - stopgrad(d)              straight-through hard decision
    g   = o_g( m * Attn_global(q_g, K_g, V_g) )           only the selected query rows are computed
    out = s + g                                           (the decoder layer adds the residual)

Global attention uses a second projection set and the query-sparse kernel path
(``ops.functional.qsparse_attention``: compacted queries with their original positions against the full K/V).
During training a fraction ``leak_prob`` of the steps runs dense attention for all tokens ("stochastic leakage").
The sparsity regulariser ``sum d^2`` of the last forward is kept in ``last_soft_sq`` / ``last_tokens`` for the
trainer.  Reference: ``examples/research/L2A/model/l2a_qwen3/modeling_qwen3.py:226-630``.
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.nn as nn

from ..ops import functional as F_ops
from .attention import Attention
from .common import RMSNorm


class L2AAttention(nn.Module):
    def __init__(self, config, layer_idx: int):
        super().__init__()
        l2a = getattr(config, "l2a_config", None) or {}
        self.layer_idx = layer_idx
        self.window = int(l2a.get("sliding_window", getattr(config, "sliding_window", None) or 512))
        self.threshold = float(l2a.get("sigmoid_threshold", 0.5))
        self.temperature = float(l2a.get("temperature", 1.0))
        self.leak_prob = float(l2a.get("leak_prob", 0.1))
        self.local = Attention(config, layer_idx, sliding_window=self.window)
        self.global_attn = Attention(config, layer_idx)          # q/k/v/o_proj (+ q/k norms) of the global stream
        self.global_norm = RMSNorm(config.hidden_size, config.rms_norm_eps)
        self.router = nn.Linear(config.hidden_size, 1, bias=False)
        self.sequence_parallel_group = None
        # training step, set by the L2A loss before every forward: the leakage coin is a function of (layer, step), so
        # the first run and the re-run of a checkpointed layer, and all ranks of a sequence-parallel group, agree on it
        self.leak_step: Optional[int] = None
        self.last_soft_sq: Optional[torch.Tensor] = None
        self.last_tokens = 0
        self.last_routed_fraction = 0.0

    def _leak_coin(self, sp) -> float:
        """Uniform number in [0, 1) deciding "dense attention for all tokens this step"."""
        if self.leak_step is not None:
            g = torch.Generator().manual_seed(1_000_003 * (self.layer_idx + 1) + int(self.leak_step))
            return float(torch.rand((), generator=g))
        coin = torch.rand(())
        if sp is not None:                         # no step was announced: rank 0 of the group decides for all
            import torch.distributed as dist
            dev = self.router.weight.device
            t = coin.to(dev if dev.type == "cuda" else "cpu")
            dist.broadcast(t, src=sp.ranks[0], group=sp.group)
            coin = t.cpu()
        return float(coin)

    def forward(self, hidden_states, residual=None, position_embeddings=None, past_key_values=None, position_ids=None,
                **kwargs):
        B, T, _ = hidden_states.shape
        # generation: the local stream keeps its window of K / V under this layer's index, the global stream keeps all
        # of its K / V under a key of its own; only the routed tokens ever read the global cache
        s, _, _ = self.local(hidden_states, position_embeddings=position_embeddings, position_ids=position_ids,
                             past_key_values=past_key_values)
        base = hidden_states if residual is None else residual
        h2 = self.global_norm(base + s)
        soft = torch.sigmoid(self.router(h2).float() / self.temperature)        # [B, T, 1]
        hard = (soft >= self.threshold).float()             # a zero router (stage 0) sends every token to global attention
        mask = hard + soft - soft.detach()
        sp = self.sequence_parallel_group
        sp_on = sp is not None and sp.size > 1
        # under sequence parallelism the ranks' regularisers add up (their gradients are summed): each holds its share
        self.last_soft_sq, self.last_tokens = (soft ** 2).sum(), B * T * (sp.size if sp_on else 1)
        self.last_routed_fraction = float(hard.mean())
        ga = self.global_attn
        q, k, v, _ = ga._qkv(h2, position_embeddings)
        offset = 0
        if past_key_values is not None and hasattr(past_key_values, "attention"):
            k, v = past_key_values.update_attention(("l2a_global", self.layer_idx), k, v)
            offset = k.shape[1] - T                 # tokens already in the cache: the new queries come after them
        leak = self.training and self.leak_prob > 0 and self._leak_coin(sp if sp_on else None) < self.leak_prob
        if leak and sp_on:
            from ..parallel.cp_attention import cp_attention
            o = cp_attention(q, k, v, sp, scale=ga.scaling)
        elif leak:
            o = F_ops.attention(q, k, v, scale=ga.scaling, causal=True)
        else:
            if sp_on:
                # the selected local queries attend the whole (gathered) sequence at their global positions; the
                # gradients of K / V are reduce-scattered back to their owners by the gather's backward
                from ..parallel.cp_attention import gather_seq
                from ..parallel.sp import zigzag_positions
                k, v = gather_seq(k, sp), gather_seq(v, sp)
                gpos = zigzag_positions(T * sp.size, sp.rank, sp.size, device=q.device)
            else:
                gpos = None
            o = torch.zeros_like(q)
            for b in range(B):                                   # rows differ per sample: compact each one
                idx = torch.nonzero(hard[b, :, 0], as_tuple=False)[:, 0]
                if idx.numel() == 0:
                    continue
                pos = idx + offset if gpos is None else gpos[idx]
                ob = F_ops.qsparse_attention(q[b:b + 1, idx], k[b:b + 1], v[b:b + 1], pos[None], scale=ga.scaling)
                o[b, idx] = ob[0].to(o.dtype)
        o = (o * mask[..., None].to(o.dtype)).reshape(B, T, -1)
        return s + ga.o_proj(o), None, past_key_values


def set_l2a_step(model: nn.Module, step: int) -> None:
    for m in model.modules():
        if isinstance(m, L2AAttention):
            m.leak_step = int(step)


def l2a_regulariser(model: nn.Module) -> torch.Tensor:
    """Mean over layers of ``sum d^2 / tokens`` from the last forward."""
    terms = [m.last_soft_sq / max(m.last_tokens, 1) for m in model.modules()
             if isinstance(m, L2AAttention) and m.last_soft_sq is not None]
    if not terms:
        return torch.zeros(())
    return torch.stack(terms).mean()


def router_sparsity(model: nn.Module) -> dict:
    """Per-layer fraction of tokens routed to global attention (logged by the L2A trainer)."""
    return {m.layer_idx: m.last_routed_fraction for m in model.modules() if isinstance(m, L2AAttention)}
