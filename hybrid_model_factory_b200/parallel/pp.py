"""Pipeline parallelism for inference: consecutive decoder layers are assigned to stages (one rank each); hidden
states travel between stages with point-to-point sends.  The first stage owns the embedding, the last stage the
final norm and ``lm_head``; sampled tokens are broadcast from the last stage so that every stage can extend its
caches.  (The reference gets this from vLLM's ``SupportsPP`` / ``make_layers`` / ``IntermediateTensors``,
``hybridqwen3.py:813-824``.)
"""
from __future__ import annotations

from typing import List, Optional, Tuple

import torch
import torch.distributed as dist

from ..models.cache import HybridCache


def partition_layers(num_layers: int, stages: int) -> List[Tuple[int, int]]:
    base, extra = divmod(num_layers, stages)
    out, start = [], 0
    for s in range(stages):
        n = base + (1 if s < extra else 0)
        out.append((start, start + n))
        start += n
    return out


class PipelineStage:
    """Runs layers ``[lo, hi)`` of ``model`` on this rank."""

    def __init__(self, model, group=None):
        self.model, self.group = model, group
        self.rank, self.size = dist.get_rank(group), dist.get_world_size(group)
        self.lo, self.hi = partition_layers(len(model.model.layers), self.size)[self.rank]
        self.first, self.last = self.rank == 0, self.rank == self.size - 1
        for i, layer in enumerate(model.model.layers):       # free the layers of other stages
            if not (self.lo <= i < self.hi):
                for p in layer.parameters():
                    p.data = p.data.new_empty(0)

    @torch.no_grad()
    def forward(self, input_ids: torch.Tensor, position_ids: torch.Tensor, cache: HybridCache) -> Optional[torch.Tensor]:
        m = self.model.model
        B, T = input_ids.shape
        dev = next(p for p in self.model.parameters() if p.numel()).device
        if self.first:
            h = m.embed_tokens(input_ids)
        else:
            h = torch.empty(B, T, self.model.config.hidden_size, device=dev, dtype=m.norm.weight.dtype)
            dist.recv(h, src=dist.get_global_rank(self.group, self.rank - 1) if self.group else self.rank - 1,
                      group=self.group)
        pe = m.rotary_emb(position_ids)
        pe = tuple(t.to(h.dtype) for t in pe)
        for i in range(self.lo, self.hi):
            out = m.layers[i](h, position_embeddings=pe, position_ids=position_ids, past_key_values=cache,
                              use_cache=True)
            h = out[0] if isinstance(out, tuple) else out
        if not self.last:
            dist.send(h.contiguous(), dst=dist.get_global_rank(self.group, self.rank + 1) if self.group else self.rank + 1,
                      group=self.group)
            return None
        return self.model.lm_head(m.norm(h[:, -1:]))

    @torch.no_grad()
    def generate(self, input_ids: torch.Tensor, max_new_tokens: int = 8) -> torch.Tensor:
        cache = HybridCache()
        ids, pos0, out = input_ids, 0, []
        src = dist.get_global_rank(self.group, self.size - 1) if self.group else self.size - 1
        for _ in range(max_new_tokens):
            pos = torch.arange(pos0, pos0 + ids.shape[1], device=ids.device)[None].expand(ids.shape[0], -1)
            logits = self.forward(ids, pos, cache)
            cache.update_offset(ids.shape[1])
            nxt = logits.argmax(-1) if self.last else torch.empty(ids.shape[0], 1, dtype=torch.long, device=ids.device)
            dist.broadcast(nxt, src=src, group=self.group)
            out.append(nxt)
            pos0 += ids.shape[1]
            ids = nxt
        return torch.cat(out, dim=1)
