"""Ulysses-style sequence parallelism for softmax attention: an all-to-all turns the sequence sharding into a head
sharding (every rank sees the whole sequence for ``H / SP`` heads), attention runs locally, and a second all-to-all
restores the sequence sharding.  Attention only; the SSM mixers always use the state chain (``ops.scan``).  Selected
with ``sequence_parallel_mode: ulysses`` (reference: ``yunchang`` Ulysses, "attention only, not for hybrid models",
``docs/SequenceParallel.md:215``).

The local tokens are the two zig-zag chunks of this rank; after the gather the chunks are put back into global
order so plain causal masking applies.
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.distributed as dist

from ..ops import functional as F_ops

Tensor = torch.Tensor


class _SeqToHead(torch.autograd.Function):
    """``[B, T_loc, H, D] -> [B, SP * T_loc, H / SP, D]`` (rank-major sequence order)."""

    @staticmethod
    def forward(ctx, x: Tensor, group, size: int):
        ctx.group, ctx.size = group, size
        B, T, H, D = x.shape
        send = x.view(B, T, size, H // size, D).permute(2, 0, 1, 3, 4).contiguous()     # [SP, B, T, H/SP, D]
        recv = torch.empty_like(send)
        dist.all_to_all_single(recv, send, group=group)
        return recv.permute(1, 0, 2, 3, 4).reshape(B, size * T, H // size, D)

    @staticmethod
    def backward(ctx, g: Tensor):
        return _HeadToSeq.apply(g, ctx.group, ctx.size), None, None


class _HeadToSeq(torch.autograd.Function):
    """Inverse of ``_SeqToHead``."""

    @staticmethod
    def forward(ctx, x: Tensor, group, size: int):
        ctx.group, ctx.size = group, size
        B, TT, Hs, D = x.shape
        T = TT // size
        send = x.view(B, size, T, Hs, D).permute(1, 0, 2, 3, 4).contiguous()            # [SP, B, T, H/SP, D]
        recv = torch.empty_like(send)
        dist.all_to_all_single(recv, send, group=group)
        return recv.permute(1, 2, 0, 3, 4).reshape(B, T, size * Hs, D)

    @staticmethod
    def backward(ctx, g: Tensor):
        return _SeqToHead.apply(g, ctx.group, ctx.size), None, None


def _global_order(sp_size: int, chunk: int, device) -> Tensor:
    """Index that turns the rank-major concatenation of zig-zag shards into global token order."""
    pos = []
    for r in range(sp_size):
        pos += [r, 2 * sp_size - 1 - r]
    chunk_of = torch.tensor(pos, device=device)                     # chunk id held at slot j
    slot_of = torch.argsort(chunk_of)                               # slot that holds chunk c
    return (slot_of[:, None] * chunk + torch.arange(chunk, device=device)[None]).reshape(-1)


def ulysses_attention(q: Tensor, k: Tensor, v: Tensor, sp, *, scale: Optional[float] = None,
                      window: Optional[int] = None) -> Tensor:
    n = sp.size
    Hq, Hkv = q.shape[2], k.shape[2]
    assert Hq % n == 0 and Hkv % n == 0, "Ulysses needs the head counts to divide by the SP size"
    qg, kg, vg = (_SeqToHead.apply(t, sp.group, n) for t in (q, k, v))
    chunk = q.shape[1] // 2
    order = _global_order(n, chunk, q.device)
    inv = torch.argsort(order)
    o = F_ops.attention(qg[:, order], kg[:, order], vg[:, order], scale=scale, causal=True, window=window)
    return _HeadToSeq.apply(o[:, inv].contiguous(), sp.group, n)
