"""Expert parallelism: experts are sharded over the ranks of a group; tokens travel to their experts' owners by
all-to-all, are processed by the grouped expert GEMMs there and travel back (dispatch / combine).

Rank ``r`` owns experts ``[r * E/size, (r+1) * E/size)``; ``shard_experts`` slices the stacked expert weights of a
``SparseMoeBlock`` accordingly.  Both all-to-alls are differentiable (the backward of an all-to-all is the
all-to-all with the split sizes swapped), so the same path serves training.  The reference has expert
parallelism only in serving, through vLLM's ``SharedFusedMoE`` (``hybridqwen3_moe.py:913-1263``), and trains MoE
with a Python loop over experts.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List

import torch
import torch.distributed as dist

Tensor = torch.Tensor


@dataclass
class EPContext:
    group: object
    rank: int
    size: int

    @classmethod
    def from_group(cls, group=None) -> "EPContext":
        return cls(group, dist.get_rank(group), dist.get_world_size(group))


class _AllToAll(torch.autograd.Function):
    """Rows of ``x`` are cut into ``in_splits`` pieces sent to ranks 0..n-1; returns the concatenation of the
    received pieces (``out_splits`` rows from each rank)."""

    @staticmethod
    def forward(ctx, x: Tensor, in_splits: List[int], out_splits: List[int], group):
        ctx.in_splits, ctx.out_splits, ctx.group = in_splits, out_splits, group
        out = x.new_empty(sum(out_splits), *x.shape[1:])
        dist.all_to_all_single(out, x.contiguous(), out_splits, in_splits, group=group)
        return out

    @staticmethod
    def backward(ctx, g: Tensor):
        out = g.new_empty(sum(ctx.in_splits), *g.shape[1:])
        dist.all_to_all_single(out, g.contiguous(), ctx.in_splits, ctx.out_splits, group=ctx.group)
        return out, None, None, None


def all_to_all_rows(x: Tensor, in_splits: List[int], out_splits: List[int], group) -> Tensor:
    return _AllToAll.apply(x, in_splits, out_splits, group)


def shard_experts(moe_block, ep: EPContext) -> None:
    """Keeps this rank's slice of the stacked expert weights (in place)."""
    E = moe_block.experts.gate_up_proj.shape[0]
    assert E % ep.size == 0, f"{E} experts do not divide over {ep.size} ranks"
    per = E // ep.size
    sl = slice(ep.rank * per, (ep.rank + 1) * per)
    moe_block.experts.gate_up_proj.data = moe_block.experts.gate_up_proj.data[sl].contiguous()
    moe_block.experts.down_proj.data = moe_block.experts.down_proj.data[sl].contiguous()
    moe_block.expert_parallel_group = ep
    moe_block.num_local_experts = per


def ep_experts_forward(x: Tensor, w_gate_up: Tensor, w_down: Tensor, weights: Tensor, indices: Tensor,
                       ep: EPContext) -> Tensor:
    """``x [T, Dm]`` local tokens, global routing ``indices [T, k]``; ``w_*`` hold this rank's experts only."""
    from ..ops.moe import experts_rows
    T, k = indices.shape
    per = w_gate_up.shape[0]
    flat_e = indices.reshape(-1)
    order = torch.argsort(flat_e, stable=True)           # by global expert = by owner rank, then local expert
    token_of = order // k
    send_e = flat_e[order]
    send_counts = torch.bincount(send_e // per, minlength=ep.size)
    recv_counts = torch.empty_like(send_counts)
    dist.all_to_all_single(recv_counts, send_counts, group=ep.group)
    in_splits, out_splits = send_counts.tolist(), recv_counts.tolist()
    # dispatch tokens and their (local) expert ids
    xr = all_to_all_rows(x[token_of], in_splits, out_splits, ep.group)
    er = torch.empty(sum(out_splits), dtype=send_e.dtype, device=x.device)
    dist.all_to_all_single(er, (send_e % per).contiguous(), out_splits, in_splits, group=ep.group)
    # local grouped experts
    y_rows = experts_rows(xr, er, w_gate_up, w_down)        # grouped tcgen05 GEMMs on the GPU
    # combine
    yb = all_to_all_rows(y_rows, out_splits, in_splits, ep.group)
    yb = yb * weights.reshape(-1)[order][:, None].to(yb.dtype)
    out = torch.zeros_like(x)
    out.index_add_(0, token_of, yb)
    return out
