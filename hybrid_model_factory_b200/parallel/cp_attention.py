"""Context-parallel softmax attention for zig-zag sequence parallelism.

Each rank holds queries, keys and values of its two zig-zag chunks.  K and V of all ranks
are gathered (GQA keeps them small: ``Hkv`` heads), put back into global order, and each
local segment attends causally to the key prefix that precedes it; in backward the key /
value gradients are reduced back to their owners.  This replaces the reference project's
ring attention monkey-patch (``model/model_utils/sequence_parallel.py:38-101``).

On GPUs with peer access the gather is not a separate collective: ``ops.cuda_ops`` pulls
remote K/V tiles over NVLink from inside the attention kernel (see ``parallel/peer.py``);
this module is the portable path (gloo on CPU, NCCL baseline on GPU) and the numerical
contract of the fused one.
"""
from __future__ import annotations

import os

from typing import Optional

import torch
import torch.distributed as dist

from ..ops import functional as F_ops
from ..utils.profiling import phase
from .sp import SPContext, zigzag_merge, zigzag_split

Tensor = torch.Tensor


def _all_gather_seq(x: Tensor, sp: SPContext) -> Tensor:
    """Gathers ``[B, L_local, ...]`` shards and returns the sequence in global order."""
    with phase("kv_gather"):
        shards = [torch.empty_like(x) for _ in range(sp.size)]
        dist.all_gather(shards, x.contiguous(), group=sp.group)
        return zigzag_merge(shards, dim=1)


def _reduce_scatter_seq(x_full: Tensor, sp: SPContext) -> Tensor:
    """Sums full-sequence tensors over the group and returns this rank's zig-zag shard."""
    if x_full.is_cuda:
        with phase("dkv_reduce_scatter"):
            parts = [zigzag_split(x_full, r, sp.size, dim=1).contiguous() for r in range(sp.size)]
            out = torch.empty_like(parts[0])
            dist.reduce_scatter(out, parts, group=sp.group)
        return out
    buf = x_full.contiguous()
    dist.all_reduce(buf, group=sp.group)  # gloo has no reduce_scatter
    return zigzag_split(buf, sp.rank, sp.size, dim=1)


class _GatherSeq(torch.autograd.Function):
    """Differentiable all-gather along the sequence: shards in, the whole sequence in global order out; the gradient
    is summed over the group (fp32) and every rank gets back its shard's part."""

    @staticmethod
    def forward(ctx, x: Tensor, sp: SPContext):
        ctx.sp, ctx.dtype = sp, x.dtype
        return _all_gather_seq(x, sp)

    @staticmethod
    def backward(ctx, g: Tensor):
        return _reduce_scatter_seq(g.float(), ctx.sp).to(ctx.dtype), None


def gather_seq(x: Tensor, sp: SPContext) -> Tensor:
    return _GatherSeq.apply(x, sp)


class _CPAttention(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q: Tensor, k: Tensor, v: Tensor, sp: SPContext, scale: Optional[float], window: Optional[int]):
        B, Ll = q.shape[0], q.shape[1]
        c = Ll // 2
        pk = getattr(sp, "peer_kv", None)
        if (pk is not None and not any(ctx.needs_input_grad[:3]) and q.is_cuda and q.dtype == torch.bfloat16
                and k.dtype == torch.bfloat16 and q.shape[-1] in (64, 128) and window is None and pk.fits(k)):
            # no gradient will be asked of this call (inference, or the first pass of a checkpointed layer): the
            # K/V gather happens inside the attention kernel, tile by tile over peer memory
            from ..utils import checkpointing as _ckpt
            D = q.shape[-1]
            sc = D ** -0.5 if scale is None else scale
            pk.publish(k.contiguous(), v.contiguous())
            wr = _ckpt.stash_for_write()
            outs = []
            for seg, cid in ((0, sp.rank), (1, 2 * sp.size - 1 - sp.rank)):
                o, lse = pk.attention(q[:, seg * c:(seg + 1) * c], cid, sc, 0, 2 ** 31 - 1)
                if wr is not None:
                    wr.append((o, lse))
                outs.append(o)
            ctx.graphs = None
            return torch.cat(outs, dim=1)
        k_all = _all_gather_seq(k, sp)
        v_all = _all_gather_seq(v, sp)
        ca, cb = sp.rank, 2 * sp.size - 1 - sp.rank
        ctx.sp, ctx.c, ctx.full_len = sp, c, k_all.shape[1]
        graphs, outs = [], []
        for seg, cid in ((0, ca), (1, cb)):
            end = (cid + 1) * c
            qs = q[:, seg * c:(seg + 1) * c].detach().requires_grad_(True)
            ks = k_all[:, :end].detach().requires_grad_(True)
            vs = v_all[:, :end].detach().requires_grad_(True)
            with torch.enable_grad():
                o = F_ops.attention(qs, ks, vs, scale=scale, causal=True, window=window)
            graphs.append((qs, ks, vs, o))
            outs.append(o.detach())
        ctx.graphs = graphs
        return torch.cat(outs, dim=1)

    @staticmethod
    def backward(ctx, d_o: Tensor):
        sp, c = ctx.sp, ctx.c
        dqs = []
        qs0, ks0, vs0, _ = ctx.graphs[0]
        dk_full = ks0.new_zeros(ks0.shape[0], ctx.full_len, *ks0.shape[2:], dtype=torch.float32)
        dv_full = torch.zeros_like(dk_full)
        for seg, (qs, ks, vs, o) in enumerate(ctx.graphs):
            dq, dk, dv = torch.autograd.grad(o, (qs, ks, vs), d_o[:, seg * c:(seg + 1) * c].to(o.dtype))
            dqs.append(dq)
            dk_full[:, :dk.shape[1]] += dk.float()
            dv_full[:, :dv.shape[1]] += dv.float()
        ctx.graphs = None
        # this rank's two contributions were summed in fp32; the sum over ranks travels in the gradient's own dtype
        # (half the bytes of an fp32 reduce-scatter; the result is stored in that dtype anyway) unless
        # HMF_CP_DKV_FP32=1
        wire = torch.float32 if os.environ.get("HMF_CP_DKV_FP32", "0") == "1" else ks0.dtype
        dk = _reduce_scatter_seq(dk_full.to(wire), sp).to(ks0.dtype)
        dv = _reduce_scatter_seq(dv_full.to(wire), sp).to(vs0.dtype)
        return torch.cat(dqs, dim=1), dk, dv, None, None, None


def cp_attention(q: Tensor, k: Tensor, v: Tensor, sp: SPContext, *, scale: Optional[float] = None,
                 window: Optional[int] = None) -> Tensor:
    """Causal attention of the local zig-zag queries against the whole (distributed) sequence."""
    return _CPAttention.apply(q, k, v, sp, scale, window)
