"""Sequence parallelism: groups, zig-zag layout, halo exchange, state transport, loss reduction.

Layout (same contract as the reference project's data split,
``data/processor/sequence_parallel.py:5-47``): a sequence of length ``L`` is cut into
``2*SP`` chunks; rank ``r`` owns chunk ``r`` followed by chunk ``2*SP-1-r``, which balances
causal-attention work.  Position ids travel with the data, so RoPE and masks are computed
from true positions.

What crosses ranks, per layer type:

* SSM mixers: a ``K-1`` token convolution halo (:func:`conv_halo_exchange`) and the
  recurrent state (``StateTransport`` used by ``ops.scan.ssm_scan``);
* sliding-window / B'MOJO attention: a window-sized K/V halo (:func:`halo_exchange`);
* full attention: K/V of all ranks (``parallel.cp_attention``);
* the loss: two scalars (:func:`reduce_loss`).

SP groups are contiguous blocks of ``sp_size`` global ranks
(reference: ``model/model_utils/sequence_parallel.py:104-142``).
"""
from __future__ import annotations

import os

from dataclasses import dataclass, field
from typing import List, Optional, Sequence, Tuple

import torch
import torch.distributed as dist

Tensor = torch.Tensor


# ----------------------------------------------------------------------------------------
# zig-zag layout helpers (pure indexing, no communication)
# ----------------------------------------------------------------------------------------
def zigzag_chunk_ids(rank: int, sp_size: int) -> Tuple[int, int]:
    return rank, 2 * sp_size - 1 - rank


def zigzag_split(x: Tensor, rank: int, sp_size: int, dim: int = 1) -> Tensor:
    """Local shard ``[chunk r ; chunk 2SP-1-r]`` of a full-sequence tensor."""
    L = x.shape[dim]
    assert L % (2 * sp_size) == 0, f"sequence length {L} must be divisible by 2*SP={2 * sp_size}"
    chunks = x.chunk(2 * sp_size, dim=dim)
    a, b = zigzag_chunk_ids(rank, sp_size)
    return torch.cat([chunks[a], chunks[b]], dim=dim)


def zigzag_merge(shards: Sequence[Tensor], dim: int = 1) -> Tensor:
    """Inverse of :func:`zigzag_split` given the shards of all ranks in rank order."""
    n = len(shards)
    chunks: List[Optional[Tensor]] = [None] * (2 * n)
    for r, s in enumerate(shards):
        a, b = s.chunk(2, dim=dim)
        chunks[r], chunks[2 * n - 1 - r] = a, b
    return torch.cat(chunks, dim=dim)


def zigzag_positions(seq_len: int, rank: int, sp_size: int, device=None) -> Tensor:
    return zigzag_split(torch.arange(seq_len, device=device)[None], rank, sp_size, dim=1)[0]


# ----------------------------------------------------------------------------------------
# state transport over a process group (gloo on CPU, NCCL on GPU)
# ----------------------------------------------------------------------------------------
class StateTransport:
    """Blocking point-to-point transport of recurrent states along the zig-zag chain.

    ``ops.scan`` calls it in a fixed, rank-consistent order so that blocking send/recv pairs
    always match.  The GPU fast path replaces it with ``parallel.peer.PeerStateTransport``,
    which pushes the state into the next rank's symmetric buffer from inside the scan kernel.
    """

    def __init__(self, group, ranks: Sequence[int]):
        self.group = group
        self.ranks = list(ranks)
        self.bytes_sent = 0
        self.messages = 0

    def _global(self, r: int) -> int:
        return self.ranks[r]

    def send_state(self, state, dst: int, tag: str = "") -> None:
        if state is None:
            return
        for s in state:
            if s is None:
                continue
            buf = s.contiguous()
            dist.send(buf, dst=self._global(dst), group=self.group)
            self.bytes_sent += buf.numel() * buf.element_size()
            self.messages += 1

    def recv_state(self, core, seg_inputs, src: int, tag: str = ""):
        shapes = core.state_shapes(seg_inputs)
        device = next(t.device for t in seg_inputs if t is not None)
        out = []
        for shape, dtype in shapes:
            if shape is None:
                out.append(None)
                continue
            buf = torch.empty(shape, dtype=dtype, device=device)
            dist.recv(buf, src=self._global(src), group=self.group)
            out.append(buf)
        return tuple(out)

    def recv_state_like(self, templates, device, src: int, tag: str = ""):
        """``templates``: ``(shape, dtype)`` per state tensor (``None`` for absent ones)."""
        out = []
        for t in templates:
            if t is None or len(t[0]) == 0:
                out.append(None)
                continue
            buf = torch.empty(t[0], dtype=t[1], device=device)
            dist.recv(buf, src=self._global(src), group=self.group)
            out.append(buf)
        return tuple(out)


@dataclass
class SPContext:
    """Everything a layer needs to know about sequence parallelism."""
    group: object
    rank: int
    size: int
    ranks: List[int]
    transport: StateTransport = field(default=None)
    mode: str = "zigzag"
    # scan cores with a scalar state transition (GLA, Mamba2 SSD, the GKA covariance) skip the serial state chain:
    # two local passes and one all-gather instead of 2 * size dependent links (``ops/scan.py``)
    parallel_scan: bool = field(default_factory=lambda: os.environ.get("HMF_SP_PARALLEL_SCAN", "0") in ("1", "2"))
    # also for the delta rule (matrix transition, one extra probing scan per segment): HMF_SP_PARALLEL_SCAN=2
    parallel_scan_matrix: bool = field(default_factory=lambda: os.environ.get("HMF_SP_PARALLEL_SCAN", "0") == "2")

    def __post_init__(self):
        if self.transport is None:
            self.transport = StateTransport(self.group, self.ranks)


_SP_CONTEXT: Optional[SPContext] = None


def init_sp_group(sp_size: int) -> Optional[SPContext]:
    """Creates the SP groups (contiguous blocks of ``sp_size`` ranks) and returns this rank's
    context; ``None`` when ``sp_size <= 1``."""
    global _SP_CONTEXT
    if sp_size <= 1:
        _SP_CONTEXT = None
        return None
    world = dist.get_world_size()
    assert world % sp_size == 0, f"world size {world} not divisible by sequence_parallel_size {sp_size}"
    me = dist.get_rank()
    ctx = None
    for start in range(0, world, sp_size):
        ranks = list(range(start, start + sp_size))
        g = dist.new_group(ranks)
        if me in ranks:
            ctx = SPContext(group=g, rank=ranks.index(me), size=sp_size, ranks=ranks)
    _SP_CONTEXT = ctx
    return ctx


def get_sp_context() -> Optional[SPContext]:
    return _SP_CONTEXT


def set_sequence_parallel_group_recursive(module: torch.nn.Module, sp: Optional[SPContext]) -> None:
    """Stores the SP context on every sub-module that declares ``sequence_parallel_group``
    (reference: ``train/pt/workflow.py:35-39``)."""
    for m in module.modules():
        if hasattr(m, "sequence_parallel_group"):
            m.sequence_parallel_group = sp


# ----------------------------------------------------------------------------------------
# halo exchange: last `halo` tokens of the preceding chunk for both local segments
# ----------------------------------------------------------------------------------------
def _exchange(sp: SPContext, send_next, send_prev, need_prev: bool, need_next: bool, like_prev, like_next):
    """send_next goes to rank+1, send_prev to rank-1; receives from rank-1 / rank+1."""
    ops, recv_prev, recv_next = [], None, None
    r, n = sp.rank, sp.size
    if r < n - 1 and send_next is not None:
        ops.append(dist.P2POp(dist.isend, send_next.contiguous(), sp.ranks[r + 1], sp.group))
    if r > 0 and send_prev is not None:
        ops.append(dist.P2POp(dist.isend, send_prev.contiguous(), sp.ranks[r - 1], sp.group))
    if r > 0 and need_prev:
        recv_prev = torch.empty_like(like_prev)
        ops.append(dist.P2POp(dist.irecv, recv_prev, sp.ranks[r - 1], sp.group))
    if r < n - 1 and need_next:
        recv_next = torch.empty_like(like_next)
        ops.append(dist.P2POp(dist.irecv, recv_next, sp.ranks[r + 1], sp.group))
    if ops:
        for w in dist.batch_isend_irecv(ops):
            w.wait()
    return recv_prev, recv_next


class _HaloExchange(torch.autograd.Function):
    """Returns ``[B, 2, halo, ...]``: for each of the two local segments the ``halo`` tokens that
    precede it in the global sequence (zeros before position 0)."""

    @staticmethod
    def forward(ctx, x: Tensor, sp: SPContext, halo: int):
        ctx.sp, ctx.halo = sp, halo
        ctx.x_shape = tuple(x.shape)
        r, n = sp.rank, sp.size
        half = x.shape[1] // 2
        tail_a = x[:, half - halo:half]
        tail_b = x[:, 2 * half - halo:]
        # segment A (chunk r) is preceded by chunk r-1 = segment A of rank r-1
        # segment B (chunk 2n-1-r) is preceded by chunk 2n-2-r = segment B of rank r+1,
        # or by this rank's own segment A when r == n-1
        halo_a, halo_b = _exchange(sp, send_next=tail_a, send_prev=tail_b, need_prev=True, need_next=True,
                                   like_prev=tail_a, like_next=tail_b)
        if halo_a is None:
            halo_a = torch.zeros_like(tail_a)
        if halo_b is None:
            halo_b = tail_a.clone()
        return torch.stack([halo_a, halo_b], dim=1)

    @staticmethod
    def backward(ctx, d_halo: Tensor):
        sp, halo = ctx.sp, ctx.halo
        r, n = sp.rank, sp.size
        d_a, d_b = d_halo[:, 0].contiguous(), d_halo[:, 1].contiguous()
        # gradient of halo_a belongs to rank r-1's tail_a; of halo_b to rank r+1's tail_b
        g_from_next, g_from_prev = None, None
        ops = []
        if r > 0:
            ops.append(dist.P2POp(dist.isend, d_a, sp.ranks[r - 1], sp.group))
        if r < n - 1:
            ops.append(dist.P2POp(dist.isend, d_b, sp.ranks[r + 1], sp.group))
            g_from_next = torch.empty_like(d_a)
            ops.append(dist.P2POp(dist.irecv, g_from_next, sp.ranks[r + 1], sp.group))
        if r > 0:
            g_from_prev = torch.empty_like(d_b)
            ops.append(dist.P2POp(dist.irecv, g_from_prev, sp.ranks[r - 1], sp.group))
        if ops:
            for w in dist.batch_isend_irecv(ops):
                w.wait()
        dx_tail_a = g_from_next if g_from_next is not None else d_b  # r == n-1: own segment A fed halo_b
        dx_tail_b = g_from_prev
        ctx_shape = ctx.x_shape
        dx = d_halo.new_zeros(ctx_shape)
        half = ctx_shape[1] // 2
        dx[:, half - halo:half] += dx_tail_a
        if dx_tail_b is not None:
            dx[:, 2 * half - halo:] += dx_tail_b
        return dx, None, None


def halo_exchange(x: Tensor, sp: SPContext, halo: int) -> Tensor:
    """``x [B, L_local, ...]`` -> halos ``[B, 2, halo, ...]`` for the two zig-zag segments."""
    assert x.shape[1] % 2 == 0 and halo <= x.shape[1] // 2
    return _HaloExchange.apply(x, sp, halo)


def segments_with_halo(x: Tensor, sp: Optional[SPContext], halo: int) -> Tuple[Tensor, Optional[Tensor]]:
    """Reshapes local tokens ``[B, L, C]`` into per-segment rows ``[S*B, L/S, C]`` (``S`` = 2 under
    SP, else 1) and returns the matching halos ``[S*B, halo, C]`` (``None`` without SP)."""
    if sp is None or sp.size == 1:
        return x, None
    B, L = x.shape[0], x.shape[1]
    h = halo_exchange(x, sp, halo)  # [B, 2, halo, C]
    seg = x.reshape(B, 2, L // 2, *x.shape[2:])
    seg = seg.transpose(0, 1).reshape(2 * B, L // 2, *x.shape[2:])
    h = h.transpose(0, 1).reshape(2 * B, halo, *x.shape[2:])
    return seg, h


def merge_segments(y: Tensor, sp: Optional[SPContext]) -> Tensor:
    """Inverse of the segment reshape of :func:`segments_with_halo`."""
    if sp is None or sp.size == 1:
        return y
    B2, Lh = y.shape[0], y.shape[1]
    B = B2 // 2
    return y.reshape(2, B, Lh, *y.shape[2:]).transpose(0, 1).reshape(B, 2 * Lh, *y.shape[2:])


# ----------------------------------------------------------------------------------------
# loss reduction over the SP group
# ----------------------------------------------------------------------------------------
def reduce_loss(loss_sum: Tensor, n_valid: Tensor, sp: Optional[SPContext]) -> Tuple[Tensor, Tensor]:
    """Mean loss over all valid tokens of the SP group.

    The returned loss keeps the autograd graph of the local sum only, divided by the global
    count: summing parameter gradients over the SP ranks then yields the gradient of the
    global mean (reference: ``train/pt/trainer.py:162-195``)."""
    if sp is None or sp.size == 1:
        return loss_sum / n_valid.clamp(min=1), n_valid
    count = n_valid.detach().clone().float()
    dist.all_reduce(count, group=sp.group)
    total = loss_sum.detach().clone().float()
    dist.all_reduce(total, group=sp.group)
    count = count.clamp(min=1)
    # value = global mean; gradient = d(local_sum)/global_count
    local = loss_sum / count
    return local + (total / count - local).detach(), count
