"""Tensor parallelism for serving: head-wise sharding of every mixer, column/row-parallel MLP and experts,
vocabulary-parallel ``lm_head``.

``shard_model(model, tp)`` slices the parameters of a fully materialised model **in place** and rewrites the
head-count attributes of each mixer, so the unchanged layer code computes this rank's heads; every mixer
and MLP output then needs one sum over the TP group (``TPContext.all_reduce``), and the logits one
gather over the vocabulary (``TPContext.gather_logits``).  The reference gets the same split from vLLM's
``ColumnParallelLinear`` / ``RowParallelLinear`` and its sharded weight loaders
(``vllm-inference/src/primed_vllm/layers/primed_gdn_layer.py``, ``primed_mamba2_layer.py``,
``primed_gka_layer.py``).

The all-reduce after a row-parallel GEMM is a reduce-scatter + all-gather; ``ops/fused_comm.py`` provides
the fused GEMM + reduce over peer memory for the decode-size case, this module falls back to NCCL.
"""
from __future__ import annotations

from typing import Optional, Sequence

import torch
import torch.distributed as dist
import torch.nn as nn


class TPContext:
    def __init__(self, group=None, rank: Optional[int] = None, size: Optional[int] = None):
        self.group = group
        self.rank = dist.get_rank(group) if rank is None else rank
        self.size = dist.get_world_size(group) if size is None else size
        self.fused_gemm = None     # optional ops.fused_comm.PeerGemmAllReduce (GEMM + all-reduce in one kernel)

    def enable_fused_gemm(self, max_m: int = 256, max_n: int = 8192) -> bool:
        """Sets up the peer-memory GEMM + all-reduce kernel (collective call; GPU ranks of one node)."""
        if self.size == 1 or not torch.cuda.is_available():
            return False
        from ..ops.fused_comm import PeerGemmAllReduce
        self.fused_gemm = PeerGemmAllReduce(self.group, max_m, max_n)
        return True

    def linear_allreduce(self, x: torch.Tensor, weight: torch.Tensor) -> torch.Tensor:
        """``all_reduce(x @ weight^T)`` for a row-parallel weight shard ``[N, K / size]``."""
        if self.size > 1 and self.fused_gemm is not None and self.fused_gemm.accepts(x, weight):
            return self.fused_gemm(x, weight)
        return self.all_reduce(torch.nn.functional.linear(x, weight))

    def all_reduce(self, x: torch.Tensor) -> torch.Tensor:
        if self.size == 1:
            return x
        x = x.contiguous()
        dist.all_reduce(x, group=self.group)
        return x

    def gather_logits(self, logits: torch.Tensor) -> torch.Tensor:
        if self.size == 1:
            return logits
        parts = [torch.empty_like(logits) for _ in range(self.size)]
        dist.all_gather(parts, logits.contiguous(), group=self.group)
        return torch.cat(parts, dim=-1)


# -- slicing helpers ---------------------------------------------------------------------------------
def _rows(t: torch.Tensor, rank: int, size: int, segments: Optional[Sequence[int]] = None) -> torch.Tensor:
    """Rank's share of dim 0.  With ``segments`` the dim is a concatenation of blocks and every block is
    split separately (``[z | x | B | C | dt]`` of Mamba2's ``in_proj``)."""
    if segments is None:
        n = t.shape[0]
        assert n % size == 0, f"dimension {n} is not divisible by the TP size {size}"
        return t[rank * n // size:(rank + 1) * n // size].clone()
    assert sum(segments) == t.shape[0]
    out, o = [], 0
    for s in segments:
        assert s % size == 0, f"segment {s} is not divisible by the TP size {size}"
        out.append(t[o + rank * s // size:o + (rank + 1) * s // size])
        o += s
    return torch.cat(out, dim=0).clone()


def _set(p: nn.Parameter, value: torch.Tensor) -> None:
    p.data = value.contiguous()


def column_parallel(lin: nn.Linear, rank, size, segments=None) -> None:
    _set(lin.weight, _rows(lin.weight.data, rank, size, segments))
    if lin.bias is not None:
        _set(lin.bias, _rows(lin.bias.data, rank, size, segments))
    lin.out_features = lin.weight.shape[0]


def row_parallel(lin: nn.Linear, rank, size, segments=None) -> None:
    w = lin.weight.data.t()
    _set(lin.weight, _rows(w, rank, size, segments).t())
    if lin.bias is not None and rank != 0:
        lin.bias.data.zero_()         # the bias is added once, by rank 0's partial sum
    lin.in_features = lin.weight.shape[1]


def _vec(p: nn.Parameter, rank, size, segments=None) -> None:
    _set(p, _rows(p.data, rank, size, segments))


# -- per-module sharding -----------------------------------------------------------------------------
def shard_attention(m, rank, size) -> None:
    assert m.num_kv_heads % size == 0 and m.num_heads % size == 0, "attention heads must divide by the TP size"
    column_parallel(m.q_proj, rank, size)
    column_parallel(m.k_proj, rank, size)
    column_parallel(m.v_proj, rank, size)
    row_parallel(m.o_proj, rank, size)
    m.num_heads //= size
    m.num_kv_heads //= size
    if hasattr(m, "num_kv_groups"):
        m.num_kv_groups = m.num_heads // m.num_kv_heads


def _shard_qkv_family(m, rank, size) -> None:
    """Shared by GDN and GKA: q/k/v (+ convolutions), per-head gates, output gate and projection."""
    for n in (m.num_q_heads, m.num_k_heads, m.num_v_heads):
        assert n % size == 0, "linear-attention heads must divide by the TP size"
    assert getattr(m, "kv_proj_rank", None) is None, "low-rank K/V expansion is not supported under TP"
    for name in ("q_proj", "k_proj", "v_proj", "g_proj", "b_proj", "gk_proj", "a_proj", "alpha_proj"):
        lin = getattr(m, name, None)
        if isinstance(lin, nn.Linear):
            column_parallel(lin, rank, size)
    for name in ("q_conv1d", "k_conv1d", "v_conv1d"):
        cv = getattr(m, name, None)
        if cv is not None:
            _vec(cv.weight, rank, size)
            if cv.bias is not None:
                _vec(cv.bias, rank, size)
            cv.hidden_size //= size
    _vec(m.A_log, rank, size)
    _vec(m.dt_bias, rank, size)
    row_parallel(m.o_proj, rank, size)
    m.num_q_heads //= size
    m.num_k_heads //= size
    m.num_v_heads //= size
    m.expanded_num_heads //= size
    for attr in ("query_dim", "key_dim", "value_dim", "expanded_dim"):
        setattr(m, attr, getattr(m, attr) // size)


def shard_mamba2(m, rank, size) -> None:
    hx = m.d_xb // m.headdim
    assert m.nheads % size == 0 and hx % size == 0, "Mamba2 heads must divide by the TP size"
    column_parallel(m.in_proj, rank, size, [m.d_inner, m.d_xb, m.d_xb, m.d_inner, m.nheads])
    # The shard's output width (d_inner/size * 2 + d_xb/size * 2 + nheads/size) is rarely a multiple of the GEMM tile
    # granularity, and cuBLAS then falls back to a legacy kernel several times slower: pad with zero rows, which the
    # layer slices off again (``in_proj_valid``).
    n = m.in_proj.weight.shape[0]
    pad = (-n) % 64
    if pad:
        w = m.in_proj.weight.data
        _set(m.in_proj.weight, torch.cat([w, w.new_zeros(pad, w.shape[1])], 0))
        if m.in_proj.bias is not None:
            _set(m.in_proj.bias, torch.cat([m.in_proj.bias.data, m.in_proj.bias.data.new_zeros(pad)], 0))
        m.in_proj.out_features = n + pad
    m.in_proj_valid = n
    seg = [m.d_xb, m.d_xb, m.d_inner]
    _vec(m.conv1d.weight, rank, size, seg)
    if m.conv1d.bias is not None:
        _vec(m.conv1d.bias, rank, size, seg)
    for p in (m.dt_bias, m.A_log, m.D, m.norm.weight):
        _vec(p, rank, size)
    row_parallel(m.out_proj, rank, size)
    m.d_inner //= size
    m.d_xb //= size
    m.nheads //= size
    m.ngroups //= size
    m.conv_dim = m.d_inner + 2 * m.d_xb
    m.conv1d.in_channels = m.conv1d.out_channels = m.conv1d.groups = m.conv_dim


def shard_mlp(m, rank, size) -> None:
    column_parallel(m.gate_proj, rank, size)
    column_parallel(m.up_proj, rank, size)
    row_parallel(m.down_proj, rank, size)
    m.intermediate_size //= size


def shard_moe(m, rank, size) -> None:
    """Every expert keeps all tokens but a ``1/size`` slice of its intermediate channels (expert tensor
    parallelism); the router is replicated."""
    gu = m.experts.gate_up_proj.data                      # [E, 2F, Dm] = [gate | up]
    E, F2, Dm = gu.shape
    Fi = F2 // 2
    assert Fi % size == 0
    sl = slice(rank * Fi // size, (rank + 1) * Fi // size)
    _set(m.experts.gate_up_proj, torch.cat([gu[:, :Fi][:, sl], gu[:, Fi:][:, sl]], dim=1))
    _set(m.experts.down_proj, m.experts.down_proj.data[:, :, sl])
    if m.shared_expert is not None:
        shard_mlp(m.shared_expert, rank, size)


def shard_model(model, tp: TPContext):
    """Shards ``model`` (a ``HybridForCausalLM``) for ``tp`` in place and returns it."""
    from ..layers.attention import Attention
    from ..layers.common import MLP
    from ..layers.gdn import GatedDeltaNet
    from ..layers.gka import GatedKalmaNet
    from ..layers.mamba2 import Mamba2
    rank, size = tp.rank, tp.size
    if size == 1:
        return model
    for layer in model.model.layers:
        mx = layer.seq_mixer
        if isinstance(mx, Attention):
            shard_attention(mx, rank, size)
        elif isinstance(mx, (GatedDeltaNet, GatedKalmaNet)):
            _shard_qkv_family(mx, rank, size)
        elif isinstance(mx, Mamba2):
            shard_mamba2(mx, rank, size)
        else:
            raise NotImplementedError(f"tensor parallelism for {type(mx).__name__}")
        if isinstance(layer.mlp, MLP):
            shard_mlp(layer.mlp, rank, size)
        else:
            shard_moe(layer.mlp, rank, size)
    if model.lm_head.weight is model.model.embed_tokens.weight:
        model.lm_head.weight = nn.Parameter(model.lm_head.weight.data.clone(), requires_grad=False)
    column_parallel(model.lm_head, rank, size)
    model._tp = tp
    # partial sums of the row-parallel projections are reduced right after each mixer / MLP
    for layer in model.model.layers:
        layer.seq_mixer.register_forward_hook(_reduce_hook(tp))
        layer.mlp.register_forward_hook(_reduce_hook(tp))
    return model


def _reduce_hook(tp: TPContext):
    def hook(_module, _inputs, output):
        if isinstance(output, tuple):
            return (tp.all_reduce(output[0]),) + tuple(output[1:])
        return tp.all_reduce(output)
    return hook


def init_tp(device: Optional[torch.device] = None) -> TPContext:
    """TP over the default process group (one rank per GPU)."""
    if not dist.is_initialized():
        return TPContext(rank=0, size=1)
    return TPContext(dist.group.WORLD)
