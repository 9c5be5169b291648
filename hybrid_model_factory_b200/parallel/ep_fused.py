"""Expert parallelism with the all-to-all fused into the grouped expert GEMMs (forward / inference path).

Per MoE layer and rank:
  1. local tokens are sorted by (owner rank, local expert) into this rank's *send buffer* (symmetric memory) and
     the per-(rank, expert) counts are published next to it; a release flag announces both to every peer;
  2. a one-thread kernel reads every peer's counts (after its flag) and builds the segment / tile tables on the
     device (no host synchronisation);
  3. grouped GEMM 1 (gate/up projection) pulls its A tiles by TMA directly from the source ranks' send buffers —
     the dispatch all-to-all never exists as a separate transfer;
  4. packed SwiGLU;
  5. grouped GEMM 2 (down projection) stores every output row directly into the source rank's *receive buffer*
     — the combine all-to-all is the GEMM epilogue; a flag after the kernel marks the rows complete;
  6. the owner waits (bounded, on the device) for all peers' flags and applies the routing weights.
Kernels: ``csrc/kernels/moe_grouped_gemm.cu``.  With ``group=None`` the same code is the single-GPU grouped-GEMM MoE.
The differentiable NCCL path for training is ``parallel/ep.py``.  (The reference serves MoE through vLLM's
``SharedFusedMoE`` with NCCL all-to-all, ``hybridqwen3_moe.py:913-1263``.)
"""
from __future__ import annotations

import ctypes
from typing import Optional

import torch

from ..ops import _lib

c_int, c_uint, c_ll = ctypes.c_int, ctypes.c_uint, ctypes.c_longlong
MAX_RANKS = 8


class FusedExpertParallel:
    def __init__(self, group, e_local: int, hidden: int, inter: int, max_send_rows: int, capacity_rows: int,
                 device: Optional[torch.device] = None):
        self.e_local, self.Dm, self.F = e_local, hidden, inter
        self.max_send, self.capacity = int(max_send_rows), int(capacity_rows)
        row_bytes = hidden * 2
        self.off_send = 0
        self.off_recv = self._al(self.max_send * row_bytes)
        self.off_cnt = self.off_recv + self._al(self.max_send * row_bytes)
        if group is None:
            self.rank, self.world = 0, 1
            dev = device or torch.device("cuda", torch.cuda.current_device())
        else:
            import torch.distributed as dist
            self.rank, self.world = dist.get_rank(group), dist.get_world_size(group)
            dev = device or torch.device("cuda", torch.cuda.current_device())
        assert self.world <= MAX_RANKS
        self.off_f1 = self.off_cnt + self._al(self.world * e_local * 4)
        self.off_f2 = self.off_f1 + 1024
        total = self.off_f2 + 1024
        if group is None:
            self.buf = torch.zeros(total, dtype=torch.uint8, device=dev)
            bases = [self.buf.data_ptr()]
        else:
            from .peer import SymmetricWorkspace
            self.ws = SymmetricWorkspace(total, group, dev)
            self.buf = self.ws.buffer
            bases = [self.ws.peer_ptr(r) for r in range(self.world)]
        self.bases = bases
        v = lambda off, shape, dt: self.buf[off:off + _numel(shape) * _esize(dt)].view(dt).view(*shape)  # noqa: E731
        self.send = v(self.off_send, (self.max_send, hidden), torch.bfloat16)
        self.recv = v(self.off_recv, (self.max_send, hidden), torch.bfloat16)
        self.cnt = v(self.off_cnt, (self.world * e_local,), torch.int32)
        self.flags1 = v(self.off_f1, (self.world,), torch.int32)
        self.flags2 = v(self.off_f2, (self.world,), torch.int32)
        i64 = lambda xs: torch.tensor(xs, dtype=torch.int64, device=dev)  # noqa: E731
        self.cnt_ptrs = i64([b + self.off_cnt for b in bases])
        self.f1_ptrs = i64([b + self.off_f1 for b in bases])
        self.f2_ptrs = i64([b + self.off_f2 for b in bases])
        nseg = self.world * e_local
        self.max_mtiles = self.capacity // 128 + nseg + 1
        self.seg1 = torch.zeros(6 * nseg, dtype=torch.int32, device=dev)
        self.seg2 = torch.zeros(6 * nseg, dtype=torch.int32, device=dev)
        self.mtile = torch.zeros(2 * self.max_mtiles, dtype=torch.int32, device=dev)
        self.counts = torch.zeros(4, dtype=torch.int32, device=dev)
        self.h = torch.empty(self.capacity + 128, 2 * inter, dtype=torch.bfloat16, device=dev)
        self.a = torch.zeros(self.capacity + 128, inter, dtype=torch.bfloat16, device=dev)
        self.maps = torch.empty(4 * MAX_RANKS * 128 + 64, dtype=torch.uint8, device=dev)
        self.sm_count = torch.cuda.get_device_properties(dev).multi_processor_count
        self.epoch = 0
        self.calls = 0

    @staticmethod
    def _al(n: int) -> int:
        return (n + 1023) // 1024 * 1024

    def _maps_slot(self) -> ctypes.c_void_p:
        base = (self.maps.data_ptr() + 63) // 64 * 64
        slot = base + (self.calls % 4) * MAX_RANKS * 128
        self.calls += 1
        return ctypes.c_void_p(slot)

    @torch.no_grad()
    def forward(self, x: torch.Tensor, weights: torch.Tensor, indices: torch.Tensor, w_gate_up: torch.Tensor,
                w_down: torch.Tensor) -> torch.Tensor:
        K = _lib.kernels()
        T, k = indices.shape
        n = T * k
        assert n <= self.max_send, f"{n} routed rows exceed the send buffer ({self.max_send})"
        st = _lib.stream_ptr(x.device)
        flat_e = indices.reshape(-1)
        order = torch.argsort(flat_e, stable=True)
        token_of = order // k
        self.cnt.copy_(torch.bincount(flat_e, minlength=self.world * self.e_local).to(torch.int32))
        torch.index_select(x, 0, token_of, out=self.send[:n])
        self.epoch += 1
        ep = c_uint(self.epoch)
        _lib.check(K.hmf_peer_signal(_lib.ptr(self.f1_ptrs), c_int(self.world), c_int(self.rank), ep, st), "peer_signal")
        _lib.check(K.hmf_moe_build_tables(_lib.ptr(self.cnt_ptrs), _lib.ptr(self.flags1), ep, c_int(self.world),
                                          c_int(self.rank), c_int(self.e_local), c_int(self.capacity),
                                          c_int(self.max_mtiles), _lib.ptr(self.seg1), _lib.ptr(self.seg2),
                                          _lib.ptr(self.mtile), _lib.ptr(self.counts), st), "moe_build_tables")
        u64 = ctypes.c_ulonglong
        # GEMM 1: pull token rows from the source ranks' send buffers, write h locally
        a_ptrs = (u64 * MAX_RANKS)(*[b + self.off_send for b in self.bases], *([0] * (MAX_RANKS - self.world)))
        out1 = (u64 * (MAX_RANKS + 1))(*([0] * MAX_RANKS), self.h.data_ptr())
        _lib.check(K.hmf_moe_grouped_gemm(a_ptrs, c_int(self.world), c_ll(self.max_send), self._maps_slot(),
                                          _lib.ptr(w_gate_up), c_int(self.e_local), c_int(2 * self.F), c_int(self.Dm),
                                          out1, c_ll(2 * self.F), _lib.ptr(self.seg1), _lib.ptr(self.mtile),
                                          _lib.ptr(self.counts), None, ep, c_int(self.sm_count), st), "moe_gemm1")
        _lib.check(K.hmf_swiglu_packed(_lib.ptr(self.h), _lib.ptr(self.a), c_ll(self.capacity), c_int(self.F),
                                       c_ll(2 * self.F), st), "swiglu_packed")
        # GEMM 2: read a locally, push result rows into the source ranks' receive buffers
        a2 = (u64 * MAX_RANKS)(self.a.data_ptr(), *([0] * (MAX_RANKS - 1)))
        out2 = (u64 * (MAX_RANKS + 1))(*[b + self.off_recv for b in self.bases], *([0] * (MAX_RANKS - self.world)), 0)
        _lib.check(K.hmf_moe_grouped_gemm(a2, c_int(1), c_ll(self.capacity + 128), self._maps_slot(), _lib.ptr(w_down),
                                          c_int(self.e_local), c_int(self.Dm), c_int(self.F), out2, c_ll(self.Dm),
                                          _lib.ptr(self.seg2), _lib.ptr(self.mtile), _lib.ptr(self.counts), None, ep,
                                          c_int(self.sm_count), st), "moe_gemm2")
        _lib.check(K.hmf_peer_signal(_lib.ptr(self.f2_ptrs), c_int(self.world), c_int(self.rank), ep, st), "peer_signal")
        _lib.check(K.hmf_peer_wait(_lib.ptr(self.flags2), c_int(self.world), ep, st), "peer_wait")
        y = self.recv[:n] * weights.reshape(-1)[order][:, None].to(torch.bfloat16)
        out = torch.zeros_like(x)
        out.index_add_(0, token_of, y)
        return out


def _numel(shape) -> int:
    n = 1
    for s in shape:
        n *= int(s)
    return n


def _esize(dt) -> int:
    return torch.empty((), dtype=dt).element_size()


def attach_fused_moe(model, group=None, max_tokens: int = 8192) -> int:
    """Gives every ``SparseMoeBlock`` of ``model`` the grouped-GEMM inference path.  With ``group`` the experts are
    sharded over its ranks first (expert parallelism) and the all-to-all runs inside the GEMMs.  One workspace is
    shared by all layers (they run one after the other).  Returns the number of blocks attached."""
    from ..models.modeling_hybrid import SparseMoeBlock
    from .ep import EPContext, shard_experts
    blocks = [m for m in model.modules() if isinstance(m, SparseMoeBlock)]
    if not blocks:
        return 0
    world = 1
    if group is not None:
        ctx = EPContext.from_group(group)
        world = ctx.size
        for b in blocks:
            if b.expert_parallel_group is None:
                shard_experts(b, ctx)
    b0 = blocks[0]
    e_local, two_f, dm = b0.experts.gate_up_proj.shape
    rows = max_tokens * b0.top_k
    shared = FusedExpertParallel(group, e_local, dm, two_f // 2, max_send_rows=rows, capacity_rows=rows * min(world, 4),
                                 device=b0.experts.gate_up_proj.device)
    for b in blocks:
        b.fused_ep = shared
    return len(blocks)
