"""Peer-memory plumbing: symmetric buffers whose address on every rank of a group is known to every other
rank, so kernels can load / store a neighbour's memory over NVLink directly.

``SymmetricWorkspace`` wraps ``torch.distributed._symmetric_memory`` (CUDA VMM allocation + handle exchange;
one process per GPU, single node).  Users:

* ``PeerStateTransport`` — sequence-parallel state chain of the SSM scans: the scan kernel of rank ``r``
  stores its final recurrent state into the *next* rank's buffer and raises a per-(batch, head) flag; the
  next rank's kernel, already launched, starts its recurrence when the flag arrives
  (``csrc/kernels/gdn_scan.cu``).  No host synchronisation, no separate send/recv kernels.  The reference
  passes these states with blocking NCCL send/recv around the kernels
  (``layers/gated_kalmanet/sequence_parallel/gka_sp_utils.py:113-226``).
* ``ops/fused_comm.py`` — tensor-parallel GEMM + all-reduce and the peer all-reduce of the decode step.
* ``parallel/cp_attention.py`` — context-parallel attention reading remote K/V tiles by TMA.

Flags are monotonically increasing epochs, never reset: a reader waits for ``flag >= epoch``.  A buffer is
reused every epoch; the chain's data dependencies order the reuse (the writer of epoch ``e+1`` has, through the
opposite chain of epoch ``e``, already waited for the reader of epoch ``e``).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional

import torch
import torch.distributed as dist

from .sp import StateTransport


class SymmetricWorkspace:
    """``nbytes`` of symmetric memory on every rank of ``group``; ``ptrs[r]`` is rank ``r``'s base address as
    mapped into this process."""

    def __init__(self, nbytes: int, group, device: Optional[torch.device] = None):
        self.group = group
        self.device = device or torch.device("cuda", torch.cuda.current_device())
        nbytes = (int(nbytes) + 1023) // 1024 * 1024
        if group is None:       # one rank: ordinary device memory, the only "peer" is this GPU
            self.buffer = torch.zeros(nbytes, dtype=torch.uint8, device=self.device)
            self.handle, self.rank, self.world = None, 0, 1
            self.ptrs = [self.buffer.data_ptr()]
            self.nbytes = nbytes
            self.multicast_ptr = 0
            return
        import torch.distributed._symmetric_memory as symm_mem
        self.buffer = symm_mem.empty(nbytes, dtype=torch.uint8, device=self.device)
        self.handle = symm_mem.rendezvous(self.buffer, group)
        self.rank, self.world = self.handle.rank, self.handle.world_size
        self.ptrs: List[int] = [int(p) for p in self.handle.buffer_ptrs]
        self.nbytes = nbytes
        # address of the same buffer through its NVSwitch multicast object (0 where NVLS is not available)
        try:
            self.multicast_ptr = int(getattr(self.handle, "multicast_ptr", 0) or 0)
        except Exception:
            self.multicast_ptr = 0
        self.buffer.zero_()
        torch.cuda.synchronize(self.device)
        dist.barrier(group=group)

    def view(self, offset: int, shape, dtype) -> torch.Tensor:
        n = 1
        for s in shape:
            n *= int(s)
        nbytes = n * torch.empty((), dtype=dtype).element_size()
        assert offset % 16 == 0 and offset + nbytes <= self.nbytes, "symmetric workspace view out of range"
        return self.buffer[offset:offset + nbytes].view(dtype).view(*shape)

    def peer_ptr(self, rank: int, offset: int = 0) -> int:
        return self.ptrs[rank] + offset

    def barrier(self) -> None:
        """All kernels launched so far on every rank of the group have finished."""
        torch.cuda.synchronize(self.device)
        if self.group is not None:
            dist.barrier(group=self.group)


@dataclass
class PeerIO:
    """What one scan launch needs to take part in the state chain."""
    recv: Optional[torch.Tensor]        # local symmetric buffer the previous rank writes (None: chain start)
    recv_flag: Optional[torch.Tensor]   # [BH] uint32 epochs, local
    push_ptr: int                       # address of the next rank's buffer (0: chain end)
    push_flag_ptr: int
    epoch: int


class PeerStateTransport(StateTransport):
    """State chain over peer memory for scan cores that implement the in-kernel push / wait
    (``core.peer_capable(inputs)``); every other core falls back to the NCCL send/recv of the base class."""

    TAGS = ("fwd_a", "fwd_b", "bwd_a", "bwd_b")

    def __init__(self, group, ranks, sp_rank: int, max_state_bytes: int = 8 << 20, max_bh: int = 4096):
        super().__init__(group, ranks)
        self.sp_rank, self.size = sp_rank, len(ranks)
        self.state_bytes = (max_state_bytes + 1023) // 1024 * 1024
        self.flag_bytes = (max_bh * 4 + 1023) // 1024 * 1024
        self.slot = self.state_bytes + self.flag_bytes
        self.ws = SymmetricWorkspace(self.slot * len(self.TAGS), group)
        self.epochs: Dict[str, int] = {t: 0 for t in self.TAGS}
        self.max_bh = max_bh
        self.fused_messages = 0

    def fits(self, shape, dtype, bh: int) -> bool:
        n = 1
        for s in shape:
            n *= int(s)
        return n * torch.empty((), dtype=dtype).element_size() <= self.state_bytes and bh <= self.max_bh

    def peer_io(self, tag: str, shape, bh: int, recv_from: Optional[int], send_to: Optional[int]) -> PeerIO:
        """``recv_from`` / ``send_to`` are SP ranks (or ``None``).  Every rank of the group must call this for
        the same sequence of tags, whether or not it receives or sends (the epoch counters advance in step)."""
        i = self.TAGS.index(tag)
        self.epochs[tag] += 1
        epoch = self.epochs[tag]
        base = i * self.slot
        recv = recv_flag = None
        if recv_from is not None:
            recv = self.ws.view(base, shape, torch.float32)
            recv_flag = self.ws.view(base + self.state_bytes, (bh,), torch.int32)
        push_ptr = push_flag_ptr = 0
        if send_to is not None:
            push_ptr = self.ws.peer_ptr(send_to, base)
            push_flag_ptr = self.ws.peer_ptr(send_to, base + self.state_bytes)
            self.fused_messages += 1
        return PeerIO(recv, recv_flag, push_ptr, push_flag_ptr, epoch)


def enable_peer_transport(sp, max_state_bytes: int = 8 << 20) -> bool:
    """Replaces the NCCL state transport of an ``SPContext`` by the peer-memory one.  Returns False (and leaves
    the context unchanged) when symmetric memory cannot be set up (CPU ranks, no P2P access)."""
    if sp is None or sp.size <= 1 or not torch.cuda.is_available():
        return False
    try:
        sp.transport = PeerStateTransport(sp.group, sp.ranks, sp.rank, max_state_bytes)
        return True
    except Exception as e:  # pragma: no cover - depends on the machine
        import warnings
        warnings.warn(f"peer-memory state transport unavailable ({e}); using NCCL send/recv")
        return False


class PeerKVExchange:
    """Keys / values of context-parallel attention in symmetric memory.

    ``publish(k, v)`` copies this rank's ``[B, T_local, Hkv, D]`` tensors into its (double-buffered) symmetric slot
    and raises ``flag[rank] = epoch`` on every peer.  ``attention(q_seg, ...)`` then runs the forward kernel whose
    TMA producer fetches every K/V tile straight from the owner's memory (non-multicast TMA over NVLink) after
    seeing that owner's flag: the all-gather of the unfused path disappears into the attention kernel.
    Double-buffering is enough: finishing the attention of layer ``l+1`` requires every peer's layer ``l+1`` flags,
    which a peer raises only after its own layer-``l`` attention has finished reading.
    """

    def __init__(self, group, sp_rank: int, sp_size: int, max_kv_bytes: int):
        self.rank, self.size = sp_rank, sp_size
        self.kv_bytes = (int(max_kv_bytes) + 1023) // 1024 * 1024
        self.flag_off = 4 * self.kv_bytes                       # [parity][k | v]
        self.ws = SymmetricWorkspace(self.flag_off + 1024, group)
        dev = self.ws.device
        self.flags = self.ws.view(self.flag_off, (sp_size,), torch.int32)
        self.flag_ptrs = torch.tensor([self.ws.peer_ptr(r, self.flag_off) for r in range(sp_size)], dtype=torch.int64,
                                      device=dev)
        self.maps = torch.empty(8 * 2 * 2 * sp_size * 128 + 64, dtype=torch.uint8, device=dev)
        self.calls = 0
        self.epoch = 0
        self.shape = None

    def fits(self, k: torch.Tensor) -> bool:
        return k.numel() * k.element_size() <= self.kv_bytes and k.shape[1] % 2 == 0 and (k.shape[1] // 2) % 64 == 0

    def _slot(self, which: int) -> int:
        return ((self.epoch & 1) * 2 + which) * self.kv_bytes

    def publish(self, k: torch.Tensor, v: torch.Tensor) -> None:
        import ctypes
        from ..ops import _lib
        self.epoch += 1
        self.shape = tuple(k.shape)
        self.ws.view(self._slot(0), k.shape, k.dtype).copy_(k)
        self.ws.view(self._slot(1), v.shape, v.dtype).copy_(v)
        _lib.check(_lib.kernels().hmf_peer_signal(_lib.ptr(self.flag_ptrs), ctypes.c_int(self.size),
                                                  ctypes.c_int(self.rank), ctypes.c_uint(self.epoch),
                                                  _lib.stream_ptr(k.device)), "peer_signal")

    def attention(self, q_seg: torch.Tensor, chunk_id: int, scale: float, lo: int, hi: int):
        """Causal attention of the queries of global chunk ``chunk_id`` against chunks ``0 .. chunk_id``."""
        import ctypes
        from ..ops import _lib
        B, T, Hkv, D = self.shape
        Lc, n = T // 2, self.size
        n_chunks = 2 * n
        arr = (ctypes.c_ulonglong * (2 * n_chunks))()
        for c in range(n_chunks):
            owner = c if c < n else n_chunks - 1 - c
            off = (0 if c < n else Lc) * Hkv * D * 2
            arr[c] = self.ws.peer_ptr(owner, self._slot(0) + off)
            arr[n_chunks + c] = self.ws.peer_ptr(owner, self._slot(1) + off)
        Bq, Tq, Hq, _ = q_seg.shape
        q_seg = q_seg if (q_seg.stride(3) == 1 and q_seg.data_ptr() % 16 == 0) else q_seg.contiguous()
        o = torch.empty(Bq, Tq, Hq, D, device=q_seg.device, dtype=torch.bfloat16)
        lse = torch.empty(Bq, Hq, Tq, device=q_seg.device, dtype=torch.float32)
        base = (self.maps.data_ptr() + 63) // 64 * 64
        slot = base + (self.calls % 8) * (2 * n_chunks * 128)
        self.calls += 1
        ll = ctypes.c_longlong
        _lib.check(_lib.kernels().hmf_attention_fwd_cp(
            _lib.ptr(q_seg), arr, ctypes.c_void_p(slot), _lib.ptr(self.flags), ctypes.c_uint(self.epoch), _lib.ptr(o),
            _lib.ptr(lse), ctypes.c_int(Bq), ctypes.c_int(Tq), ctypes.c_int(Lc), ctypes.c_int(n_chunks),
            ctypes.c_int(chunk_id + 1), ctypes.c_int(Hq), ctypes.c_int(Hkv), ctypes.c_int(D), ll(q_seg.stride(0)),
            ll(q_seg.stride(1)), ll(q_seg.stride(2)), ll(T * Hkv * D), ctypes.c_int(lo), ctypes.c_int(hi),
            ctypes.c_int(chunk_id * Lc), ctypes.c_float(scale), _lib.stream_ptr(q_seg.device)), "attention_fwd_cp")
        return o, lse


def enable_peer_kv(sp, max_kv_bytes: int) -> bool:
    """Attaches a ``PeerKVExchange`` to the SP context (``sp.peer_kv``); collective call."""
    if sp is None or sp.size <= 1 or not torch.cuda.is_available():
        return False
    sp.peer_kv = PeerKVExchange(sp.group, sp.rank, sp.size, max_kv_bytes)
    return True
