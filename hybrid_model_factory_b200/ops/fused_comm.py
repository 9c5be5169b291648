"""Compute + collective kernels over peer memory (tensor parallelism).

Three forms of one kernel (``csrc/kernels/gemm_allreduce.cu``), each ONE launch per rank with the transfer riding on
the tiles (no separate collective):

* ``PeerGemmAllReduce(x, W)``: ``y = all_reduce(x @ W_shard^T)`` (row-parallel projection);
* ``PeerGemmAllReduce.reduce_scatter(x, W)``: the same sum, each rank keeping its ``N / world`` output columns
  (GEMM -> reduce-scatter);
* ``PeerAllGatherGemm(x_shard, W)``: ``y = concat_r(x_r) @ W^T`` with the activations sharded over the ranks along the
  hidden dimension, fetched shard by shard from the owners' symmetric buffers inside the GEMM (all-gather -> GEMM).

``PeerGemmAllReduce``: ``y = all_reduce(x @ W_shard^T)`` for decode-sized ``x`` in ONE kernel per rank
(``csrc/kernels/gemm_allreduce.cu``): tcgen05 GEMM tile -> partial tile into a symmetric buffer -> per-tile flags
-> peer loads + ordered sum.  Replaces the row-parallel linear + NCCL all-reduce pair of the attention / mixer
output projection and of the MLP down projection (the reference relies on vLLM's ``RowParallelLinear`` with
its custom all-reduce, ``vllm-inference/src/primed_vllm/layers/primed_gdn_layer.py``).
"""
from __future__ import annotations

import ctypes

import torch

from . import _lib

c_int, c_ll = ctypes.c_int, ctypes.c_longlong


class PeerGemmAllReduce:
    MAX_WORLD = 8

    def __init__(self, group, max_m: int = 256, max_n: int = 8192, device=None):
        from ..parallel.peer import SymmetricWorkspace
        self.max_m, self.max_n = max_m, max_n
        self.MAX_SPLIT = 4
        self.part_stride = max_m * max_n * self.MAX_SPLIT      # elements per parity buffer (all K splits)
        part_bytes = 2 * self.part_stride * 2
        self.max_tiles = max_n // 128
        flag_bytes = self.max_tiles * self.MAX_WORLD * self.MAX_SPLIT * 4
        arr = ctypes.c_ulonglong * self.MAX_WORLD
        if group is None:       # single rank: ordinary device memory (the kernel then reduces over one partial)
            dev = device or torch.device("cuda", torch.cuda.current_device())
            self.local = torch.zeros(part_bytes + flag_bytes, dtype=torch.uint8, device=dev)
            self.rank, self.world = 0, 1
            bases = [self.local.data_ptr()]
            self.mc_part = 0
        else:
            self.ws = SymmetricWorkspace(part_bytes + flag_bytes, group, device)
            self.rank, self.world = self.ws.rank, self.ws.world
            dev = self.ws.device
            bases = [self.ws.peer_ptr(r, 0) for r in range(self.world)]
            self.mc_part = self.ws.multicast_ptr          # the partial buffers start at offset 0 of the workspace
        # NVLS reduction (multimem.ld_reduce inside the kernel) when the buffers have a multicast mapping and
        # HMF_TP_NVLS=1; the peer-load reduction (bit-identical on every rank) otherwise
        import os
        self.use_nvls = bool(self.mc_part) and os.environ.get("HMF_TP_NVLS", "0") == "1"
        assert self.world <= self.MAX_WORLD
        pad = [0] * (self.MAX_WORLD - self.world)
        self.part_ptrs = arr(*bases, *pad)
        self.flag_ptrs = arr(*[b + part_bytes for b in bases], *pad)
        self.sync = torch.zeros(2, dtype=torch.int32, device=dev)
        self.calls = 0

    def accepts(self, x: torch.Tensor, weight: torch.Tensor) -> bool:
        return (x.is_cuda and x.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16 and x.dim() == 2
                and 1 <= x.shape[0] <= self.max_m and weight.shape[0] % 128 == 0 and weight.shape[0] <= self.max_n
                and x.shape[1] % 64 == 0 and x.shape[1] == weight.shape[1] and x.stride(1) == 1
                and weight.stride(1) == 1 and x.stride(0) % 8 == 0 and weight.stride(0) % 8 == 0
                and x.data_ptr() % 16 == 0 and weight.data_ptr() % 16 == 0)

    def __call__(self, x: torch.Tensor, weight: torch.Tensor) -> torch.Tensor:
        M, Ks = x.shape
        N = weight.shape[0]
        y = torch.empty(M, N, device=x.device, dtype=torch.bfloat16)
        # K splits: more CTAs on the weight stream when the shard has few 128-column tiles
        tiles, splits = N // 128, 1
        # ... but every (rank, split) partial is read by every rank, so world * splits is kept at 8 or below
        while (splits < self.MAX_SPLIT and tiles * splits * 2 <= 148 and Ks % (splits * 2 * 64) == 0
               and Ks // (splits * 2) >= 256 and self.world * splits * 2 <= 8):
            splits *= 2
        if self.use_nvls:
            return self._nvls(x, weight, y, splits, 0)
        _lib.check(_lib.kernels().hmf_gemm_allreduce(
            _lib.ptr(x), _lib.ptr(weight), _lib.ptr(y), c_int(M), c_int(N), c_int(Ks), c_ll(x.stride(0)),
            c_ll(weight.stride(0)), self.part_ptrs, self.flag_ptrs, _lib.ptr(self.sync), c_ll(self.part_stride),
            c_int(self.max_tiles), c_int(self.rank), c_int(self.world), c_int(splits), _lib.stream_ptr(x.device)),
            "gemm_allreduce")
        self.calls += 1
        return y

    def _nvls(self, x, weight, y, splits: int, mode: int) -> torch.Tensor:
        M, Ks = x.shape
        N = weight.shape[0]
        _lib.check(_lib.kernels().hmf_gemm_reduce_nvls(
            _lib.ptr(x), _lib.ptr(weight), _lib.ptr(y), c_int(M), c_int(N), c_int(Ks), c_ll(x.stride(0)),
            c_ll(weight.stride(0)), self.part_ptrs, self.flag_ptrs, _lib.ptr(self.sync), c_ll(self.part_stride),
            c_int(self.max_tiles), c_int(self.rank), c_int(self.world), c_int(splits), c_int(mode),
            ctypes.c_void_p(self.mc_part), _lib.stream_ptr(x.device)), "gemm_reduce_nvls")
        self.calls += 1
        return y

    def _splits(self, N: int, Ks: int) -> int:
        tiles, splits = N // 128, 1
        while (splits < self.MAX_SPLIT and tiles * splits * 2 <= 148 and Ks % (splits * 2 * 64) == 0
               and Ks // (splits * 2) >= 256 and self.world * splits * 2 <= 8):
            splits *= 2
        return splits

    def reduce_scatter(self, x: torch.Tensor, weight: torch.Tensor) -> torch.Tensor:
        """``sum_r x_r W_r^T`` with this rank keeping output columns ``[rank N / world, (rank + 1) N / world)``."""
        M, Ks = x.shape
        N = weight.shape[0]
        assert (N // 128) % self.world == 0, "reduce-scatter needs N / 128 tiles divisible by the number of ranks"
        y = torch.empty(M, N // self.world, device=x.device, dtype=torch.bfloat16)
        if self.use_nvls:
            return self._nvls(x, weight, y, self._splits(N, Ks), 1)
        _lib.check(_lib.kernels().hmf_gemm_reduce_scatter(
            _lib.ptr(x), _lib.ptr(weight), _lib.ptr(y), c_int(M), c_int(N), c_int(Ks), c_ll(x.stride(0)),
            c_ll(weight.stride(0)), self.part_ptrs, self.flag_ptrs, _lib.ptr(self.sync), c_ll(self.part_stride),
            c_int(self.max_tiles), c_int(self.rank), c_int(self.world), c_int(self._splits(N, Ks)),
            _lib.stream_ptr(x.device)), "gemm_reduce_scatter")
        self.calls += 1
        return y


class PeerAllGatherGemm:
    """``y [M, N] = concat_r(x_r) [M, world * Ks] @ W [N, world * Ks]^T``: the all-gather of the hidden-sharded
    activations happens inside the GEMM.  Each call copies this rank's shard into its symmetric buffer and raises its
    flag on every peer; the kernel's producer waits (bounded) for a shard's flag before the first tile it loads from
    that rank.  Two parity buffers: a rank publishes epoch ``e + 2`` only after every peer has published ``e + 1``,
    which on the peer's stream follows its epoch-``e`` GEMM, so no shard is overwritten while it can still be read."""

    MAX_WORLD = 8

    def __init__(self, group, max_m: int = 256, max_ks: int = 8192, max_n: int = 8192, device=None):
        from ..parallel.peer import SymmetricWorkspace
        self.max_m, self.max_ks = max_m, max_ks
        shard_bytes = max_m * max_ks * 2
        self.off_flags = 2 * shard_bytes
        self.ws = SymmetricWorkspace(self.off_flags + 1024, group, device)
        self.rank, self.world = self.ws.rank, self.ws.world
        dev = self.ws.device
        self.shard_bytes = shard_bytes
        self.flags = self.ws.view(self.off_flags, (self.world,), torch.int32)
        self.flag_ptrs_dev = torch.tensor([self.ws.peer_ptr(r, self.off_flags) for r in range(self.world)],
                                          dtype=torch.int64, device=dev)
        self.local = PeerGemmAllReduce(None, max_m, max_n, dev)       # partial / flag scratch of the 1-rank reduction
        self.max_slots = 16
        self.maps = torch.empty(self.max_slots * self.MAX_WORLD * 128 + 64, dtype=torch.uint8, device=dev)
        self._slots = {}            # (M, Ks, parity) -> descriptor slot that already holds the maps of that shape
        self.epoch = 0
        self.calls = 0

    def __call__(self, x_shard: torch.Tensor, weight: torch.Tensor) -> torch.Tensor:
        K = _lib.kernels()
        M, Ks = x_shard.shape
        N = weight.shape[0]
        assert M <= self.max_m and Ks <= self.max_ks and weight.shape[1] == Ks * self.world
        st = _lib.stream_ptr(x_shard.device)
        self.epoch += 1
        par = self.epoch & 1
        if self.epoch > 2:          # every peer is past the GEMM that read this parity buffer last
            _lib.check(K.hmf_peer_wait(_lib.ptr(self.flags), c_int(self.world), ctypes.c_uint(self.epoch - 1), st), "peer_wait")
        self.ws.view(par * self.shard_bytes, (M, Ks), torch.bfloat16).copy_(x_shard)
        _lib.check(K.hmf_peer_signal(_lib.ptr(self.flag_ptrs_dev), c_int(self.world), c_int(self.rank),
                                     ctypes.c_uint(self.epoch), st), "peer_signal")
        arr = ctypes.c_ulonglong * self.MAX_WORLD
        x_ptrs = arr(*[self.ws.peer_ptr(r, par * self.shard_bytes) for r in range(self.world)],
                     *([0] * (self.MAX_WORLD - self.world)))
        key = (M, Ks, par)
        ready = key in self._slots
        if not ready:
            if len(self._slots) >= self.max_slots:
                torch.cuda.current_stream(x_shard.device).synchronize()     # no kernel still reads the old descriptors
                self._slots.clear()
            self._slots[key] = len(self._slots)
        slot = (self.maps.data_ptr() + 63) // 64 * 64 + self._slots[key] * self.MAX_WORLD * 128
        y = torch.empty(M, N, device=x_shard.device, dtype=torch.bfloat16)
        lo = self.local
        _lib.check(K.hmf_allgather_gemm(x_ptrs, ctypes.c_void_p(slot), _lib.ptr(self.flags), ctypes.c_uint(self.epoch),
                                        c_int(self.world), _lib.ptr(weight), _lib.ptr(y), c_int(M), c_int(N), c_int(Ks),
                                        c_ll(Ks), c_ll(weight.stride(0)), lo.part_ptrs, lo.flag_ptrs, _lib.ptr(lo.sync),
                                        c_ll(lo.part_stride), c_int(lo.max_tiles), c_int(1), c_int(int(ready)), st),
                   "allgather_gemm")
        self.calls += 1
        return y
