"""Compute + collective kernels over peer memory (tensor parallelism).

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
        else:
            self.ws = SymmetricWorkspace(part_bytes + flag_bytes, group, device)
            self.rank, self.world = self.ws.rank, self.ws.world
            dev = self.ws.device
            bases = [self.ws.peer_ptr(r, 0) for r in range(self.world)]
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
        _lib.check(_lib.kernels().hmf_gemm_allreduce(
            _lib.ptr(x), _lib.ptr(weight), _lib.ptr(y), c_int(M), c_int(N), c_int(Ks), c_ll(x.stride(0)),
            c_ll(weight.stride(0)), self.part_ptrs, self.flag_ptrs, _lib.ptr(self.sync), c_ll(self.part_stride),
            c_int(self.max_tiles), c_int(self.rank), c_int(self.world), c_int(splits), _lib.stream_ptr(x.device)),
            "gemm_allreduce")
        self.calls += 1
        return y
