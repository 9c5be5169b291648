"""ctypes binding of the native scheduler / block manager (``csrc/runtime/scheduler.cpp``)."""
from __future__ import annotations

import ctypes
from dataclasses import dataclass
from typing import List, Sequence

from ..ops import _lib

i64, i32 = ctypes.c_int64, ctypes.c_int32


@dataclass
class ScheduledSeq:
    req_id: int
    num_tokens: int
    start_pos: int
    slot: int
    restore_from: int  # snapshot slot to copy the recurrent state from before running (-1: none)

    @property
    def is_decode(self) -> bool:
        return self.num_tokens == 1 and self.start_pos > 0


class NativeScheduler:
    def __init__(self, num_blocks: int, block_size: int, num_slots: int, max_num_seqs: int = 64,
                 max_num_batched_tokens: int = 8192, enable_prefix_caching: bool = False,
                 num_snapshot_slots: int = 0, require_snapshot: bool = False, whole_prompts: bool = False):
        lib = _lib.runtime()
        lib.hmf_sched_create.restype = ctypes.c_void_p
        lib.hmf_sched_block_table.restype = ctypes.c_int
        self._lib = lib
        self._h = ctypes.c_void_p(lib.hmf_sched_create(num_blocks, block_size, num_slots, max_num_seqs,
                                                       max_num_batched_tokens, int(enable_prefix_caching),
                                                       num_snapshot_slots, int(require_snapshot)))
        if whole_prompts:   # do not split a prompt that fits a step of its own (see Scheduler::step)
            lib.hmf_sched_set_whole_prompts(self._h, 1)
        self.block_size, self.max_num_seqs = block_size, max_num_seqs
        n = max_num_seqs * 2 + 8
        self._ids, self._ntok = (i64 * n)(), (i32 * n)()
        self._start, self._slots, self._restore = (i32 * n)(), (i32 * n)(), (i32 * n)()
        self._n = n

    def __del__(self):
        try:
            self._lib.hmf_sched_destroy(self._h)
        except Exception:
            pass

    def add_request(self, req_id: int, prompt: Sequence[int], max_new_tokens: int) -> None:
        arr = (i32 * len(prompt))(*prompt)
        rc = self._lib.hmf_sched_add(self._h, i64(req_id), arr, len(prompt), max_new_tokens)
        if rc != 0:
            raise ValueError(f"request id {req_id} already exists")

    def step(self) -> List[ScheduledSeq]:
        n = self._lib.hmf_sched_step(self._h, self._ids, self._ntok, self._start, self._slots, self._restore, self._n)
        return [ScheduledSeq(int(self._ids[i]), int(self._ntok[i]), int(self._start[i]), int(self._slots[i]),
                             int(self._restore[i])) for i in range(n)]

    def advance(self, req_id: int, n: int) -> None:
        self._lib.hmf_sched_advance(self._h, i64(req_id), n)

    def append_token(self, req_id: int, token: int) -> None:
        self._lib.hmf_sched_append_token(self._h, i64(req_id), token)

    def finish(self, req_id: int) -> None:
        self._lib.hmf_sched_finish(self._h, i64(req_id))

    def is_finished(self, req_id: int) -> bool:
        return self._lib.hmf_sched_is_finished(self._h, i64(req_id)) == 1

    def block_table(self, req_id: int, max_blocks: int = 4096) -> List[int]:
        return self.block_table_array(req_id, max_blocks).tolist()

    def block_table_array(self, req_id: int, max_blocks: int = 4096):
        """Block ids of a request as an ``int32`` numpy array (a copy)."""
        import numpy as np
        if getattr(self, "_bt_buf", None) is None or len(self._bt_buf) < max_blocks:
            self._bt_buf = (i32 * max_blocks)()
        n = self._lib.hmf_sched_block_table(self._h, i64(req_id), self._bt_buf, len(self._bt_buf))
        if n < 0:
            raise KeyError(req_id)
        if n > len(self._bt_buf):
            return self.block_table_array(req_id, n)
        return np.ctypeslib.as_array(self._bt_buf)[:n].copy()

    def register_snapshot(self, req_id: int, pos: int) -> int:
        return int(self._lib.hmf_sched_register_snapshot(self._h, i64(req_id), pos))

    def stats(self) -> dict:
        out = (i64 * 8)()
        self._lib.hmf_sched_stats(self._h, out)
        keys = ["free_blocks", "free_slots", "running", "waiting", "prefix_hits", "prefix_queries", "snapshots", "evictions"]
        return {k: int(out[i]) for i, k in enumerate(keys)}
