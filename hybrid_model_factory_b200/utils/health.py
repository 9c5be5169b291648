"""Host-side failure detection for multi-process jobs.

Ranks publish a heartbeat (step number + wall time) in the job's key-value store between steps; before a rank
enters its next collective it checks that every peer is alive and has not fallen behind for longer than
``timeout_s``.  A peer that exited, raised or hangs on the host is therefore noticed *before* the next launch,
and the job stops with ``PeerFailure`` instead of waiting inside a collective (a short process-group timeout is
the second line of defence).  No device-side fault is involved: failures are host events.
The reference has no health checks; restart = resume from the last checkpoint (``launcher.py:74-113``).
"""
from __future__ import annotations

import time
from typing import Dict, List, Optional

import torch.distributed as dist


class PeerFailure(RuntimeError):
    def __init__(self, ranks: List[int], reason: str):
        super().__init__(f"rank(s) {ranks} {reason}")
        self.ranks, self.reason = ranks, reason


class Heartbeat:
    def __init__(self, store, rank: int, world: int, timeout_s: float = 60.0, prefix: str = "hb"):
        self.store, self.rank, self.world, self.timeout_s, self.prefix = store, rank, world, timeout_s, prefix
        self.step = 0

    @classmethod
    def from_default_group(cls, timeout_s: float = 60.0) -> "Heartbeat":
        from torch.distributed.distributed_c10d import _get_default_store
        return cls(_get_default_store(), dist.get_rank(), dist.get_world_size(), timeout_s)

    def _key(self, rank: int) -> str:
        return f"{self.prefix}/{rank}"

    def beat(self, step: Optional[int] = None, status: str = "ok") -> None:
        self.step = self.step + 1 if step is None else step
        self.store.set(self._key(self.rank), f"{self.step}:{time.time():.3f}:{status}")

    def fail(self, reason: str = "failed") -> None:
        """Called from an exception handler so that peers stop promptly."""
        self.store.set(self._key(self.rank), f"{self.step}:{time.time():.3f}:{reason}")

    def read(self, rank: int):
        try:
            if hasattr(self.store, "check") and not self.store.check([self._key(rank)]):
                return None
            step, t, status = self.store.get(self._key(rank)).decode().split(":", 2)
            return int(step), float(t), status
        except Exception:
            return None

    def check(self, min_step: Optional[int] = None) -> Dict[int, tuple]:
        """Raises ``PeerFailure`` when a peer reported a failure, or has no fresh heartbeat within the timeout."""
        now = time.time()
        seen, failed, stale = {}, [], []
        for r in range(self.world):
            if r == self.rank:
                continue
            rec = self.read(r)
            if rec is None:
                stale.append(r)
                continue
            seen[r] = rec
            if rec[2] != "ok":
                failed.append(r)
            elif now - rec[1] > self.timeout_s and (min_step is None or rec[0] < min_step):
                stale.append(r)
        if failed:
            raise PeerFailure(failed, "reported a failure: " + ", ".join(seen[r][2] for r in failed))
        if stale:
            raise PeerFailure(stale, f"sent no heartbeat for more than {self.timeout_s:.0f} s")
        return seen

    def wait_for_peers(self, step: int, poll_s: float = 0.05) -> None:
        """Blocks (bounded by ``timeout_s``) until every peer has reached ``step``; raises on failure."""
        deadline = time.time() + self.timeout_s
        while True:
            behind = []
            for r in range(self.world):
                if r == self.rank:
                    continue
                rec = self.read(r)
                if rec is not None and rec[2] != "ok":
                    raise PeerFailure([r], f"reported a failure: {rec[2]}")
                if rec is None or rec[0] < step:
                    behind.append(r)
            if not behind:
                return
            if time.time() > deadline:
                raise PeerFailure(behind, f"did not reach step {step} within {self.timeout_s:.0f} s")
            time.sleep(poll_s)
