"""Host-side replay model of the peer-memory signalling protocols (no GPU involved).

The kernels signal with monotonically increasing epochs: a writer stores its payload, then ``flag = epoch``
(release); a reader waits for ``flag >= epoch`` (acquire) and then reads.  Buffers are reused every epoch (SP
state chain) or every other epoch (GEMM + all-reduce partials).  ``simulate`` runs the per-rank event programs
under every interleaving allowed by the waits (or a random sample of them) and checks that

* no reader ever observes a payload of a different epoch than the one it waited for (no premature overwrite);
* every program terminates (no deadlock), also when a chosen flag write is dropped — then the affected waits
  must end through their bounded-timeout branch, which the model reports instead of hanging.
"""
from __future__ import annotations

import random
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Tuple

# event kinds: ("write", buf, epoch) ("flag", flag, epoch) ("wait", flag, epoch) ("read", buf, epoch)
Event = Tuple[str, str, int]


@dataclass
class Result:
    ok: bool
    violations: List[str] = field(default_factory=list)
    timeouts: List[Tuple[int, Event]] = field(default_factory=list)


def sp_chain_program(rank: int, world: int, epochs: int) -> List[Event]:
    """Forward state chain of ``ops.scan`` under the in-kernel transport (two segments per epoch)."""
    prog: List[Event] = []
    for e in range(1, epochs + 1):
        if rank > 0:
            prog += [("wait", f"a{rank}", e), ("read", f"a{rank}", e)]
        if rank < world - 1:
            prog += [("write", f"a{rank + 1}", e), ("flag", f"a{rank + 1}", e)]
            prog += [("wait", f"b{rank}", e), ("read", f"b{rank}", e)]
        if rank > 0:
            prog += [("write", f"b{rank - 1}", e), ("flag", f"b{rank - 1}", e)]
    return prog


def gemm_allreduce_program(rank: int, world: int, epochs: int) -> List[Event]:
    """One tile of the fused GEMM + all-reduce: partials double-buffered by epoch parity."""
    prog: List[Event] = []
    for e in range(1, epochs + 1):
        prog.append(("write", f"p{rank}.{e & 1}", e))
        prog += [("flag", f"f{peer}.{rank}", e) for peer in range(world)]
        prog += [("wait", f"f{rank}.{src}", e) for src in range(world)]
        prog += [("read", f"p{src}.{e & 1}", e) for src in range(world)]
    return prog


def simulate(programs: List[List[Event]], seed: int = 0, trials: int = 200,
             drop: Optional[Tuple[int, int]] = None) -> Result:
    """``drop = (rank, index)`` removes that rank's ``index``-th flag write (a lost signal)."""
    rng = random.Random(seed)
    res = Result(True)
    for _ in range(trials):
        pcs = [0] * len(programs)
        bufs: Dict[str, int] = {}
        flags: Dict[str, int] = {}
        flag_count = [0] * len(programs)
        timed_out = set()
        while True:
            runnable = []
            for r, prog in enumerate(programs):
                if pcs[r] >= len(prog):
                    continue
                kind, name, e = prog[pcs[r]]
                if kind == "wait" and flags.get(name, 0) < e and (r, pcs[r]) not in timed_out:
                    continue
                runnable.append(r)
            if not runnable:
                blocked = [(r, programs[r][pcs[r]]) for r in range(len(programs)) if pcs[r] < len(programs[r])]
                if not blocked:
                    break
                # bounded waits: the blocked ranks give up, report, and continue
                for r, ev in blocked:
                    timed_out.add((r, pcs[r]))
                    res.timeouts.append((r, ev))
                continue
            r = rng.choice(runnable)
            kind, name, e = programs[r][pcs[r]]
            if kind == "write":
                bufs[name] = e
            elif kind == "flag":
                idx = flag_count[r]
                flag_count[r] += 1
                if drop != (r, idx):
                    flags[name] = max(flags.get(name, 0), e)
            elif kind == "read":
                if (r, pcs[r] - 1) not in timed_out and bufs.get(name) != e:
                    res.ok = False
                    res.violations.append(f"rank {r} read {name} expecting epoch {e}, found {bufs.get(name)}")
            pcs[r] += 1
        if drop is None and res.timeouts:
            res.ok = False
            res.violations.append("deadlock without an injected fault")
            break
    return res
