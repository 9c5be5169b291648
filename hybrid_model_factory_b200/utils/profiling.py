"""Device-side timing and trace annotations.

* ``DeviceTimer``: named CUDA-event intervals on the current stream, read after one synchronise; ``summary()``
  gives per-name mean / total in ms and, under ``torch.distributed``, the maximum over ranks (the number that
  bounds a step).
* ``nvtx_range``: context manager / decorator emitting an NVTX range (no-op on CPU) so kernels group by phase
  in a timeline tool.
* ``PHASES`` / ``phase(name)``: one process-wide timer that the communication sites of the training step
  (K/V gather, dK/dV reduce-scatter, gradient reduce-scatter, parameter all-gather, state-chain scans) record
  into when a benchmark switches it on; disabled it costs one attribute test per site.
* ``StepBreakdown``: wraps the modules of a model with forward timers to attribute step time to layer types.
"""
from __future__ import annotations

import contextlib
import functools
from collections import defaultdict
from typing import Dict, List

import torch
import torch.distributed as dist


class DeviceTimer:
    def __init__(self, enabled: bool = True):
        self.enabled = enabled and torch.cuda.is_available()
        self._open: Dict[str, torch.cuda.Event] = {}
        self._pairs: Dict[str, List[tuple]] = defaultdict(list)

    def start(self, name: str) -> None:
        if self.enabled:
            ev = torch.cuda.Event(enable_timing=True)
            ev.record()
            self._open[name] = ev

    def stop(self, name: str) -> None:
        if self.enabled:
            ev = torch.cuda.Event(enable_timing=True)
            ev.record()
            self._pairs[name].append((self._open.pop(name), ev))

    @contextlib.contextmanager
    def time(self, name: str):
        self.start(name)
        try:
            yield
        finally:
            self.stop(name)

    def summary(self, reduce_max: bool = True) -> Dict[str, dict]:
        if not self.enabled:
            return {}
        torch.cuda.synchronize()
        out = {}
        for name, pairs in sorted(self._pairs.items()):
            ms = [a.elapsed_time(b) for a, b in pairs]
            total = sum(ms)
            if reduce_max and dist.is_initialized() and dist.get_world_size() > 1:
                t = torch.tensor([total], device="cuda")
                dist.all_reduce(t, op=dist.ReduceOp.MAX)
                total = float(t)
            out[name] = {"calls": len(ms), "total_ms": total, "mean_ms": total / max(len(ms), 1)}
        return out

    def reset(self) -> None:
        self._open.clear()
        self._pairs.clear()


PHASES = DeviceTimer(enabled=False)


def enable_phases(on: bool = True) -> None:
    PHASES.enabled = bool(on) and torch.cuda.is_available()
    PHASES.reset()


@contextlib.contextmanager
def phase(name: str):
    """Times the enclosed stream work under ``name`` in ``PHASES`` (no-op unless ``enable_phases()`` ran)."""
    if not PHASES.enabled:
        yield
        return
    key = f"{name}#{len(PHASES._pairs[name])}"
    if key in PHASES._open:         # the same phase entered again inside itself (a scan whose backward runs another
        yield                       # scan): the outer interval already covers it
        return
    PHASES.start(key)
    try:
        yield
    finally:
        ev = torch.cuda.Event(enable_timing=True)
        ev.record()
        PHASES._pairs[name].append((PHASES._open.pop(key), ev))


@contextlib.contextmanager
def nvtx_range(name: str):
    on = torch.cuda.is_available()
    if on:
        torch.cuda.nvtx.range_push(name)
    try:
        yield
    finally:
        if on:
            torch.cuda.nvtx.range_pop()


def nvtx(name: str):
    def deco(fn):
        @functools.wraps(fn)
        def wrapped(*a, **k):
            with nvtx_range(name):
                return fn(*a, **k)
        return wrapped
    return deco


class StepBreakdown:
    """Forward-time attribution per module class (sequence mixers, MLPs, norms) with CUDA events."""

    def __init__(self, model: torch.nn.Module, classes=None):
        self.timer = DeviceTimer()
        self.handles = []
        from ..models.patterns import MIXER_ATTR
        leaves = tuple("." + a for a in set(MIXER_ATTR.values())) + (".mlp",)      # model.layers.N.{self_attn,gdn,...}
        for name, mod in model.named_modules():
            if classes is not None and not isinstance(mod, tuple(classes)):
                continue
            if classes is None and not name.endswith(leaves):
                continue
            key = type(mod).__name__
            self.handles.append(mod.register_forward_pre_hook(lambda m, a, k=key: self.timer.start(k)))
            self.handles.append(mod.register_forward_hook(lambda m, a, o, k=key: self.timer.stop(k)))

    def summary(self):
        return self.timer.summary()

    def remove(self) -> None:
        for h in self.handles:
            h.remove()
