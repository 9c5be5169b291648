"""Per-layer activation checkpointing with an attention stash.

``layer_checkpoint(fn, *tensors)`` runs ``fn`` without building a graph, keeps only its tensor
inputs, and re-runs it with autograd enabled when the backward pass reaches it (like
``torch.utils.checkpoint``).  In addition, ops may *stash* small results of the first run that are
expensive to recompute: the flash-attention binding stores ``(o, lse)`` per call, and during the
re-run returns the stored output instead of launching the forward kernel again while still
registering its backward.  At 128K context this removes one full attention forward per attention
layer per step for 1 GB of extra activation memory per layer.
"""
from __future__ import annotations

import threading
from typing import Callable, List, Optional

import torch

_state = threading.local()
# Offloaded checkpoints: the saved layer inputs wait in pinned host memory between the forward and the backward pass
# (at 128K tokens one hidden state is 1 GB per layer).  Off by default; `set_offload(True)` or the trainer argument
# `offload_checkpoints`.  The copies are ordinary stream-ordered `copy_` calls, so they overlap with nothing by
# themselves; they trade PCIe time for memory.
_offload = {"enabled": False, "min_bytes": 1 << 20, "force_cpu_copy": False}


def set_offload(enabled: bool, min_bytes: int = 1 << 20, force_cpu_copy: bool = False) -> None:
    """``force_cpu_copy`` also moves CPU tensors through a copy (lets CPU tests exercise the path)."""
    _offload.update(enabled=bool(enabled), min_bytes=int(min_bytes), force_cpu_copy=bool(force_cpu_copy))


def _to_host(t: torch.Tensor):
    if not _offload["enabled"] or t.numel() * t.element_size() < _offload["min_bytes"]:
        return None
    if t.is_cuda:
        host = torch.empty(t.shape, dtype=t.dtype, device="cpu", pin_memory=True)
        host.copy_(t, non_blocking=True)
        return host
    return t.detach().clone() if _offload["force_cpu_copy"] else None


# Probe of what a layer's autograd graph holds: while on, the re-run of a checkpointed layer (the only time its graph
# exists) records the growth of the allocator's live bytes under the layer's key.  The trainer uses the figures to
# decide which layers fit in memory WITHOUT checkpointing (`train/trainer.py::Trainer.plan_recompute`).
_probe = {"on": False, "sizes": {}, "mem_fn": None}


def start_probe(mem_fn: Optional[Callable[[], int]] = None) -> None:
    """``mem_fn`` returns the live bytes (default: ``torch.cuda.memory_allocated`` of the current device)."""
    _probe.update(on=True, sizes={}, mem_fn=mem_fn)


def stop_probe() -> dict:
    _probe["on"] = False
    return dict(_probe["sizes"])


def _live_bytes() -> int:
    if _probe["mem_fn"] is not None:
        return int(_probe["mem_fn"]())
    return int(torch.cuda.memory_allocated()) if torch.cuda.is_available() else 0


def stash_for_write() -> Optional[List]:
    """List to append to while inside the first (graph-free) run of a checkpointed layer."""
    return getattr(_state, "write", None)


def stash_for_read() -> Optional[List]:
    """List to pop from (front) while inside the re-run of a checkpointed layer."""
    return getattr(_state, "read", None)


class _LayerCheckpoint(torch.autograd.Function):
    @staticmethod
    def forward(ctx, fn: Callable, use_stash: bool, key, *args):
        ctx.fn = fn
        ctx.key = key
        tensors = [a for a in args if isinstance(a, torch.Tensor)]
        ctx.hosted = [(i, _to_host(t), t.device, t.requires_grad) for i, t in enumerate(tensors)]
        ctx.hosted = [h for h in ctx.hosted if h[1] is not None]
        moved = {i for i, _, _, _ in ctx.hosted}
        # offloaded inputs are replaced by empty placeholders in the autograd-saved list
        ctx.save_for_backward(*[t.new_empty(0) if i in moved else t for i, t in enumerate(tensors)])
        ctx.arg_is_tensor = [isinstance(a, torch.Tensor) for a in args]
        ctx.non_tensor = [a for a in args if not isinstance(a, torch.Tensor)]
        ctx.stash = [] if use_stash else None
        prev = getattr(_state, "write", None)
        _state.write = ctx.stash
        try:
            with torch.no_grad():
                out = fn(*args)
        finally:
            _state.write = prev
        ctx.single = isinstance(out, torch.Tensor)
        outs = (out,) if ctx.single else tuple(out)
        ctx.out_is_tensor = [isinstance(o, torch.Tensor) for o in outs]
        return tuple(o if isinstance(o, torch.Tensor) else torch.zeros((), device=args[0].device) for o in outs)

    @staticmethod
    def backward(ctx, *grads):
        tensors = list(ctx.saved_tensors)
        for i, host, device, _ in ctx.hosted:          # bring the offloaded inputs back
            tensors[i] = host.to(device, non_blocking=True)
        ctx.hosted = []
        non_tensor = list(ctx.non_tensor)
        args, leaves = [], []
        for is_t in ctx.arg_is_tensor:
            if is_t:
                t = tensors.pop(0)
                d = t.detach()
                if t.is_floating_point():
                    d.requires_grad_(True)
                leaves.append(d)
                args.append(d)
            else:
                args.append(non_tensor.pop(0))
        prev = getattr(_state, "read", None)
        _state.read = ctx.stash
        probing = _probe["on"] and ctx.key is not None
        before = _live_bytes() if probing else 0
        try:
            with torch.enable_grad():
                out = ctx.fn(*args)
        finally:
            _state.read = prev
        if probing:
            _probe["sizes"][ctx.key] = max(_probe["sizes"].get(ctx.key, 0), _live_bytes() - before)
        outs = (out,) if isinstance(out, torch.Tensor) else tuple(out)
        pairs = [(o, g) for o, g, is_t in zip(outs, grads, ctx.out_is_tensor)
                 if is_t and o.requires_grad and g is not None]
        if pairs:
            torch.autograd.backward([o for o, _ in pairs], [g for _, g in pairs])
        ctx.stash = None
        res, li = [], 0
        for is_t in ctx.arg_is_tensor:
            if is_t:
                leaf = leaves[li]
                li += 1
                res.append(leaf.grad if leaf.requires_grad else None)
            else:
                res.append(None)
        return (None, None, None, *res)


def layer_checkpoint(fn: Callable, *args, use_stash: bool = True, key=None):
    """Checkpointed call of ``fn(*args)`` (tensor and non-tensor positional arguments).  ``key`` names the layer for the
    activation-size probe."""
    out = _LayerCheckpoint.apply(fn, use_stash, key, *args)
    return out


def choose_unchecked_layers(sizes: dict, budget: float) -> List:
    """Layers (keys of ``sizes``: bytes their graphs hold) to run without checkpointing so that the sum stays within
    ``budget`` bytes: taken from the last layer backwards (their activations are the first to be freed again), skipping
    what does not fit."""
    chosen = []
    for k in sorted(sizes, reverse=True):
        if 0 < sizes[k] <= budget:
            chosen.append(k)
            budget -= sizes[k]
    return sorted(chosen)
