"""Universal linear-recurrence scan with sequence-parallel state passing.

Every SSM-style mixer of the framework (Gated DeltaNet, Gated KalmaNet's two states, Mamba2
SSD) is expressed as a *scan core*: a function of per-token inputs and an incoming recurrent
state that returns per-token outputs and the outgoing state,

    ``core.forward(inputs, state0) -> (out, stateT, tensors_to_save, meta)``
    ``core.backward(saved_tensors, meta, d_out, d_stateT) -> (d_inputs, d_state0)``

:func:`ssm_scan` turns a core into one autograd node.  Without sequence parallelism it is a
plain call.  With a sequence-parallel context the local tokens are the two zig-zag segments
of this rank (chunk ``r`` and chunk ``2*SP-1-r`` of the global sequence); the node then runs
the state chain ``0 -> 1 -> ... -> SP-1`` over the first segments and ``SP-1 -> ... -> 0`` over
the second ones, handing each segment's final state to the owner of the next chunk, and the
mirrored chain for the state gradients in backward.  Each segment is scanned exactly once
with its true incoming state: no all-gather of activations, no redundant full-sequence
recomputation, no second correction pass.  (The reference project gathers the whole sequence
on every rank for Gated DeltaNet, ``model_utils/allgather_sp_helper.py:73-174``, and runs the
scan twice for GKA/Mamba2, ``gated_kalmanet/sequence_parallel/gka_sp_utils.py:113-226``.)

All communication happens inside the node in a fixed order, so blocking transports (gloo on
CPU) cannot deadlock on autograd's scheduling.
"""
from __future__ import annotations

from typing import Callable, List, Optional, Sequence, Tuple

import torch
import torch.distributed as dist

from ..utils.profiling import phase

Tensor = torch.Tensor
State = Optional[Tuple[Tensor, ...]]


class ScanCore:
    """Interface of a scan core (see module docstring)."""

    n_state: int = 1

    def forward(self, inputs: Sequence[Tensor], state0: State):
        """-> ``(out, stateT, tensors_to_save, meta)``"""
        raise NotImplementedError

    def backward(self, saved, meta, d_out: Tensor, d_stateT: State):
        """-> ``(d_inputs, d_state0)``"""
        raise NotImplementedError

    def state_shapes(self, inputs: Sequence[Tensor]):
        raise NotImplementedError


class TorchScanCore(ScanCore):
    """Wraps a differentiable PyTorch function ``fn(*inputs, initial_state=...) -> (out, state)``.
    Forward runs without building a graph and saves only the segment inputs (through
    ``save_for_backward``, so activation checkpointing can drop them); backward re-evaluates the
    function with autograd enabled and differentiates it."""

    def __init__(self, fn: Callable, n_state: int = 1, state_shape_fn: Optional[Callable] = None, **kwargs):
        self.fn = fn
        self.kwargs = kwargs
        self.n_state = n_state
        self.state_shape_fn = state_shape_fn

    def state_shapes(self, inputs):
        """``[(shape, dtype), ...]`` of the recurrent state for segment inputs ``inputs``."""
        return self.state_shape_fn(inputs)

    def _run(self, inputs, s0):
        init = None if s0 is None else (s0[0] if self.n_state == 1 else s0)
        out, sT = self.fn(*inputs, initial_state=init, **self.kwargs)
        sT = (sT,) if self.n_state == 1 else tuple(sT)
        return out, sT

    def forward(self, inputs, state0):
        with torch.no_grad():
            out, sT = self._run(list(inputs), state0)
        saved = list(inputs) + (list(state0) if state0 is not None else [])
        meta = (len(inputs), 0 if state0 is None else len(state0))
        return out, tuple(sT), saved, meta

    def backward(self, saved, meta, d_out, d_stateT):
        n_in, n_st = meta
        leaves = [t.detach().requires_grad_(t.is_floating_point()) if t is not None else None for t in saved[:n_in]]
        s0 = tuple(s.detach().requires_grad_(True) for s in saved[n_in:n_in + n_st]) if n_st else None
        with torch.enable_grad():
            out, sT = self._run(leaves, s0)
        outs, grads = [out], [d_out.to(out.dtype)]
        if d_stateT is not None:
            for s, ds in zip(sT, d_stateT):
                if s is not None and ds is not None and s.requires_grad:
                    outs.append(s)
                    grads.append(ds.to(s.dtype))
        wrt = [t for t in leaves if t is not None and t.requires_grad] + list(s0 or [])
        g = list(torch.autograd.grad(outs, wrt, grads, allow_unused=True))
        d_inputs = []
        for t in leaves:
            if t is not None and t.requires_grad:
                gi = g.pop(0)
                d_inputs.append(torch.zeros_like(t) if gi is None else gi)
            else:
                d_inputs.append(None)
        d_s0 = None
        if s0 is not None:
            d_s0 = tuple(torch.zeros_like(s) if gi is None else gi for s, gi in zip(s0, g))
        return d_inputs, d_s0


def _split_time(t: Optional[Tensor]):
    if t is None:
        return None, None
    half = t.shape[1] // 2
    return t[:, :half], t[:, half:]


def _peer_plan(core, transport, seg_inputs):
    """``(state shape, batch*heads)`` when both the core and the transport can run the state chain inside the
    scan kernels (peer-memory push / flag wait), else ``None``."""
    if not hasattr(transport, "peer_io") or not getattr(core, "peer_capable", None):
        return None
    if not core.peer_capable(seg_inputs):
        return None
    shape, dtype = core.state_shapes(seg_inputs)[0]
    bh = int(shape[0]) * int(shape[1])
    return (tuple(shape), bh) if transport.fits(shape, dtype, bh) else None


# -- chain-free sequence parallelism for cores with a scalar state transition ---------------------------------------
# Gated linear attention, Mamba2's SSD and the key covariance of Gated KalmaNet all update their state as
# ``h_out = e^{L} h_in + h_local`` with ``L`` the summed log-decay of the segment (one scalar per batch and head).  The
# states entering the 2n zig-zag chunks then follow from every chunk's ``(h_local, L)`` by a prefix over chunks, so the
# ranks need not wait for one another: each scans its two segments from a zero state, one all-gather exchanges
# ``(h_local, L)``, and each scans again from its true incoming states.  Two passes of local work replace a serial chain
# of 2n links.  The backward pass mirrors it with the state gradients (``d_h_in = e^{L} d_h_out + d_h_local``).
# A core opts in with ``scalar_transition = True`` and ``decay_input`` (index of the log-decay tensor ``[B, T, H]`` among
# its inputs, or ``None``); the SP context switches the mode on with ``parallel_scan``.
# The delta rule has a matrix transition ``h_out = A h_in + h_local``; a core that sets ``matrix_transition = True`` and
# ``value_input`` gets the same treatment with ``A`` probed by one more scan (zero values, identity start state), i.e.
# three passes of local work; worth it only for long chains (``parallel_scan_matrix`` on the SP context).
def _segment_log_decay(core, seg_inputs, like: Tensor) -> Tensor:
    idx = getattr(core, "decay_input", None)
    g = None if idx is None else seg_inputs[idx]
    if g is None:
        return like.new_zeros(like.shape[0], like.shape[1])
    return g.float().sum(dim=1)


def _segment_transition(core, seg_inputs, like: Tensor) -> Tensor:
    """Matrix transition ``A`` of a segment (``h_out = A h_in + h_local``, ``A [B, H, Dk, Dk]``) for cores that declare
    ``matrix_transition``: the state reached from the identity when the values are zero (needs ``Dv == Dk``)."""
    vi = core.value_input
    zeroed = list(seg_inputs)
    zeroed[vi] = torch.zeros_like(seg_inputs[vi])
    B, H, Dk, Dv = like.shape
    assert Dk == Dv, "the identity-state probe of the transition needs square states"
    eye = torch.eye(Dk, device=like.device, dtype=like.dtype).expand(B, H, Dk, Dk).contiguous()
    _, (A,), _, _ = core.forward(zeroed, (eye,))
    return A.float()


def _apply(T: Tensor, S: Tensor, transpose: bool = False) -> Tensor:
    """Applies a segment transition (scalar log-decay ``[B, H]`` or matrix ``[B, H, Dk, Dk]``) to a state."""
    if T.dim() == 2:
        return torch.exp(T)[..., None, None] * S
    return (T.transpose(-1, -2) if transpose else T) @ S


def _gather_chunks(sp, mine_a: Tensor, mine_b: Tensor) -> List[Tensor]:
    """All-gathers one tensor per local segment and returns them ordered by global chunk (rank ``r`` owns chunks ``r``
    and ``2n - 1 - r``)."""
    n = sp.size
    payload = torch.stack([mine_a, mine_b]).contiguous()
    parts = [torch.empty_like(payload) for _ in range(n)]
    dist.all_gather(parts, payload, group=sp.group)
    chunks: List[Optional[Tensor]] = [None] * (2 * n)
    for rr, p in enumerate(parts):
        chunks[rr], chunks[2 * n - 1 - rr] = p[0], p[1]
    return chunks


def _bcast_from_first(sp, t: Optional[Tensor], like: Tensor) -> Tensor:
    """The tensor held by SP rank 0 (zeros when it has none) on every rank."""
    buf = like.new_zeros(like.shape) if (t is None or sp.rank != 0) else t.to(like.dtype).contiguous().clone()
    dist.broadcast(buf, src=sp.ranks[0], group=sp.group)
    return buf


parallel_scan_calls = 0      # forward passes that took the chain-free form (diagnostics, tests)


def _parallel_forward(ctx, core, sp, seg_a, seg_b, state0):
    global parallel_scan_calls
    parallel_scan_calls += 1
    r, n = sp.rank, sp.size
    with torch.no_grad():
        _, (la,), _, _ = core.forward(seg_a, None)              # local contributions from a zero state
        _, (lb,), _, _ = core.forward(seg_b, None)
        if getattr(core, "scalar_transition", False):
            La, Lb = _segment_log_decay(core, seg_a, la), _segment_log_decay(core, seg_b, lb)
        else:
            La, Lb = _segment_transition(core, seg_a, la), _segment_transition(core, seg_b, lb)
        loc = _gather_chunks(sp, la.float(), lb.float())
        dec = _gather_chunks(sp, La, Lb)
        S = _bcast_from_first(sp, None if state0 is None else state0[0], la.float())
        incoming = []
        for c in range(2 * n):
            incoming.append(S)
            S = _apply(dec[c], S) + loc[c]
    ca, cb = r, 2 * n - 1 - r
    out_a, sT_a, saved_a, meta_a = core.forward(seg_a, (incoming[ca].to(la.dtype),))
    out_b, sT_b, saved_b, meta_b = core.forward(seg_b, (incoming[cb].to(lb.dtype),))
    ctx.save_for_backward(*saved_a, *saved_b, *[d.contiguous() for d in dec])
    ctx.counts, ctx.metas = [len(saved_a), len(saved_b)], [meta_a, meta_b]
    ctx.state_templates = ((S.shape, la.dtype),)
    ctx.peer = None
    return (torch.cat([out_a, out_b], dim=1), S.to(la.dtype))


def _parallel_backward(ctx, core, sp, saved_all, d_a, d_b, d_state):
    r, n = sp.rank, sp.size
    na, nb = ctx.counts
    saved_a, saved_b, dec = saved_all[:na], saved_all[na:na + nb], saved_all[na + nb:]
    shape, dtype = ctx.state_templates[0]
    with torch.no_grad():
        _, dla = core.backward(saved_a, ctx.metas[0], d_a, None)      # state gradients with nothing coming from later chunks
        _, dlb = core.backward(saved_b, ctx.metas[1], d_b, None)
        zero = d_a.new_zeros(shape, dtype=torch.float32)
        dla = zero if (dla is None or dla[0] is None) else dla[0].float()
        dlb = zero if (dlb is None or dlb[0] is None) else dlb[0].float()
        dloc = _gather_chunks(sp, dla, dlb)
        Dg = _bcast_from_first(sp, None if d_state is None else d_state[0], zero)   # gradient of the final state
        outgoing: List[Optional[Tensor]] = [None] * (2 * n)
        for c in reversed(range(2 * n)):
            outgoing[c] = Dg
            Dg = _apply(dec[c], Dg, transpose=True) + dloc[c]
    ca, cb = r, 2 * n - 1 - r
    d_in_a, _ = core.backward(saved_a, ctx.metas[0], d_a, (outgoing[ca].to(dtype),))
    d_in_b, _ = core.backward(saved_b, ctx.metas[1], d_b, (outgoing[cb].to(dtype),))
    d_inputs = [None if ga is None else torch.cat([ga, gb], dim=1) for ga, gb in zip(d_in_a, d_in_b)]
    d_s0 = ([Dg.to(dtype)] if r == 0 else [None]) if ctx.n_state0 else []
    return (None, None, None, None, *d_inputs, *d_s0)


class _SSMScan(torch.autograd.Function):
    @staticmethod
    def forward(ctx, core: ScanCore, sp, n_inputs: int, want_state: bool, *tensors):
        with phase("ssm_scan_fwd"):
            return _SSMScan._forward(ctx, core, sp, n_inputs, want_state, *tensors)

    @staticmethod
    def backward(ctx, d_out, *d_state):
        with phase("ssm_scan_bwd"):
            return _SSMScan._backward(ctx, d_out, *d_state)

    @staticmethod
    def _forward(ctx, core: ScanCore, sp, n_inputs: int, want_state: bool, *tensors):
        inputs = list(tensors[:n_inputs])
        state0 = tensors[n_inputs:]
        state0 = tuple(state0) if len(state0) else None
        ctx.core, ctx.sp, ctx.n_inputs, ctx.n_state0 = core, sp, n_inputs, 0 if state0 is None else len(state0)
        if sp is None or sp.size == 1:
            out, sT, saved, meta = core.forward(inputs, state0)
            ctx.save_for_backward(*saved)
            ctx.counts, ctx.metas = [len(saved)], [meta]
            ctx.state_templates = tuple((s.shape, s.dtype) if s is not None else None for s in sT)
            return (out, *[s if s is not None else out.new_zeros(()) for s in sT])
        # --- sequence-parallel zig-zag chain -------------------------------------------------
        r, n = sp.rank, sp.size
        seg_a, seg_b = zip(*[_split_time(t) for t in inputs])
        tr = sp.transport
        ctx.parallel = bool(getattr(sp, "parallel_scan", False) and (
            getattr(core, "scalar_transition", False)
            or (getattr(core, "matrix_transition", False) and getattr(sp, "parallel_scan_matrix", False))))
        if ctx.parallel:
            return _parallel_forward(ctx, core, sp, list(seg_a), list(seg_b), state0)
        ctx.peer = _peer_plan(core, tr, list(seg_a))
        if ctx.peer is not None:
            # in-kernel state chain over peer memory: both launches are queued at once, the kernels wait for
            # the incoming state themselves and push the outgoing one into the next rank's buffer
            shape, bh = ctx.peer
            io_a = tr.peer_io("fwd_a", shape, bh, r - 1 if r > 0 else None, r + 1 if r < n - 1 else None)
            out_a, sT_a, saved_a, meta_a = core.forward(list(seg_a), state0 if r == 0 else None, peer=io_a)
            io_b = tr.peer_io("fwd_b", shape, bh, r + 1 if r < n - 1 else None, r - 1 if r > 0 else None)
            out_b, sT_b, saved_b, meta_b = core.forward(list(seg_b), sT_a if r == n - 1 else None, peer=io_b)
        else:
            # first segments: chunk r, chain 0 -> n-1
            if r > 0:
                h0 = tr.recv_state(core, list(seg_a), src=r - 1, tag="fwd_a")
            else:
                h0 = state0
            out_a, sT_a, saved_a, meta_a = core.forward(list(seg_a), h0)
            if r < n - 1:
                tr.send_state(sT_a, dst=r + 1, tag="fwd_a")
                h0b = tr.recv_state(core, list(seg_b), src=r + 1, tag="fwd_b")
            else:
                h0b = sT_a
            out_b, sT_b, saved_b, meta_b = core.forward(list(seg_b), h0b)
            if r > 0:
                tr.send_state(sT_b, dst=r - 1, tag="fwd_b")
        ctx.save_for_backward(*saved_a, *saved_b)
        ctx.counts, ctx.metas = [len(saved_a), len(saved_b)], [meta_a, meta_b]
        ctx.state_templates = tuple((s.shape, s.dtype) if s is not None else None for s in sT_b)
        out = torch.cat([out_a, out_b], dim=1)
        return (out, *[s if s is not None else out.new_zeros(()) for s in sT_b])

    @staticmethod
    def _backward(ctx, d_out, *d_state):
        core, sp = ctx.core, ctx.sp
        d_state = tuple(d_state) if len(d_state) else None
        if d_state is not None and all(ds is None for ds in d_state):
            d_state = None
        saved_all = list(ctx.saved_tensors)
        if sp is None or sp.size == 1:
            d_inputs, d_s0 = core.backward(saved_all, ctx.metas[0], d_out, d_state)
            grads = list(d_inputs) + (list(d_s0) if (d_s0 is not None and ctx.n_state0) else [None] * ctx.n_state0)
            return (None, None, None, None, *grads)
        r, n = sp.rank, sp.size
        tr = sp.transport
        half = d_out.shape[1] // 2
        d_a, d_b = d_out[:, :half], d_out[:, half:]
        if ctx.parallel:
            return _parallel_backward(ctx, core, sp, saved_all, d_a, d_b, d_state)
        saved_a, saved_b = saved_all[:ctx.counts[0]], saved_all[ctx.counts[0]:]
        device = d_out.device
        if ctx.peer is not None:
            shape, bh = ctx.peer
            io_b = tr.peer_io("bwd_b", shape, bh, r - 1 if r > 0 else None, r + 1 if r < n - 1 else None)
            d_in_b, d_h0b = core.backward(saved_b, ctx.metas[1], d_b, d_state if r == 0 else None, peer=io_b)
            io_a = tr.peer_io("bwd_a", shape, bh, r + 1 if r < n - 1 else None, r - 1 if r > 0 else None)
            d_in_a, d_h0a = core.backward(saved_a, ctx.metas[0], d_a, d_h0b if r == n - 1 else None, peer=io_a)
        else:
            # second segments first: chain 0 -> n-1 (reverse of the forward chain n-1 -> 0)
            if r > 0:
                dhT_b = tr.recv_state_like(ctx.state_templates, device, src=r - 1, tag="bwd_b")
            else:
                dhT_b = d_state
            d_in_b, d_h0b = core.backward(saved_b, ctx.metas[1], d_b, dhT_b)
            if r < n - 1:
                tr.send_state(d_h0b, dst=r + 1, tag="bwd_b")
                dhT_a = tr.recv_state_like(ctx.state_templates, device, src=r + 1, tag="bwd_a")
            else:
                dhT_a = d_h0b
            d_in_a, d_h0a = core.backward(saved_a, ctx.metas[0], d_a, dhT_a)
            if r > 0:
                tr.send_state(d_h0a, dst=r - 1, tag="bwd_a")
        d_inputs = []
        for ga, gb in zip(d_in_a, d_in_b):
            d_inputs.append(None if ga is None else torch.cat([ga, gb], dim=1))
        if ctx.n_state0:
            d_s0 = list(d_h0a) if (r == 0 and d_h0a is not None) else [None] * ctx.n_state0
        else:
            d_s0 = []
        return (None, None, None, None, *d_inputs, *d_s0)


def ssm_scan(core: ScanCore, inputs: Sequence[Tensor], initial_state: State = None, sp=None):
    """Runs ``core`` over ``inputs`` (time on dim 1).  Returns ``(out, final_state_tuple)``.

    Under sequence parallelism ``initial_state`` is only consumed by rank 0 (start of the
    global sequence) and the returned final state is the global one on rank 0 only."""
    state = () if initial_state is None else tuple(initial_state)
    res = _SSMScan.apply(core, sp, len(inputs), True, *inputs, *state)
    return res[0], tuple(res[1:])
