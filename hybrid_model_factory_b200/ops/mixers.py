"""Mixer-level ops (Gated DeltaNet, Gated KalmaNet, Mamba2 SSD) on top of ``ops.scan``.

Each function builds the scan core for the device of its inputs (CUDA kernels or the PyTorch
reference) and runs it through :func:`ops.scan.ssm_scan`, which also handles the
sequence-parallel state chain.  Decode steps (``recurrent=True``) use the token-by-token
kernels / definitions.
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch

from . import _lib
from . import reference as R
from .scan import TorchScanCore, ssm_scan

Tensor = torch.Tensor


# -- Gated DeltaNet ------------------------------------------------------------------------
def _gdn_state_shapes(inputs):
    q, k, v = inputs[0], inputs[1], inputs[2]
    return [((q.shape[0], q.shape[2], q.shape[3], v.shape[3]), torch.float32)]


def gated_delta_rule(q: Tensor, k: Tensor, v: Tensor, g: Tensor, beta: Tensor, *, scale: Optional[float] = None,
                     initial_state: Optional[Tensor] = None, sp=None, chunk_size: int = 64,
                     use_qk_l2norm: bool = True, recurrent: bool = False) -> Tuple[Tensor, Tensor]:
    """Gated delta rule over ``q,k [B,T,H,Dk]``, ``v [B,T,H,Dv]``, ``g,beta [B,T,H]``.
    Returns ``(o [B,T,H,Dv], final_state [B,H,Dk,Dv] fp32)``."""
    if _lib.use_cuda_kernels(q, k, v):
        from . import cuda_ops
        core = cuda_ops.GDNCore(scale=scale, chunk_size=chunk_size, use_qk_l2norm=use_qk_l2norm, recurrent=recurrent)
    else:
        fn = R.gated_delta_rule_recurrent if recurrent else R.gated_delta_rule_chunk
        kw = dict(scale=scale, use_qk_l2norm=use_qk_l2norm)
        if not recurrent:
            kw["chunk_size"] = chunk_size
        core = TorchScanCore(fn, n_state=1, state_shape_fn=_gdn_state_shapes, **kw)
    state = None if initial_state is None else (initial_state,)
    o, (sT,) = ssm_scan(core, [q, k, v, g, beta], state, sp)
    return o, sT


# -- Gated KalmaNet --------------------------------------------------------------------------
def _gka_state_shapes(inputs):
    q, v = inputs[0], inputs[2]
    B, H, D = q.shape[0], q.shape[2], q.shape[3]
    return [((B, H, D, D), torch.float32), ((B, H, D, v.shape[3]), torch.float32)]


def _gka_ref(q, k, v, alpha, g, gk, initial_state=None, **kw):
    return R.gka_forward(q, k, v, alpha, g, gk, initial_state=initial_state, **kw)


def gka(q: Tensor, k: Tensor, v: Tensor, alpha: Optional[Tensor], g: Tensor, gk: Optional[Tensor], *,
        scale: Optional[float] = None, ridge_ratio: float = 0.02, num_iter: int = 30,
        initial_state: Optional[Tuple[Tensor, Tensor]] = None, sp=None, chunk_size: int = 64,
        recurrent: bool = False):
    """GKA core: Chebyshev ridge solve against the running key covariance, alpha-mix, simple GLA.
    Returns ``(o, (h_kk, h_kv))`` with both states ``[B,H,D,D]`` in fp32."""
    if _lib.use_cuda_kernels(q, k, v):
        from . import cuda_ops
        core = cuda_ops.GKACore(scale=scale, ridge_ratio=ridge_ratio, num_iter=num_iter, chunk_size=chunk_size,
                                recurrent=recurrent)
    else:
        core = TorchScanCore(_gka_ref, n_state=2, state_shape_fn=_gka_state_shapes, scale=scale,
                             ridge_ratio=ridge_ratio, num_iter=num_iter, chunk_size=chunk_size, recurrent=recurrent)
    state = None
    if initial_state is not None and initial_state[1] is not None:
        h_kk0, h_kv0 = initial_state
        if h_kk0 is None:
            h_kk0 = torch.zeros(q.shape[0], q.shape[2], q.shape[3], q.shape[3], device=q.device)
        state = (h_kk0, h_kv0)
    o, sT = ssm_scan(core, [q, k, v, alpha, g, gk], state, sp)
    return o, (sT[0] if sT[0].dim() else None, sT[1])


# -- Mamba2 SSD ------------------------------------------------------------------------------
def _ssd_state_shapes(inputs):
    x, Bm = inputs[0], inputs[3]
    return [((x.shape[0], x.shape[2], x.shape[3], Bm.shape[3]), torch.float32)]


def _ssd_ref(x, dt, g, Bm, Cm, initial_state=None, chunk_size=256, recurrent=False):
    H, Gr = x.shape[2], Bm.shape[2]
    kq = Bm.float().repeat_interleave(H // Gr, dim=2)
    qq = Cm.float().repeat_interleave(H // Gr, dim=2)
    v = x.float() * dt.float()[..., None]
    h0 = None if initial_state is None else initial_state.float().transpose(-1, -2)
    if recurrent:
        y, hT = R.simple_gla_recurrent(qq, kq, v, g, scale=1.0, initial_state=h0)
    else:
        y, hT = R.simple_gla_chunk(qq, kq, v, g, scale=1.0, initial_state=h0, chunk_size=chunk_size)
    return y, hT.transpose(-1, -2)


def ssd(x: Tensor, dt: Tensor, A: Tensor, Bm: Tensor, Cm: Tensor, D: Optional[Tensor] = None, *,
        initial_state: Optional[Tensor] = None, sp=None, chunk_size: int = 256, recurrent: bool = False):
    """Mamba2 selective state-space scan.  ``x [B,T,H,P]``, ``dt [B,T,H]`` (post-softplus),
    ``A [H]``, ``Bm,Cm [B,T,G,N]``.  Returns ``(y [B,T,H,P], state [B,H,P,N] fp32)``."""
    g = dt.float() * A.float()
    if _lib.use_cuda_kernels(x, dt, Bm, Cm):
        from . import cuda_ops
        core = cuda_ops.SSDCore(chunk_size=chunk_size, recurrent=recurrent)
    else:
        core = TorchScanCore(_ssd_ref, n_state=1, state_shape_fn=_ssd_state_shapes, chunk_size=chunk_size,
                             recurrent=recurrent)
    state = None if initial_state is None else (initial_state,)
    y, (sT,) = ssm_scan(core, [x, dt, g, Bm, Cm], state, sp)
    if D is not None:
        y = y + D.float()[None, None, :, None] * x.float()
    return y, sT
