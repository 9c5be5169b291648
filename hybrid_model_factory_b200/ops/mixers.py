"""Mixer-level ops (Gated DeltaNet, Gated KalmaNet, Mamba2 SSD) on top of ``ops.scan``.

Each function builds the scan core for the device of its inputs (CUDA kernels or the PyTorch
reference) and runs it through :func:`ops.scan.ssm_scan`, which also handles the
sequence-parallel state chain.  Decode steps (``recurrent=True``) use the token-by-token
definitions (the serving engine has dedicated slot-indexed decode kernels).

Mamba2's SSD and GKA's output stage are both plain gated linear attention
(``S_t = e^{g_t} S_{t-1} + k_t v_t^T``), which the GDN kernels evaluate in their ``gla`` mode
(WY factors degenerate to ``w = 0``, ``u = v``).
"""
from __future__ import annotations

import os

from typing import Optional, Tuple

import torch

from . import _lib
from . import reference as R
from .scan import TorchScanCore, ssm_scan

Tensor = torch.Tensor


def _qkv_state_shapes(inputs):
    q, v = inputs[0], inputs[2]
    return [((q.shape[0], q.shape[2], q.shape[3], v.shape[3]), torch.float32)]


KERNEL_DIM = 128     # key / value width the chunk kernels are written for


def _pad_to_kernel_width(q: Tensor, k: Tensor, v: Tensor, initial_state: Optional[Tensor], scale: Optional[float]):
    """The chunk kernels work on 128-wide keys and values.  Narrower heads (Mamba2 with head_dim 64 and d_state 128,
    small test models) are zero-padded to that width instead of leaving the tensor cores: zero key columns add nothing
    to any score or state row, zero value columns produce zero outputs, so the result is the same and only the value
    side does up to 2x the arithmetic.  Returns the padded tensors, the scale of the unpadded problem and ``(Dk, Dv)``
    (``None`` when nothing was padded)."""
    Dk, Dv = q.shape[-1], v.shape[-1]
    if not (q.is_cuda and q.dtype == torch.bfloat16) or (Dk == KERNEL_DIM and Dv == KERNEL_DIM) \
            or Dk > KERNEL_DIM or Dv > KERNEL_DIM:
        return q, k, v, initial_state, scale, None
    import torch.nn.functional as F
    scale = Dk ** -0.5 if scale is None else scale
    q = F.pad(q, (0, KERNEL_DIM - Dk))
    k = F.pad(k, (0, KERNEL_DIM - Dk))
    v = F.pad(v, (0, KERNEL_DIM - Dv))
    if initial_state is not None:
        initial_state = F.pad(initial_state, (0, KERNEL_DIM - Dv, 0, KERNEL_DIM - Dk))
    return q, k, v, initial_state, scale, (Dk, Dv)


def _unpad(o: Tensor, sT: Tensor, dims):
    if dims is None:
        return o, sT
    Dk, Dv = dims
    return o[..., :Dv], (sT[..., :Dk, :Dv] if sT is not None and sT.dim() >= 2 else sT)


# -- Gated DeltaNet ------------------------------------------------------------------------
def gated_delta_rule(q: Tensor, k: Tensor, v: Tensor, g: Tensor, beta: Tensor, *, scale: Optional[float] = None,
                     initial_state: Optional[Tensor] = None, sp=None, chunk_size: int = 64,
                     use_qk_l2norm: bool = True, recurrent: bool = False) -> Tuple[Tensor, Tensor]:
    """Gated delta rule over ``q,k [B,T,H,Dk]``, ``v [B,T,H,Dv]``, ``g,beta [B,T,H]``.
    Returns ``(o [B,T,H,Dv], final_state [B,H,Dk,Dv] fp32)``."""
    dims = None
    if _lib.use_cuda_kernels(q, k, v) and not recurrent:
        q, k, v, initial_state, scale, dims = _pad_to_kernel_width(q, k, v, initial_state, scale)
    if _lib.use_cuda_kernels(q, k, v):
        from . import cuda_ops
        core = cuda_ops.GDNCore(scale=scale, chunk_size=chunk_size, use_qk_l2norm=use_qk_l2norm, recurrent=recurrent)
    else:
        fn = R.gated_delta_rule_recurrent if recurrent else R.gated_delta_rule_chunk
        kw = dict(scale=scale, use_qk_l2norm=use_qk_l2norm)
        if not recurrent:
            kw["chunk_size"] = chunk_size
        core = TorchScanCore(fn, n_state=1, state_shape_fn=_qkv_state_shapes, **kw)
    core.matrix_transition, core.value_input = True, 2       # S_out = A S_in + S_local with A from (k, beta, g) only
    state = None if initial_state is None else (initial_state,)
    o, (sT,) = ssm_scan(core, [q, k, v, g, beta], state, sp)
    return _unpad(o, sT, dims)


# -- plain gated linear attention ------------------------------------------------------------
def _gla_ref(q, k, v, g, beta=None, initial_state=None, scale=None, chunk_size=64, recurrent=False):
    if recurrent:
        return R.simple_gla_recurrent(q, k, v, g, scale=scale, initial_state=initial_state)
    return R.simple_gla_chunk(q, k, v, g, scale=scale, initial_state=initial_state, chunk_size=chunk_size)


def simple_gla(q: Tensor, k: Tensor, v: Tensor, g: Tensor, *, scale: Optional[float] = None,
               initial_state: Optional[Tensor] = None, sp=None, chunk_size: int = 64, recurrent: bool = False):
    """``S_t = e^{g_t} S_{t-1} + k_t v_t^T``, ``o_t = S_t^T q_t * scale``.  State ``[B,H,Dk,Dv]`` fp32."""
    core, dims = None, None
    if _lib.use_cuda_kernels(q, k, v) and not recurrent:
        q, k, v, initial_state, scale, dims = _pad_to_kernel_width(q, k, v, initial_state, scale)
    if _lib.use_cuda_kernels(q, k, v) and not recurrent:
        from . import gdn_cuda
        if gdn_cuda.available():
            core = gdn_cuda.GDNChunkCore(scale=scale, use_qk_l2norm=False, gla=True)
    if core is None:
        core = TorchScanCore(_gla_ref, n_state=1, state_shape_fn=_qkv_state_shapes, scale=scale,
                             chunk_size=chunk_size, recurrent=recurrent)
    core.scalar_transition, core.decay_input = True, 3       # S_out = e^{sum g} S_in + S_local: chain-free SP possible
    state = None if initial_state is None else (initial_state,)
    o, (sT,) = ssm_scan(core, [q, k, v, g, None], state, sp)
    return _unpad(o, sT, dims)


# -- Gated KalmaNet --------------------------------------------------------------------------
def _cheb_state_shapes(inputs):
    q = inputs[0]
    B, H, D = q.shape[0], q.shape[2], q.shape[3]
    return [((B, H, D, D), torch.float32)]


def _cheb_ref(q, k, gk, initial_state=None, ridge_ratio=0.02, num_iter=30, chunk_size=64, recurrent=False):
    if not recurrent and q.is_cuda:
        # all chunks at once: num_iter rounds of large batched GEMMs instead of N x num_iter small ones
        from .gka_parallel import chebyshev_chunk_parallel
        return chebyshev_chunk_parallel(q, k, gk, ridge_ratio=ridge_ratio, num_iter=num_iter,
                                        initial_state=initial_state, chunk_size=chunk_size)
    if recurrent:
        return R.gka_chebyshev_recurrent(q, k, gk, ridge_ratio=ridge_ratio, num_iter=num_iter,
                                         initial_state=initial_state)
    return R.gka_chebyshev_chunk(q, k, gk, ridge_ratio=ridge_ratio, num_iter=num_iter, initial_state=initial_state,
                                 chunk_size=chunk_size)


def chebyshev_solve(q: Tensor, k: Tensor, gk: Optional[Tensor], *, ridge_ratio: float = 0.02, num_iter: int = 30,
                    initial_state: Optional[Tensor] = None, sp=None, chunk_size: int = 64, recurrent: bool = False):
    """Per-token ridge solve ``(H_t + lambda_t I) x_t = q_t`` (``H_t`` the decayed key covariance).
    Returns ``(x [B,T,H,D] fp32, H_T [B,H,D,D] fp32)``."""
    core = None
    if not recurrent and q.is_cuda and os.environ.get("HMF_GKA_KERNEL", "1") == "1":
        from .gka_parallel import ChebyshevCore
        if ChebyshevCore.supported(q, k, gk, chunk_size):       # one-kernel solve, implicit backward
            core = ChebyshevCore(ridge_ratio, num_iter, chunk_size)
    if core is None:
        core = TorchScanCore(_cheb_ref, n_state=1, state_shape_fn=_cheb_state_shapes, ridge_ratio=ridge_ratio,
                             num_iter=num_iter, chunk_size=chunk_size, recurrent=recurrent)
    core.scalar_transition, core.decay_input = True, 2       # the key covariance decays by e^{sum gk} per segment
    state = None if initial_state is None else (initial_state,)
    x, (hT,) = ssm_scan(core, [q, k, gk], state, sp)
    return x, hT


def gka(q: Tensor, k: Tensor, v: Tensor, alpha: Optional[Tensor], g: Tensor, gk: Optional[Tensor], *,
        scale: Optional[float] = None, ridge_ratio: float = 0.02, num_iter: int = 30,
        initial_state: Optional[Tuple[Tensor, Tensor]] = None, sp=None, chunk_size: int = 64,
        recurrent: bool = False):
    """GKA core: Chebyshev ridge solve against the running key covariance, alpha-mix, simple GLA.
    Returns ``(o, (h_kk, h_kv))`` with both states ``[B,H,D,D]`` in fp32."""
    h_kk0, h_kv0 = (None, None) if initial_state is None else initial_state
    h_kk = None
    qm = q
    if num_iter > 0:
        x, h_kk = chebyshev_solve(q, k, gk, ridge_ratio=ridge_ratio, num_iter=num_iter, initial_state=h_kk0, sp=sp,
                                  chunk_size=chunk_size, recurrent=recurrent)
        qf = q.float()
        qm = (qf + alpha.float()[..., None] * (x - qf)) if alpha is not None else x
        qm = qm.to(q.dtype)
    o, h_kv = simple_gla(qm, k, v, g, scale=scale, initial_state=h_kv0, sp=sp, chunk_size=chunk_size,
                         recurrent=recurrent)
    return o, (h_kk, h_kv)


# -- Mamba2 SSD ------------------------------------------------------------------------------
def ssd(x: Tensor, dt: Tensor, A: Tensor, Bm: Tensor, Cm: Tensor, D: Optional[Tensor] = None, *,
        initial_state: Optional[Tensor] = None, sp=None, chunk_size: int = 256, recurrent: bool = False):
    """Mamba2 selective state-space scan.  ``x [B,T,H,P]``, ``dt [B,T,H]`` (post-softplus),
    ``A [H]``, ``Bm,Cm [B,T,G,N]``.  Returns ``(y [B,T,H,P], state [B,H,P,N] fp32)``.
    Evaluated as gated linear attention with ``q=C``, ``k=B``, ``v=dt*x``, ``g=dt*A`` (state transposed)."""
    H, Gr = x.shape[2], Bm.shape[2]
    rep = H // Gr
    g = dt.float() * A.float()
    v = (x.float() * dt.float()[..., None]).to(x.dtype)
    k = Bm if rep == 1 else Bm.repeat_interleave(rep, dim=2)
    q = Cm if rep == 1 else Cm.repeat_interleave(rep, dim=2)
    h0 = None if initial_state is None else initial_state.float().transpose(-1, -2).contiguous()
    on_cuda = _lib.use_cuda_kernels(x, Bm, Cm)
    y, hT = simple_gla(q, k, v, g, scale=1.0, initial_state=h0, sp=sp, chunk_size=64 if on_cuda else chunk_size,
                       recurrent=recurrent)
    if D is not None:
        y = y.float() + D.float()[None, None, :, None] * x.float()
    return y, hT.transpose(-1, -2)
