"""Chunk-parallel Chebyshev ridge solve of Gated KalmaNet for the GPU.

``ops.reference.gka_chebyshev_chunk`` walks the chunks one after the other (``N x num_iter`` rounds of small
launches).  Here the chunk-start covariance states are produced first for *all* chunks (a decay-weighted
cumulative sum over chunks, one GEMM), after which every chunk's ``num_iter`` Chebyshev steps run as one batch
over ``[B, H, N]``: ``num_iter`` rounds of four large batched GEMMs in fp32 / TF32 on the tensor cores, independent
of the sequence length.  Differentiable (used through ``TorchScanCore``, which re-evaluates it in backward).
Same math as the reference project's chunked kernels (``chebyshev_iteration.py:25-300``,
``chunk_fwd_h_kk`` in ``gka/ops``), evaluated with library GEMMs instead of one fused kernel.
"""
from __future__ import annotations

from typing import Optional

import torch

Tensor = torch.Tensor


def _prefix_kernel(U: Tensor, gl: Tensor, h0: Optional[Tensor]) -> Tensor:
    """``states[n + 1] = e^{gl[n]} states[n] + U[n]`` from ``states[0] = h0`` (zeros when ``None``): ``U [B,H,N,E]``,
    ``gl [B,H,N]``, all fp32 and contiguous -> ``[B,H,N+1,E]``.  One bandwidth-bound pass of the decayed prefix-sum
    kernel (``csrc/kernels/gdn_scan.cu::gla_segment_prefix_kernel``)."""
    import ctypes
    from . import _lib
    B, Hh, N, E = U.shape
    states = torch.empty(B, Hh, N + 1, E, device=U.device, dtype=torch.float32)
    ll = ctypes.c_longlong
    _lib.check(_lib.kernels().hmf_gla_segment_prefix(
        _lib.ptr(U), _lib.ptr(gl), _lib.ptr(h0), _lib.ptr(states), ctypes.c_void_p(states.data_ptr() + N * E * 4),
        ctypes.c_int(N), ctypes.c_int(B * Hh), ctypes.c_int(1), ctypes.c_int(E), ll(E), ll(N * E), ll(1), ll(N),
        ll(E), ll((N + 1) * E), ll((N + 1) * E), _lib.stream_ptr(U.device)), "gla_segment_prefix")
    return states


class _DecayedPrefix(torch.autograd.Function):
    """Differentiable form of :func:`_prefix_kernel`.  The gradient obeys the same recurrence run backwards
    (``R[n] = dS[n] + e^{gl[n]} R[n + 1]``), so the backward pass is the same kernel on the flipped sequence:
    ``dU[n] = R[n + 1]``, ``dgl[n] = e^{gl[n]} <R[n + 1], S[n]>``, ``dh0 = R[0]``.  Replaces a ``[N + 1, N]`` weight
    product whose cost grows with the square of the number of chunks (2048 chunks at 128K tokens)."""

    @staticmethod
    def forward(ctx, U, gl, h0):
        U, gl = U.float().contiguous(), gl.float().contiguous()
        h0c = None if h0 is None else h0.float().contiguous()
        states = _prefix_kernel(U, gl, h0c)
        ctx.save_for_backward(states, gl)
        ctx.has_h0 = h0 is not None
        return states

    @staticmethod
    def backward(ctx, dS):
        states, gl = ctx.saved_tensors
        N = gl.shape[-1]
        dS = dS.float()
        Q = _prefix_kernel(dS[:, :, :N].flip(2).contiguous(), gl.flip(-1).contiguous(), dS[:, :, N].contiguous())
        Rv = Q.flip(2)                                              # R[0 .. N]
        dU = Rv[:, :, 1:]
        dgl = torch.exp(gl) * (dU * states[:, :, :N]).sum(-1)
        return dU, dgl, (Rv[:, :, 0] if ctx.has_h0 else None)


def chunk_states(k: Tensor, G: Tensor, H0: Optional[Tensor]) -> Tensor:
    """``k [B,H,N,C,D]``, inclusive in-chunk cumulative gates ``G [B,H,N,C]`` -> states ``[B,H,N+1,D,D]``
    (state at the start of chunk ``n``; index ``N`` is the final state)."""
    B, Hh, N, C, D = k.shape
    Glast = G[..., -1]                                            # [B,H,N]
    kdec = k * torch.exp(Glast[..., None] - G)[..., None]
    U = kdec.transpose(-1, -2) @ k                                # [B,H,N,D,D] contribution of chunk m at its end
    if k.is_cuda and B * Hh <= 65535:
        # one pass of the decayed prefix-sum kernel (and one more, backwards, for the gradient) instead of the
        # [N+1, N] weight product
        from . import _lib
        if _lib.use_cuda_kernels(k):
            h0 = None if H0 is None else H0.reshape(B, Hh, D * D)
            Uf = U.reshape(B, Hh, N, D * D)
            if torch.is_grad_enabled() and (Uf.requires_grad or Glast.requires_grad or (h0 is not None and h0.requires_grad)):
                states = _DecayedPrefix.apply(Uf, Glast, h0)
            else:
                states = _prefix_kernel(Uf.float().contiguous(), Glast.float().contiguous(),
                                        None if h0 is None else h0.float().contiguous())
            return states.view(B, Hh, N + 1, D, D)
    tot = torch.cumsum(Glast, dim=-1)                             # log decay up to the end of chunk m
    tot0 = torch.cat([torch.zeros_like(tot[..., :1]), tot], dim=-1)          # [B,H,N+1]: up to the start of chunk n
    # state_n = e^{tot0_n} H0 + sum_{m<n} e^{tot0_n - tot_m} U_m
    diff = tot0[..., :, None] - tot[..., None, :]                 # [B,H,N+1,N]
    idx_n = torch.arange(N + 1, device=k.device)[:, None]
    idx_m = torch.arange(N, device=k.device)[None, :]
    lower = idx_m < idx_n
    W = torch.where(lower, torch.exp(torch.where(lower, diff, torch.zeros_like(diff))), torch.zeros_like(diff))
    states = (W @ U.reshape(B, Hh, N, D * D)).view(B, Hh, N + 1, D, D)
    if H0 is not None:
        states = states + torch.exp(tot0)[..., None, None] * H0[:, :, None]
    return states


def _kernel_ok(q: Tensor, k: Tensor, gk: Optional[Tensor], chunk_size: int) -> bool:
    from . import _lib
    if not (q.is_cuda and q.dtype == torch.bfloat16 and k.dtype == torch.bfloat16 and q.shape[-1] == 128
            and chunk_size == 64 and q.stride(-1) == 1 and k.stride(-1) == 1):
        return False
    if torch.is_grad_enabled() and (q.requires_grad or k.requires_grad or (gk is not None and gk.requires_grad)):
        return False                    # the backward differentiates the PyTorch formulation
    return _lib.use_cuda_kernels(q, k)


def _solve_kernel(q: Tensor, k: Tensor, gk: Optional[Tensor], states: Tensor, ridge_ratio: float, num_iter: int,
                  N: int) -> Tensor:
    """One CTA per (chunk, head); ``states [B,H,N+1,D,D]`` fp32 contiguous.  ``csrc/kernels/gka_cheb_tc.cu`` (tcgen05,
    operands read from shared memory by the tensor core, accumulators in tensor memory)."""
    import ctypes
    from . import _lib
    fn = _lib.kernels().hmf_gka_cheb_fwd_tc
    B, T, Hh, D = q.shape
    g = None if gk is None else gk.float().contiguous()
    states = states.contiguous()
    x = torch.empty(B, T, Hh, D, device=q.device, dtype=torch.float32)
    ll = ctypes.c_longlong
    _lib.check(fn(
        _lib.ptr(q), _lib.ptr(k), _lib.ptr(g), _lib.ptr(states), _lib.ptr(x), ctypes.c_int(B), ctypes.c_int(T),
        ctypes.c_int(Hh), ctypes.c_int(N), ctypes.c_int(states.shape[2]), ll(q.stride(0)), ll(q.stride(1)),
        ll(q.stride(2)), ll(k.stride(0)), ll(k.stride(1)), ll(k.stride(2)), ctypes.c_float(ridge_ratio),
        ctypes.c_int(num_iter), _lib.stream_ptr(q.device)), "gka_cheb_fwd")
    return x


def _chunk_layout(q: Optional[Tensor], k: Tensor, gk: Optional[Tensor], initial_state: Optional[Tensor], chunk_size: int,
                  need_mask: bool = True):
    """Pads to whole chunks and returns ``(qf, kf [B,H,N,C,D] fp32, G [B,H,N,C], m [B,H,N,C,C], states, N)``."""
    B, T, Hh, D = k.shape
    C = chunk_size
    pad = (-T) % C
    kf = k.float()
    qf = None if q is None else q.float()
    gf = torch.zeros(B, T, Hh, device=k.device) if gk is None else gk.float()
    if pad:
        z = lambda t: torch.cat([t, t.new_zeros(B, pad, *t.shape[2:])], dim=1)  # noqa: E731
        kf, gf = z(kf), z(gf)
        qf = None if qf is None else z(qf)
    N = (T + pad) // C
    if qf is not None:
        qf = qf.view(B, N, C, Hh, D).permute(0, 3, 1, 2, 4)       # [B,H,N,C,D]
    kf = kf.view(B, N, C, Hh, D).permute(0, 3, 1, 2, 4)
    G = gf.view(B, N, C, Hh).permute(0, 3, 1, 2).cumsum(-1)       # [B,H,N,C]
    m = None
    if need_mask:
        idx = torch.arange(C, device=k.device)
        lower = idx[:, None] >= idx[None, :]
        diff = G[..., :, None] - G[..., None, :]
        m = torch.where(lower, torch.exp(torch.where(lower, diff, torch.zeros_like(diff))), torch.zeros_like(diff))
    H0 = None if initial_state is None else initial_state.float()
    states = chunk_states(kf, G, H0)
    return qf, kf, G, m, states, N


def _fro(kf: Tensor, G: Tensor, m: Tensor, Hs: Tensor) -> Tensor:
    """``|H_i|_F`` for every token, ``[B,H,N,C,1]`` (closed form over the chunk: Gram, state and cross terms)."""
    eg = torch.exp(G)[..., None]
    gram = kf @ kf.transpose(-1, -2)
    fro2 = ((m @ (gram * gram)) * m).sum(-1, keepdim=True)
    fro2 = fro2 + eg * eg * Hs.pow(2).sum((-1, -2))[..., None, None]
    kHk = (kf * (kf @ Hs)).sum(-1)
    fro2 = fro2 + 2 * eg * (m * kHk[..., None, :]).sum(-1, keepdim=True)
    return fro2.clamp(min=0).sqrt()


def chunk_fro(k: Tensor, gk: Optional[Tensor], initial_state: Optional[Tensor], chunk_size: int = 64):
    """``(|H_t|_F  [B,T,H], H_T [B,H,D,D])``, differentiable in ``k``, ``gk`` and the initial state."""
    B, T, Hh, D = k.shape
    _, kf, G, m, states, N = _chunk_layout(None, k, gk, initial_state, chunk_size)
    fro = _fro(kf, G, m, states[:, :, :N])
    return fro[..., 0].permute(0, 2, 3, 1).reshape(B, N * chunk_size, Hh)[:, :T], states[:, :, N]


def chebyshev_chunk_parallel(q: Tensor, k: Tensor, gk: Optional[Tensor], *, ridge_ratio: float = 0.02,
                             num_iter: int = 30, initial_state: Optional[Tensor] = None, chunk_size: int = 64):
    """Returns ``(x [B,T,H,D] fp32, H_T [B,H,D,D] fp32)``; see ``ops.reference.gka_chebyshev_chunk``."""
    B, T, Hh, D = q.shape
    C = chunk_size
    if _kernel_ok(q, k, gk, chunk_size):
        # no graph to record (inference, forward of the scan core): the whole per-chunk solve runs in one kernel,
        # which builds the decay mask and reads q itself; only the chunk-start states are prepared here
        _, _, _, _, states, N = _chunk_layout(None, k, gk, initial_state, chunk_size, need_mask=False)
        return _solve_kernel(q, k, gk, states, ridge_ratio, num_iter, N), states[:, :, N]
    qf, kf, G, m, states, N = _chunk_layout(q, k, gk, initial_state, chunk_size)
    Hs = states[:, :, :N]                                         # [B,H,N,D,D]
    eg = torch.exp(G)[..., None]                                  # [B,H,N,C,1]
    fro = _fro(kf, G, m, Hs)
    lam = ridge_ratio * fro
    denom = 2 * lam + fro
    denom = torch.where(denom == 0, torch.ones_like(denom), denom)
    step = 2.0 / denom
    c = (fro / denom / 2.0) ** 2
    kT = kf.transpose(-1, -2)
    x_prev = torch.zeros_like(qf)
    x = step * qf
    omega = torch.full_like(fro, 2.0)
    for _ in range(num_iter):
        omega = 1.0 / (1.0 - c * omega)
        Hx = (x * eg) @ Hs + ((x @ kT) * m) @ kf
        upd = step * omega * (Hx + lam * x - qf) + (omega - 1.0) * x_prev
        x_prev = x
        x = omega * x - upd
    out = x.permute(0, 2, 3, 1, 4).reshape(B, N * C, Hh, D)[:, :T]
    return out, states[:, :, N]


class ChebyshevCore:
    """Scan core of the ridge solve on the GPU: forward by the one-kernel solve, backward by implicit
    differentiation of ``(H_t + lam_t I) x_t = q_t`` — the way the reference's backward works
    (``chebyshev_iteration.py:606-690``):

    * ``dq_t = (H_t + lam_t I)^-1 dx_t``: the same solve with the upstream gradient as right-hand side;
    * ``dH_t = -x_t dq_t^T`` reaches ``k``, the gates and the incoming state through the gated-linear-attention form
      ``x_t H_t = GLA(q=x, k=k, v=k)_t`` contracted with ``dq`` (chunked GLA kernels, their own backward);
    * ``dlam_t = -dq_t . x_t`` reaches them through ``lam_t = ridge |H_t|_F`` and the closed form of ``|H_t|_F``.
    """
    n_state = 1

    def __init__(self, ridge_ratio: float, num_iter: int, chunk_size: int = 64, bp_lambda: bool = True):
        self.ridge_ratio, self.num_iter, self.chunk_size, self.bp_lambda = ridge_ratio, num_iter, chunk_size, bp_lambda

    @staticmethod
    def supported(q: Tensor, k: Tensor, gk: Optional[Tensor], chunk_size: int) -> bool:
        with torch.no_grad():
            return _kernel_ok(q.detach(), k.detach(), None if gk is None else gk.detach(), chunk_size)

    def state_shapes(self, inputs):
        q = inputs[0]
        return [((q.shape[0], q.shape[2], q.shape[3], q.shape[3]), torch.float32)]

    def forward(self, inputs, state0):
        q, k, gk = inputs
        h0 = None if state0 is None else state0[0]
        with torch.no_grad():
            x, hT = chebyshev_chunk_parallel(q, k, gk, ridge_ratio=self.ridge_ratio, num_iter=self.num_iter,
                                             initial_state=h0, chunk_size=self.chunk_size)
        saved = [q, k, gk, x] + ([h0] if h0 is not None else [])
        return x, (hT,), saved, h0 is not None

    def backward(self, saved, meta, d_out, d_stateT):
        from . import mixers
        q, k, gk, x = saved[:4]
        h0 = saved[4] if meta else None
        with torch.no_grad():
            dq, _ = chebyshev_chunk_parallel(d_out.to(q.dtype), k, gk, ridge_ratio=self.ridge_ratio,
                                             num_iter=self.num_iter, initial_state=h0, chunk_size=self.chunk_size)
            dlam = -(dq * x).sum(-1)                                        # [B,T,H]
        k1 = k.detach().requires_grad_(True)
        g1 = None if gk is None else gk.detach().float().requires_grad_(True)
        h1 = None if h0 is None else h0.detach().float().requires_grad_(True)
        with torch.enable_grad():
            gz = torch.zeros(k.shape[:3], device=k.device) if g1 is None else g1
            # the forward multiplies rows from the left (x_t H_t), so dH_t = -x_t dq_t^T: x takes the query role
            o, hT = mixers.simple_gla(x.to(k.dtype), k1, k1, gz, scale=1.0, initial_state=h1,
                                      chunk_size=self.chunk_size)
            term = -(dq * o.float()).sum()
            d_hT = None if d_stateT is None else d_stateT[0]
            if d_hT is not None:
                term = term + (d_hT.float() * hT.float()).sum()
            if self.bp_lambda:
                fro, _ = chunk_fro(k1, g1, h1, self.chunk_size)
                term = term + (self.ridge_ratio * dlam * fro).sum()
            wrt = [t for t in (k1, g1, h1) if t is not None]
            grads = list(torch.autograd.grad(term, wrt, allow_unused=True))
        dk = grads.pop(0)
        dgk = grads.pop(0) if g1 is not None else None
        dh0 = grads.pop(0) if h1 is not None else None
        d_inputs = [dq.to(q.dtype), torch.zeros_like(k) if dk is None else dk.to(k.dtype),
                    None if gk is None else (torch.zeros_like(gk) if dgk is None else dgk.to(gk.dtype))]
        d_s0 = None if h0 is None else ((torch.zeros_like(h0) if dh0 is None else dh0.to(h0.dtype)),)
        return d_inputs, d_s0
