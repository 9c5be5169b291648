"""Plain PyTorch reference implementations (oracles) of every hot op.

These functions define the numerical contract of the CUDA kernels: the GPU tests compare
each kernel against the function of the same name here evaluated in fp32, and CPU runs
(unit tests, the gloo sequence-parallel test, stage-0 priming) execute them directly.  They
are differentiable through autograd, which is also how the backward kernels are checked.

Math follows the reference project's layers:
  * Gated DeltaNet: ``layers/gated_deltanet/gdn.py:401-487`` (chunked gated delta rule)
  * Gated KalmaNet: ``layers/gated_kalmanet/ops/chebyshev/chebyshev_iteration.py:388-434``
    and ``gka_chebyshev_solve.py:107-164``
  * Mamba2 SSD: ``layers/mamba/mamba2.py:442-661``
  * B'MOJO-F merge: ``layers/bmojo_f/bmojo_attention_utils.py:409-426``
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch
import torch.nn.functional as F

Tensor = torch.Tensor


# ----------------------------------------------------------------------------------------
# Elementwise / normalisation
# ----------------------------------------------------------------------------------------
def rms_norm(x: Tensor, weight: Optional[Tensor], eps: float = 1e-6, zero_centered: bool = False) -> Tensor:
    """``x / sqrt(mean(x^2) + eps) * w`` computed in fp32, returned in ``x.dtype``.
    ``zero_centered`` uses ``(1 + w)`` as the scale (Qwen3-Next convention)."""
    xf = x.float()
    y = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)
    if weight is not None:
        w = weight.float()
        y = y * (1.0 + w if zero_centered else w)
    return y.to(x.dtype)


def fused_add_rms_norm(x: Tensor, residual: Tensor, weight: Tensor, eps: float = 1e-6) -> Tuple[Tensor, Tensor]:
    """``residual' = x + residual`` (stored in ``x.dtype``); returns ``(rms_norm(residual'), residual')``."""
    r = (x.float() + residual.float()).to(x.dtype)
    return rms_norm(r, weight, eps), r


def gated_rms_norm(x: Tensor, gate: Tensor, weight: Tensor, eps: float = 1e-5, norm_before_gate: bool = True) -> Tensor:
    """Per-head gated RMSNorm over the last dim.

    ``norm_before_gate=True``  (GDN/GKA): ``rms_norm(x) * w * silu(gate)``
    ``norm_before_gate=False`` (Mamba2):  ``rms_norm(x * silu(gate)) * w``
    """
    xf, gf = x.float(), gate.float()
    if norm_before_gate:
        y = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps) * weight.float()
        y = y * F.silu(gf)
    else:
        xf = xf * F.silu(gf)
        y = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps) * weight.float()
    return y.to(x.dtype)


def l2_norm(x: Tensor, eps: float = 1e-6) -> Tensor:
    xf = x.float()
    return (xf * torch.rsqrt(xf.pow(2).sum(-1, keepdim=True) + eps)).to(x.dtype)


def swiglu(gate: Tensor, up: Tensor) -> Tensor:
    return (F.silu(gate.float()) * up.float()).to(gate.dtype)


def rope_tables(positions: Tensor, dim: int, theta: float = 1e6) -> Tuple[Tensor, Tensor]:
    """cos/sin tables ``[..., dim]`` (each half repeated, rotate-half convention)."""
    inv = 1.0 / (theta ** (torch.arange(0, dim, 2, dtype=torch.float32, device=positions.device) / dim))
    freqs = positions.float()[..., None] * inv
    emb = torch.cat([freqs, freqs], dim=-1)
    return emb.cos(), emb.sin()


def apply_rope(x: Tensor, cos: Tensor, sin: Tensor, rotary_dim: Optional[int] = None) -> Tensor:
    """Rotate-half RoPE on ``x [B, T, H, D]`` with tables ``[B, T, R]`` (``R <= D``)."""
    R = cos.shape[-1] if rotary_dim is None else rotary_dim
    xr, xp = x[..., :R].float(), x[..., R:]
    c, s = cos[..., None, :R].float(), sin[..., None, :R].float()
    x1, x2 = xr[..., : R // 2], xr[..., R // 2:]
    rot = torch.cat([-x2, x1], dim=-1)
    out = (xr * c + rot * s).to(x.dtype)
    return torch.cat([out, xp], dim=-1) if xp.shape[-1] else out


def softplus(x: Tensor) -> Tensor:
    return F.softplus(x.float())


def gka_prepare(q: Tensor, k: Tensor, v: Tensor, beta: Optional[Tensor] = None, eps: float = 1e-6):
    """Gated KalmaNet input preparation: ``q / (|q| + eps)``, ``(beta + eps) k / (|k| + eps)``, ``(beta + eps) v`` with
    the norms over the last dimension and ``beta [...]`` one value per row (``None``: factor 1).  fp32 math, results in
    the input dtype."""
    qf, kf, vf = q.float(), k.float(), v.float()
    qn = qf / (torch.linalg.vector_norm(qf, dim=-1, keepdim=True) + eps)
    kn = kf / (torch.linalg.vector_norm(kf, dim=-1, keepdim=True) + eps)
    if beta is not None:
        c = beta.float()[..., None] + eps
        kn, vf = c * kn, c * vf
    return qn.to(q.dtype), kn.to(k.dtype), vf.to(v.dtype)


def gdn_gating(a: Tensor, b: Tensor, A_log: Tensor, dt_bias: Tensor, beta_scale: float = 1.0) -> Tuple[Tensor, Tensor]:
    """``g = -exp(A_log) * softplus(a + dt_bias)`` (fp32), ``beta = sigmoid(b) * beta_scale``."""
    g = -torch.exp(A_log.float()) * F.softplus(a.float() + dt_bias.float())
    beta = torch.sigmoid(b.float()) * beta_scale
    return g, beta


# ----------------------------------------------------------------------------------------
# Depthwise causal conv1d (+ SiLU)
# ----------------------------------------------------------------------------------------
def causal_conv1d(x: Tensor, weight: Tensor, bias: Optional[Tensor] = None, activation: Optional[str] = "silu",
                  initial_state: Optional[Tensor] = None, return_final_state: bool = False):
    """``x [B, T, C]``, ``weight [C, K]``; token t sees ``x[t-K+1 .. t]``.

    ``initial_state [B, K-1, C]`` supplies the tokens before position 0 (cache or a
    sequence-parallel halo); zeros when absent.  The final state is the last ``K-1`` inputs.
    """
    B, T, C = x.shape
    K = weight.shape[-1]
    if initial_state is None:
        initial_state = x.new_zeros(B, K - 1, C)
    xp = torch.cat([initial_state.to(x.dtype), x], dim=1)  # [B, T+K-1, C]
    y = F.conv1d(xp.transpose(1, 2).float(), weight.float().unsqueeze(1), None if bias is None else bias.float(),
                 groups=C).transpose(1, 2)
    if activation in ("silu", "swish"):
        y = F.silu(y)
    y = y.to(x.dtype)
    if return_final_state:
        return y, xp[:, T:, :]
    return y


def causal_conv1d_update(x: Tensor, conv_state: Tensor, weight: Tensor, bias: Optional[Tensor] = None,
                         activation: Optional[str] = "silu") -> Tuple[Tensor, Tensor]:
    """Single-token step: ``x [B, C]``, ``conv_state [B, K-1, C]`` -> ``(y [B, C], new_state)``."""
    window = torch.cat([conv_state.to(x.dtype), x[:, None, :]], dim=1)  # [B, K, C]
    y = (window.float() * weight.float().t()[None]).sum(1)
    if bias is not None:
        y = y + bias.float()
    if activation in ("silu", "swish"):
        y = F.silu(y)
    return y.to(x.dtype), window[:, 1:, :]


# ----------------------------------------------------------------------------------------
# Softmax attention (GQA; causal / sliding window / hollow window / explicit positions)
# ----------------------------------------------------------------------------------------
def attention_mask(q_pos: Tensor, k_pos: Tensor, causal: bool = True, window: Optional[int] = None,
                   hollow: Optional[int] = None) -> Tensor:
    """Boolean ``[..., Tq, Tk]`` visibility from absolute positions.

    causal: ``k <= q``.  window ``w``: ``q - k < w``.  hollow ``w`` (B'MOJO fading stream):
    ``w <= q - k < 2w`` i.e. query i sees keys ``[i-2w+1, i-w]``.
    """
    d = q_pos[..., :, None] - k_pos[..., None, :]
    m = torch.ones_like(d, dtype=torch.bool)
    if causal:
        m &= d >= 0
    if window is not None:
        m &= d < window
    if hollow is not None:
        m &= (d >= hollow) & (d < 2 * hollow)
    return m


def attention(q: Tensor, k: Tensor, v: Tensor, *, scale: Optional[float] = None, causal: bool = True,
              window: Optional[int] = None, hollow: Optional[int] = None, q_pos: Optional[Tensor] = None,
              k_pos: Optional[Tensor] = None, return_lse: bool = False):
    """``q [B, Tq, Hq, D]``, ``k, v [B, Tk, Hkv, D]`` -> ``o [B, Tq, Hq, D]`` (and ``lse [B, Hq, Tq]``).

    Rows without any visible key produce zeros and ``lse = -inf``.
    """
    B, Tq, Hq, D = q.shape
    Tk, Hkv = k.shape[1], k.shape[2]
    G = Hq // Hkv
    scale = D ** -0.5 if scale is None else scale
    if q_pos is None:
        q_pos = torch.arange(Tk - Tq, Tk, device=q.device).expand(B, Tq)
    if k_pos is None:
        k_pos = torch.arange(Tk, device=q.device).expand(B, Tk)
    qf = q.float().permute(0, 2, 1, 3).reshape(B, Hkv, G, Tq, D)
    kf = k.float().permute(0, 2, 1, 3)
    vf = v.float().permute(0, 2, 1, 3)
    s = torch.einsum("bhgqd,bhkd->bhgqk", qf, kf) * scale
    m = attention_mask(q_pos, k_pos, causal, window, hollow)[:, None, None]
    s = s.masked_fill(~m, float("-inf"))
    lse = torch.logsumexp(s, dim=-1)
    p = torch.exp(s - torch.where(torch.isinf(lse), torch.zeros_like(lse), lse)[..., None])
    p = torch.where(m, p, torch.zeros_like(p))
    o = torch.einsum("bhgqk,bhkd->bhgqd", p, vf).reshape(B, Hq, Tq, -1).permute(0, 2, 1, 3).to(q.dtype)
    if return_lse:
        return o, lse.reshape(B, Hq, Tq)
    return o


def merge_attention_states(o1: Tensor, lse1: Tensor, o2: Tensor, lse2: Tensor) -> Tuple[Tensor, Tensor]:
    """Exact softmax combination of two partial attentions over disjoint key sets.
    ``o [B, T, H, D]``, ``lse [B, H, T]``; ``-inf`` LSE marks an empty set."""
    l1, l2 = lse1.float().transpose(1, 2)[..., None], lse2.float().transpose(1, 2)[..., None]
    m = torch.maximum(l1, l2)
    m = torch.where(torch.isinf(m), torch.zeros_like(m), m)
    w1, w2 = torch.exp(l1 - m), torch.exp(l2 - m)
    den = w1 + w2
    safe = torch.where(den == 0, torch.ones_like(den), den)
    o = (o1.float() * w1 + o2.float() * w2) / safe
    lse = (m + torch.log(safe)).masked_fill(den == 0, float("-inf"))
    return o.to(o1.dtype), lse[..., 0].transpose(1, 2)


def qsparse_attention(q: Tensor, k: Tensor, v: Tensor, q_index: Tensor, *, scale: Optional[float] = None) -> Tensor:
    """Query-sparse causal attention: only rows ``q_index [B, Nq]`` (original positions of the
    compacted queries ``q [B, Nq, Hq, D]``) attend to the full ``k, v``; causality uses the
    original index."""
    B, Tk = k.shape[0], k.shape[1]
    k_pos = torch.arange(Tk, device=q.device).expand(B, Tk)
    return attention(q, k, v, scale=scale, causal=True, q_pos=q_index, k_pos=k_pos)


# ----------------------------------------------------------------------------------------
# Cross entropy over a vocabulary projection (chunked; never materialises [T, V] in fp32 at once)
# ----------------------------------------------------------------------------------------
def linear_cross_entropy(hidden: Tensor, weight: Tensor, labels: Tensor, ignore_index: int = -100,
                         reduction: str = "sum", chunk: int = 4096) -> Tuple[Tensor, Tensor]:
    """``sum/mean CE(hidden @ weight.T, labels)`` and the number of valid labels."""
    h = hidden.reshape(-1, hidden.shape[-1])
    y = labels.reshape(-1)
    total = h.new_zeros((), dtype=torch.float32)
    for s in range(0, h.shape[0], chunk):
        logits = (h[s:s + chunk] @ weight.t()).float()
        total = total + F.cross_entropy(logits, y[s:s + chunk], ignore_index=ignore_index, reduction="sum")
    n = (y != ignore_index).sum()
    if reduction == "mean":
        total = total / n.clamp(min=1)
    return total, n


# ----------------------------------------------------------------------------------------
# Gated delta rule
# ----------------------------------------------------------------------------------------
def _pad_time(x: Tensor, C: int, dim: int = 1) -> Tensor:
    T = x.shape[dim]
    pad = (-T) % C
    if pad == 0:
        return x
    shape = list(x.shape)
    shape[dim] = pad
    return torch.cat([x, x.new_zeros(shape)], dim=dim)


def gated_delta_rule_recurrent(q: Tensor, k: Tensor, v: Tensor, g: Tensor, beta: Tensor, *, scale: Optional[float] = None,
                               initial_state: Optional[Tensor] = None, use_qk_l2norm: bool = True):
    """Token-by-token definition.  ``q,k [B,T,H,Dk]``, ``v [B,T,H,Dv]``, ``g,beta [B,T,H]``.
    ``S_t = a_t S_{t-1} + beta_t k_t (v_t - (a_t S_{t-1})^T k_t)^T``, ``o_t = S_t^T q_t * scale``.
    State ``[B,H,Dk,Dv]`` in fp32.  Returns ``(o, final_state)``."""
    B, T, H, Dk = q.shape
    Dv = v.shape[-1]
    scale = Dk ** -0.5 if scale is None else scale
    if use_qk_l2norm:
        q, k = l2_norm(q.float()), l2_norm(k.float())
    q, k, v, g, beta = q.float(), k.float(), v.float(), g.float(), beta.float()
    S = q.new_zeros(B, H, Dk, Dv) if initial_state is None else initial_state.float()
    outs = []
    for t in range(T):
        S = S * torch.exp(g[:, t])[..., None, None]
        pred = torch.einsum("bhkv,bhk->bhv", S, k[:, t])
        dv = (v[:, t] - pred) * beta[:, t][..., None]
        S = S + torch.einsum("bhk,bhv->bhkv", k[:, t], dv)
        outs.append(torch.einsum("bhkv,bhk->bhv", S, q[:, t]) * scale)
    return torch.stack(outs, dim=1), S


def gated_delta_rule_chunk(q: Tensor, k: Tensor, v: Tensor, g: Tensor, beta: Tensor, *, scale: Optional[float] = None,
                           initial_state: Optional[Tensor] = None, use_qk_l2norm: bool = True, chunk_size: int = 64):
    """Chunk-parallel form of :func:`gated_delta_rule_recurrent` (WY representation):

    per chunk with inclusive cumulative gate ``G``:
      ``A_ij = beta_i (k_i.k_j) e^{G_i-G_j}`` (i>j),  ``Tm = (I + A)^{-1}``
      ``u = Tm (beta v)``,  ``w = Tm (beta e^{G} k)``
      ``v' = u - w S``;  ``o = (q e^{G}) S + ((q k^T) . e^{G_i-G_j} . [i>=j]) v'``
      ``S <- e^{G_last} S + (k e^{G_last-G})^T v'``
    """
    B, T, H, Dk = q.shape
    Dv = v.shape[-1]
    C = chunk_size
    scale = Dk ** -0.5 if scale is None else scale
    if use_qk_l2norm:
        q, k = l2_norm(q.float()), l2_norm(k.float())
    q, k, v, g, beta = (_pad_time(t.float(), C) for t in (q, k, v, g, beta))
    N = q.shape[1] // C
    # [B, H, N, C, D]
    q = q.view(B, N, C, H, Dk).permute(0, 3, 1, 2, 4) * scale
    k = k.view(B, N, C, H, Dk).permute(0, 3, 1, 2, 4)
    v = v.view(B, N, C, H, Dv).permute(0, 3, 1, 2, 4)
    g = g.view(B, N, C, H).permute(0, 3, 1, 2)
    beta = beta.view(B, N, C, H).permute(0, 3, 1, 2)
    G = g.cumsum(-1)
    diff = G[..., :, None] - G[..., None, :]
    idx = torch.arange(C, device=q.device)
    lower = idx[:, None] >= idx[None, :]
    strict = idx[:, None] > idx[None, :]
    decay = torch.where(lower, torch.exp(torch.where(lower, diff, torch.zeros_like(diff))), torch.zeros_like(diff))
    kk = k @ k.transpose(-1, -2)
    A = torch.where(strict, beta[..., None] * kk * decay, torch.zeros_like(kk))
    eye = torch.eye(C, device=q.device, dtype=q.dtype)
    Tm = torch.linalg.solve_triangular(eye + A, eye.expand_as(A), upper=False)
    u = Tm @ (v * beta[..., None])
    w = Tm @ (k * (beta * torch.exp(G))[..., None])
    qk = (q @ k.transpose(-1, -2)) * decay
    qg = q * torch.exp(G)[..., None]
    Glast = G[..., -1]
    kdec = k * torch.exp(Glast[..., None] - G)[..., None]
    S = q.new_zeros(B, H, Dk, Dv) if initial_state is None else initial_state.float()
    outs = []
    for n in range(N):
        v_new = u[:, :, n] - w[:, :, n] @ S
        outs.append(qg[:, :, n] @ S + qk[:, :, n] @ v_new)
        S = S * torch.exp(Glast[:, :, n])[..., None, None] + kdec[:, :, n].transpose(-1, -2) @ v_new
    o = torch.stack(outs, dim=2)  # [B,H,N,C,Dv]
    o = o.permute(0, 2, 3, 1, 4).reshape(B, N * C, H, Dv)[:, :T]
    return o, S


# ----------------------------------------------------------------------------------------
# Simple gated linear attention (scalar decay per head)
# ----------------------------------------------------------------------------------------
def simple_gla_recurrent(q: Tensor, k: Tensor, v: Tensor, g: Tensor, *, scale: Optional[float] = None,
                         initial_state: Optional[Tensor] = None):
    """``S_t = e^{g_t} S_{t-1} + k_t v_t^T``, ``o_t = S_t^T q_t * scale``."""
    B, T, H, Dk = q.shape
    scale = Dk ** -0.5 if scale is None else scale
    q, k, v, g = q.float(), k.float(), v.float(), g.float()
    S = q.new_zeros(B, H, Dk, v.shape[-1]) if initial_state is None else initial_state.float()
    outs = []
    for t in range(T):
        S = S * torch.exp(g[:, t])[..., None, None] + torch.einsum("bhk,bhv->bhkv", k[:, t], v[:, t])
        outs.append(torch.einsum("bhkv,bhk->bhv", S, q[:, t]) * scale)
    return torch.stack(outs, dim=1), S


def simple_gla_chunk(q: Tensor, k: Tensor, v: Tensor, g: Tensor, *, scale: Optional[float] = None,
                     initial_state: Optional[Tensor] = None, chunk_size: int = 64):
    B, T, H, Dk = q.shape
    Dv = v.shape[-1]
    C = chunk_size
    scale = Dk ** -0.5 if scale is None else scale
    q, k, v, g = (_pad_time(t.float(), C) for t in (q, k, v, g))
    N = q.shape[1] // C
    q = q.view(B, N, C, H, Dk).permute(0, 3, 1, 2, 4) * scale
    k = k.view(B, N, C, H, Dk).permute(0, 3, 1, 2, 4)
    v = v.view(B, N, C, H, Dv).permute(0, 3, 1, 2, 4)
    g = g.view(B, N, C, H).permute(0, 3, 1, 2)
    G = g.cumsum(-1)
    diff = G[..., :, None] - G[..., None, :]
    idx = torch.arange(C, device=q.device)
    lower = idx[:, None] >= idx[None, :]
    decay = torch.where(lower, torch.exp(torch.where(lower, diff, torch.zeros_like(diff))), torch.zeros_like(diff))
    qk = (q @ k.transpose(-1, -2)) * decay
    qg = q * torch.exp(G)[..., None]
    Glast = G[..., -1]
    kdec = k * torch.exp(Glast[..., None] - G)[..., None]
    S = q.new_zeros(B, H, Dk, Dv) if initial_state is None else initial_state.float()
    outs = []
    for n in range(N):
        outs.append(qg[:, :, n] @ S + qk[:, :, n] @ v[:, :, n])
        S = S * torch.exp(Glast[:, :, n])[..., None, None] + kdec[:, :, n].transpose(-1, -2) @ v[:, :, n]
    o = torch.stack(outs, dim=2).permute(0, 2, 3, 1, 4).reshape(B, N * C, H, Dv)[:, :T]
    return o, S


# ----------------------------------------------------------------------------------------
# Gated KalmaNet: Chebyshev solve of (H_t + lambda_t I) x_t = q_t
# ----------------------------------------------------------------------------------------
def _chebyshev_rows(Hx, q: Tensor, fro: Tensor, ridge_ratio: float, num_iter: int) -> Tensor:
    """Shared iteration.  ``Hx(x)`` applies the per-row operator ``H_t`` to each row of ``x``.
    ``q [..., C, D]``, ``fro [..., C, 1]``."""
    lam = ridge_ratio * fro
    denom = 2 * lam + fro
    denom = torch.where(denom == 0, torch.ones_like(denom), denom)
    step = 2.0 / denom
    c = (fro / denom / 2.0) ** 2
    x_prev = torch.zeros_like(q)
    x = step * q
    omega = torch.full_like(fro, 2.0)
    for _ in range(num_iter):
        omega = 1.0 / (1.0 - c * omega)
        upd = step * omega * (Hx(x) + lam * x - q) + (omega - 1.0) * x_prev
        x_prev = x
        x = omega * x - upd
    return x


def gka_chebyshev_recurrent(q: Tensor, k: Tensor, gk: Optional[Tensor], *, ridge_ratio: float = 0.02, num_iter: int = 30,
                            initial_state: Optional[Tensor] = None):
    """Token-by-token definition: ``H_t = e^{gk_t} H_{t-1} + k_t k_t^T``, ``f_t = ||H_t||_F``,
    ``lambda_t = ridge_ratio f_t`` and ``num_iter`` Chebyshev steps on ``(H_t + lambda_t I) x = q_t``.
    Returns ``(x [B,T,H,D], H_T [B,H,D,D])``."""
    B, T, Hh, D = q.shape
    q, k = q.float(), k.float()
    Hs = q.new_zeros(B, Hh, D, D) if initial_state is None else initial_state.float()
    outs = []
    for t in range(T):
        if gk is not None:
            Hs = Hs * torch.exp(gk[:, t].float())[..., None, None]
        Hs = Hs + torch.einsum("bhi,bhj->bhij", k[:, t], k[:, t])
        fro = Hs.pow(2).sum((-1, -2)).sqrt()[..., None, None]  # [B,H,1,1]
        qt = q[:, t][..., None, :]  # [B,H,1,D]
        x = _chebyshev_rows(lambda xx: xx @ Hs, qt, fro, ridge_ratio, num_iter)
        outs.append(x[..., 0, :])
    return torch.stack(outs, dim=1), Hs


def gka_chebyshev_chunk(q: Tensor, k: Tensor, gk: Optional[Tensor], *, ridge_ratio: float = 0.02, num_iter: int = 30,
                        initial_state: Optional[Tensor] = None, chunk_size: int = 64):
    """Chunk-parallel form.  Inside a chunk with inclusive cumulative gate ``G`` and start
    state ``H0`` the row operator is ``x_i -> (x_i e^{G_i}) H0 + sum_{j<=i} (x_i.k_j) e^{G_i-G_j} k_j``
    and ``||H_i||_F^2`` expands into three closed-form terms (state, cross, Gram)."""
    B, T, Hh, D = q.shape
    C = chunk_size
    q, k = _pad_time(q.float(), C), _pad_time(k.float(), C)
    gkf = torch.zeros(B, q.shape[1], Hh, device=q.device) if gk is None else _pad_time(gk.float(), C)
    N = q.shape[1] // C
    q = q.view(B, N, C, Hh, D).permute(0, 3, 1, 2, 4)
    k = k.view(B, N, C, Hh, D).permute(0, 3, 1, 2, 4)
    g = gkf.view(B, N, C, Hh).permute(0, 3, 1, 2)
    G = g.cumsum(-1)
    idx = torch.arange(C, device=q.device)
    lower = idx[:, None] >= idx[None, :]
    diff = G[..., :, None] - G[..., None, :]
    mask = torch.where(lower, torch.exp(torch.where(lower, diff, torch.zeros_like(diff))), torch.zeros_like(diff))
    Hs = q.new_zeros(B, Hh, D, D) if initial_state is None else initial_state.float()
    outs = []
    for n in range(N):
        kn, qn, Gn, mn = k[:, :, n], q[:, :, n], G[:, :, n], mask[:, :, n]
        eg = torch.exp(Gn)[..., None]  # [B,H,C,1]
        gram = kn @ kn.transpose(-1, -2)
        fro2 = ((mn @ (gram * gram)) * mn).sum(-1, keepdim=True)
        fro2 = fro2 + eg * eg * Hs.pow(2).sum((-1, -2))[..., None, None]
        kHk = (kn * (kn @ Hs)).sum(-1)  # [B,H,C]
        fro2 = fro2 + 2 * eg * (mn * kHk[..., None, :]).sum(-1, keepdim=True)
        fro = fro2.clamp(min=0).sqrt()

        def Hx(x, Hs=Hs, kn=kn, mn=mn, eg=eg):
            return (x * eg) @ Hs + ((x @ kn.transpose(-1, -2)) * mn) @ kn

        outs.append(_chebyshev_rows(Hx, qn, fro, ridge_ratio, num_iter))
        Glast = Gn[..., -1]
        kdec = kn * torch.exp(Glast[..., None] - Gn)[..., None]
        Hs = Hs * torch.exp(Glast)[..., None, None] + kdec.transpose(-1, -2) @ kn
    x = torch.stack(outs, dim=2).permute(0, 2, 3, 1, 4).reshape(B, N * C, Hh, D)[:, :T]
    return x, Hs


def gka_forward(q: Tensor, k: Tensor, v: Tensor, alpha: Optional[Tensor], g: Tensor, gk: Optional[Tensor], *,
                scale: Optional[float] = None, ridge_ratio: float = 0.02, num_iter: int = 30,
                initial_state: Optional[Tuple[Optional[Tensor], Optional[Tensor]]] = None, chunk_size: int = 64,
                recurrent: bool = False):
    """Full GKA mixer core: solve, ``q' = q + alpha (x - q)``, then simple GLA with ``q'``.
    ``initial_state = (h_kk, h_kv)``.  Returns ``(o, (h_kk_T, h_kv_T))``."""
    h_kk0, h_kv0 = (None, None) if initial_state is None else initial_state
    qf = q.float()
    h_kk = None
    if num_iter > 0:
        solver = gka_chebyshev_recurrent if recurrent else gka_chebyshev_chunk
        kwargs = {} if recurrent else {"chunk_size": chunk_size}
        x, h_kk = solver(q, k, gk, ridge_ratio=ridge_ratio, num_iter=num_iter, initial_state=h_kk0, **kwargs)
        if alpha is not None:
            qf = qf + alpha.float()[..., None] * (x - qf)
        else:
            qf = x
    gla = simple_gla_recurrent if recurrent else simple_gla_chunk
    kwargs = {} if recurrent else {"chunk_size": chunk_size}
    o, h_kv = gla(qf, k, v, g, scale=scale, initial_state=h_kv0, **kwargs)
    return o, (h_kk, h_kv)


# ----------------------------------------------------------------------------------------
# Mamba2 SSD
# ----------------------------------------------------------------------------------------
def ssd_recurrent(x: Tensor, dt: Tensor, A: Tensor, Bm: Tensor, Cm: Tensor, D: Optional[Tensor] = None, *,
                  initial_state: Optional[Tensor] = None):
    """``x [B,T,H,P]``, ``dt [B,T,H]`` (already softplus'ed), ``A [H]`` (negative),
    ``Bm, Cm [B,T,G,N]`` (heads share groups).  ``h_t = e^{dt A} h_{t-1} + dt x_t B_t^T``,
    ``y_t = h_t C_t + D x_t``.  State ``[B,H,P,N]``.  Returns ``(y, h_T)``."""
    Bsz, T, H, P = x.shape
    Gr, N = Bm.shape[2], Bm.shape[3]
    rep = H // Gr
    x, dt, Bm, Cm = x.float(), dt.float(), Bm.float(), Cm.float()
    Bh = Bm.repeat_interleave(rep, dim=2)
    Ch = Cm.repeat_interleave(rep, dim=2)
    h = x.new_zeros(Bsz, H, P, N) if initial_state is None else initial_state.float()
    ys = []
    for t in range(T):
        a = torch.exp(dt[:, t] * A.float())[..., None, None]
        h = h * a + torch.einsum("bhp,bhn->bhpn", x[:, t] * dt[:, t][..., None], Bh[:, t])
        y = torch.einsum("bhpn,bhn->bhp", h, Ch[:, t])
        if D is not None:
            y = y + D.float()[None, :, None] * x[:, t]
        ys.append(y)
    return torch.stack(ys, dim=1), h


def ssd_chunk(x: Tensor, dt: Tensor, A: Tensor, Bm: Tensor, Cm: Tensor, D: Optional[Tensor] = None, *,
              initial_state: Optional[Tensor] = None, chunk_size: int = 256):
    """Chunked SSD: identical to simple GLA with ``q=C``, ``k=B``, ``v=dt*x``, ``g=dt*A`` and a
    transposed state (``[P,N]`` instead of ``[N,P]``)."""
    Bsz, T, H, P = x.shape
    Gr = Bm.shape[2]
    rep = H // Gr
    g = dt.float() * A.float()
    v = x.float() * dt.float()[..., None]
    kq = Bm.float().repeat_interleave(rep, dim=2)
    qq = Cm.float().repeat_interleave(rep, dim=2)
    h0 = None if initial_state is None else initial_state.float().transpose(-1, -2)
    y, hT = simple_gla_chunk(qq, kq, v, g, scale=1.0, initial_state=h0, chunk_size=chunk_size)
    if D is not None:
        y = y + D.float()[None, None, :, None] * x.float()
    return y, hT.transpose(-1, -2)


def selective_state_update(state: Tensor, x: Tensor, dt: Tensor, A: Tensor, Bm: Tensor, Cm: Tensor,
                           D: Optional[Tensor] = None) -> Tuple[Tensor, Tensor]:
    """Decode step of SSD: ``state [B,H,P,N]``, ``x [B,H,P]``, ``dt [B,H]``, ``Bm,Cm [B,G,N]``."""
    y, h = ssd_recurrent(x[:, None], dt[:, None], A, Bm[:, None], Cm[:, None], D, initial_state=state)
    return y[:, 0], h


# ----------------------------------------------------------------------------------------
# MoE
# ----------------------------------------------------------------------------------------
def moe_router(logits: Tensor, top_k: int, norm_topk_prob: bool = True) -> Tuple[Tensor, Tensor]:
    """Softmax over experts, top-k, optional renormalisation.  Returns ``(weights, indices)``."""
    probs = torch.softmax(logits.float(), dim=-1)
    w, idx = torch.topk(probs, top_k, dim=-1)
    if norm_topk_prob:
        w = w / w.sum(-1, keepdim=True)
    return w, idx


def moe_experts(x: Tensor, w_gate_up: Tensor, w_down: Tensor, weights: Tensor, indices: Tensor) -> Tensor:
    """``x [T, Dm]``; ``w_gate_up [E, 2F, Dm]``; ``w_down [E, Dm, F]``; top-k routing ``[T, k]``."""
    T, Dm = x.shape
    E = w_gate_up.shape[0]
    out = torch.zeros(T, Dm, dtype=torch.float32, device=x.device)
    flat_idx = indices.reshape(-1)
    token_of = torch.arange(T, device=x.device).repeat_interleave(indices.shape[1])
    for e in torch.unique(flat_idx).tolist():
        sel = flat_idx == e
        tok = token_of[sel]
        h = x[tok].float() @ w_gate_up[e].float().t()
        gate, up = h.chunk(2, dim=-1)
        y = (F.silu(gate) * up) @ w_down[e].float().t()
        out.index_add_(0, tok, y * weights.reshape(-1)[sel][:, None].float())
    return out.to(x.dtype)
