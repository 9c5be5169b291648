"""Bindings of the sm_100a kernels as autograd functions.

Each public function mirrors the function of the same name in ``ops/reference.py``; inputs
are bf16 CUDA tensors (fp32 where the contract says so).  Tensors of another dtype are
evaluated with the reference formulas on the GPU (an explicit numerics-debugging path: the
training and serving paths are bf16).
"""
from __future__ import annotations

import ctypes
import os
from typing import Optional, Tuple

import torch

from . import _lib
from . import reference as R

Tensor = torch.Tensor
c_int, c_ll, c_float = ctypes.c_int, ctypes.c_longlong, ctypes.c_float
BF16 = torch.bfloat16


def _K():
    return _lib.kernels()


def _is_bf16(*ts) -> bool:
    for t in ts:
        if t is not None and t.dtype != BF16:
            return False
    return True


class _NoCtx:
    """Stand-in for the autograd context when no graph is recorded (inference): the op's ``forward`` runs directly,
    without the dispatch cost of ``Function.apply`` (a prefill pass of a 36-layer model calls ~300 of these)."""
    needs_input_grad = (False,) * 16

    def save_for_backward(self, *tensors):
        pass

    def set_materialize_grads(self, value):
        pass

    def mark_non_differentiable(self, *tensors):
        pass


def _apply(fn, *args):
    if torch.is_grad_enabled():
        return fn.apply(*args)
    return fn.forward(_NoCtx(), *args)


def _st(t: Tensor):
    return _lib.stream_ptr(t.device)


# ----------------------------------------------------------------------------------------
# RMSNorm
# ----------------------------------------------------------------------------------------
class _RMSNorm(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, eps, zero_centered):
        shape = x.shape
        D = shape[-1]
        x2 = x.reshape(-1, D).contiguous()
        N = x2.shape[0]
        y = torch.empty_like(x2)
        rstd = torch.empty(N, device=x.device, dtype=torch.float32)
        w = None if weight is None else weight.contiguous()
        _lib.check(_K().hmf_rms_norm_fwd(_lib.ptr(x2), None, _lib.ptr(w), _lib.ptr(y), None, _lib.ptr(rstd), c_ll(N),
                                         c_int(D), c_float(eps), c_int(int(zero_centered)), _st(x)), "rms_norm_fwd")
        ctx.save_for_backward(x2, w, rstd)
        ctx.zero_centered, ctx.shape = zero_centered, shape
        return y.view(shape)

    @staticmethod
    def backward(ctx, dy):
        x2, w, rstd = ctx.saved_tensors
        N, D = x2.shape
        dy2 = dy.reshape(-1, D).contiguous()
        dx = torch.empty_like(x2)
        dw = None
        part = None
        if w is not None and ctx.needs_input_grad[1]:
            nb = _K().hmf_rms_norm_bwd_blocks(c_ll(N))
            part = torch.empty(nb, D, device=x2.device, dtype=torch.float32)
            dw = torch.empty(D, device=x2.device, dtype=BF16)
        _lib.check(_K().hmf_rms_norm_bwd(_lib.ptr(x2), _lib.ptr(w), _lib.ptr(dy2), _lib.ptr(rstd), _lib.ptr(dx),
                                         _lib.ptr(part), _lib.ptr(dw), c_int(1), c_ll(N), c_int(D),
                                         c_int(int(ctx.zero_centered)), _st(x2)), "rms_norm_bwd")
        return dx.view(ctx.shape), dw, None, None


def rms_norm(x: Tensor, weight: Optional[Tensor], eps: float, zero_centered: bool = False) -> Tensor:
    if not _is_bf16(x, weight) or x.shape[-1] % 8 != 0:
        return R.rms_norm(x, weight, eps, zero_centered)
    return _apply(_RMSNorm, x, weight, eps, zero_centered)


def fused_add_rms_norm(x: Tensor, residual: Tensor, weight: Tensor, eps: float) -> Tuple[Tensor, Tensor]:
    """Inference-path fusion (no autograd): residual add + norm in one pass."""
    if not _is_bf16(x, residual, weight) or torch.is_grad_enabled() and (x.requires_grad or residual.requires_grad):
        return R.fused_add_rms_norm(x, residual, weight, eps)
    D = x.shape[-1]
    x2, r2 = x.reshape(-1, D).contiguous(), residual.reshape(-1, D).contiguous()
    y, r_out = torch.empty_like(x2), torch.empty_like(x2)
    weight = weight.contiguous()
    _lib.check(_K().hmf_rms_norm_fwd(_lib.ptr(x2), _lib.ptr(r2), _lib.ptr(weight), _lib.ptr(y),
                                     _lib.ptr(r_out), None, c_ll(x2.shape[0]), c_int(D), c_float(eps), c_int(0), _st(x)),
               "fused_add_rms_norm")
    return y.view(x.shape), r_out.view(x.shape)


# ----------------------------------------------------------------------------------------
# gated RMSNorm over the head dimension
# ----------------------------------------------------------------------------------------
class _GatedNorm(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, gate, weight, eps, mode):
        shape = x.shape
        D = shape[-1]
        x2, g2 = _lib.aligned(x.reshape(-1, D)), _lib.aligned(gate.reshape(-1, D))
        w = weight.contiguous()
        w_rows = 1 if w.dim() == 1 else w.shape[0]
        N = x2.shape[0]
        y = torch.empty_like(x2)
        rstd = torch.empty(N, device=x.device, dtype=torch.float32)
        _lib.check(_K().hmf_gated_norm_fwd(_lib.ptr(x2), _lib.ptr(g2), _lib.ptr(w), _lib.ptr(y), _lib.ptr(rstd), c_ll(N),
                                           c_int(D), c_int(w_rows), c_float(eps), c_int(mode), _st(x)), "gated_norm_fwd")
        ctx.save_for_backward(x2, g2, w, rstd)
        ctx.mode, ctx.shape, ctx.w_rows, ctx.gshape = mode, shape, w_rows, gate.shape
        return y.view(shape)

    @staticmethod
    def backward(ctx, dy):
        x2, g2, w, rstd = ctx.saved_tensors
        N, D = x2.shape
        dy2 = dy.reshape(-1, D).contiguous()
        dx, dg = torch.empty_like(x2), torch.empty_like(g2)
        dw = torch.zeros(w.shape, device=x2.device, dtype=torch.float32)
        _lib.check(_K().hmf_gated_norm_bwd(_lib.ptr(x2), _lib.ptr(g2), _lib.ptr(w), _lib.ptr(dy2), _lib.ptr(rstd),
                                           _lib.ptr(dx), _lib.ptr(dg), _lib.ptr(dw), c_ll(N), c_int(D),
                                           c_int(ctx.w_rows), c_int(ctx.mode), _st(x2)), "gated_norm_bwd")
        return dx.view(ctx.shape), dg.view(ctx.gshape), dw.to(w.dtype), None, None


def gated_rms_norm(x: Tensor, gate: Tensor, weight: Tensor, eps: float, norm_before_gate: bool = True) -> Tensor:
    D = x.shape[-1]
    if not _is_bf16(x, gate, weight) or D not in (64, 128, 256):
        return R.gated_rms_norm(x, gate, weight, eps, norm_before_gate)
    if weight.dim() == 2:
        # per-head weights [H, D]: rows are (token, head) pairs with the head fastest
        assert x.shape[-2] == weight.shape[0], "per-head weight needs x[..., H, D]"
    return _apply(_GatedNorm, x, gate, weight, eps, 0 if norm_before_gate else 1)


# ----------------------------------------------------------------------------------------
# SwiGLU
# ----------------------------------------------------------------------------------------
class _SwiGLU(torch.autograd.Function):
    @staticmethod
    def forward(ctx, g, u):
        g, u = g.contiguous(), u.contiguous()
        y = torch.empty_like(g)
        _lib.check(_K().hmf_swiglu_fwd(_lib.ptr(g), _lib.ptr(u), _lib.ptr(y), c_ll(g.numel()), _st(g)), "swiglu_fwd")
        ctx.save_for_backward(g, u)
        return y

    @staticmethod
    def backward(ctx, dy):
        g, u = ctx.saved_tensors
        dy = dy.contiguous()
        dg, du = torch.empty_like(g), torch.empty_like(u)
        _lib.check(_K().hmf_swiglu_bwd(_lib.ptr(g), _lib.ptr(u), _lib.ptr(dy), _lib.ptr(dg), _lib.ptr(du),
                                       c_ll(g.numel()), _st(g)), "swiglu_bwd")
        return dg, du


def swiglu_backward(gate: Tensor, up: Tensor, dy: Tensor) -> Tuple[Tensor, Tensor]:
    """Gradients of ``silu(gate) * up`` with respect to ``gate`` and ``up`` (bf16, one kernel)."""
    g, u, dy = gate.contiguous(), up.contiguous(), dy.contiguous()
    dg, du = torch.empty_like(g), torch.empty_like(u)
    _lib.check(_K().hmf_swiglu_bwd(_lib.ptr(g), _lib.ptr(u), _lib.ptr(dy), _lib.ptr(dg), _lib.ptr(du),
                                   c_ll(g.numel()), _st(g)), "swiglu_bwd")
    return dg, du


def swiglu(gate: Tensor, up: Tensor) -> Tensor:
    if not _is_bf16(gate, up) or gate.numel() % 8 != 0:
        return R.swiglu(gate, up)
    return _apply(_SwiGLU, gate, up)


# ----------------------------------------------------------------------------------------
# RoPE
# ----------------------------------------------------------------------------------------
def _rope_launch(x: Tensor, cos: Tensor, sin: Tensor, backward: bool) -> Tensor:
    B, T, H, D = x.shape
    R_ = cos.shape[-1]
    if x.stride(-1) != 1 or x.stride(2) != D or x.stride(0) != T * x.stride(1):
        x = x.contiguous()
    y = torch.empty(B, T, H, D, device=x.device, dtype=x.dtype)
    _lib.check(_K().hmf_rope(_lib.ptr(x), _lib.ptr(cos), _lib.ptr(sin), _lib.ptr(y), c_ll(B * T), c_int(H), c_int(D),
                             c_int(R_), c_int(int(backward)), c_ll(x.stride(1)), _st(x)), "rope")
    return y


class _RoPE(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, cos, sin):
        cos2 = cos.expand(x.shape[0], x.shape[1], cos.shape[-1]).to(BF16).contiguous()
        sin2 = sin.expand(x.shape[0], x.shape[1], sin.shape[-1]).to(BF16).contiguous()
        ctx.save_for_backward(cos2, sin2)
        return _rope_launch(x, cos2, sin2, False)

    @staticmethod
    def backward(ctx, dy):
        cos2, sin2 = ctx.saved_tensors
        return _rope_launch(dy, cos2, sin2, True), None, None


def apply_rope(x: Tensor, cos: Tensor, sin: Tensor) -> Tensor:
    Rr = cos.shape[-1]
    if not _is_bf16(x) or Rr % 16 != 0 or x.shape[-1] % 8 != 0 or (x.data_ptr() % 16) != 0:
        return R.apply_rope(x, cos, sin)
    return _apply(_RoPE, x, cos, sin)


def rope_tables_bf16(position_embeddings, lead_shape):
    """``(cos, sin)`` as contiguous bf16 ``[rows, rot]`` tables for ``rows = prod(lead_shape)`` tokens; converted once
    per forward pass (the result is cached on the ``cos`` tensor, which every layer of the pass receives)."""
    cos, sin = position_embeddings
    rows = 1
    for d in lead_shape:
        rows *= int(d)
    cached = getattr(cos, "_hmf_bf16_tables", None)
    if cached is not None and cached[0].shape[0] == rows:
        return cached
    rot = cos.shape[-1]
    cs = cos.expand(*lead_shape, rot).to(BF16).reshape(rows, rot).contiguous()
    sn = sin.expand(*lead_shape, rot).to(BF16).reshape(rows, rot).contiguous()
    cos._hmf_bf16_tables = (cs, sn)
    return cs, sn


def heads_norm_rope_ok(x: Tensor, head_dim: int, position_embeddings) -> bool:
    """The fused inference kernel applies: no autograd graph, bf16 on the GPU, heads of 128 channels, even rotary
    width."""
    if torch.is_grad_enabled() or not x.is_cuda or x.dtype != BF16 or head_dim != 128 or x.stride(-1) != 1:
        return False
    if position_embeddings is not None and position_embeddings[0].shape[-1] % 2 != 0:
        return False
    return _lib.use_cuda_kernels(x)


def heads_norm_rope(x: Tensor, n_plain: int, n_b: int, n_c: int, wb: Optional[Tensor], wc: Optional[Tensor], eps: float,
                    zero_centered: bool, position_embeddings) -> Tensor:
    """``x [..., (n_plain + n_b + n_c) * 128]`` (the last dimension may be a column slice of a wider tensor): the first
    ``n_plain`` heads are copied, the next ``n_b`` / ``n_c`` heads get RMSNorm with ``wb`` / ``wc`` (or none) and the
    rotary embedding; returns a contiguous tensor of the same shape.  One launch instead of split, two norms, two
    rotations and a concatenation (``csrc/kernels/decode_fused.cu::heads_norm_rope_kernel``)."""
    lead, cols = x.shape[:-1], x.shape[-1]
    assert cols == (n_plain + n_b + n_c) * 128
    rows = 1
    for d in lead:
        rows *= int(d)
    x2 = x.reshape(rows, cols)
    if x2.stride(1) != 1 or x2.stride(0) % 8 != 0:
        x2 = x2.contiguous()
    out = torch.empty(rows, cols, device=x.device, dtype=BF16)
    cs = sn = None
    rot = 0
    if position_embeddings is not None:
        cs, sn = rope_tables_bf16(position_embeddings, lead)
        rot = cs.shape[-1]
    if wb is not None and wc is None:
        wc = wb
    if wc is not None and wb is None:
        wb = wc
    _lib.check(_K().hmf_heads_norm_rope(_lib.ptr(x2), c_ll(x2.stride(0)), _lib.ptr(out), c_ll(cols), c_int(n_plain),
                                        c_int(n_b), c_int(n_c), _lib.ptr(wb), _lib.ptr(wc), c_float(eps),
                                        c_int(int(zero_centered)), _lib.ptr(cs), _lib.ptr(sn), c_int(rot), c_int(rows),
                                        _st(x)), "heads_norm_rope")
    return out.view(*lead, cols)


# ----------------------------------------------------------------------------------------
# gating (tiny [T, H] tensors: plain PyTorch elementwise math)
# ----------------------------------------------------------------------------------------
class _GKAPrepare(torch.autograd.Function):
    """q / k normalisation and beta scaling of Gated KalmaNet in one kernel each way (``csrc/kernels/gka_prep.cu``)."""

    @staticmethod
    def forward(ctx, q, k, v, beta, eps):
        D = q.shape[-1]
        q2, k2, v2 = (_lib.aligned(t.reshape(-1, D)) for t in (q, k, v))
        N = q2.shape[0]
        bt = None if beta is None else beta.reshape(-1).float().contiguous()
        qn, kn, vn = (torch.empty(N, D, device=q.device, dtype=BF16) for _ in range(3))
        nq = torch.empty(N, device=q.device, dtype=torch.float32)
        nk = torch.empty_like(nq)
        _lib.check(_K().hmf_gka_prep_fwd(_lib.ptr(q2), _lib.ptr(k2), _lib.ptr(v2), _lib.ptr(bt), _lib.ptr(qn), _lib.ptr(kn),
                                         _lib.ptr(vn), _lib.ptr(nq), _lib.ptr(nk), c_ll(N), c_int(D), c_ll(q2.stride(0)),
                                         c_ll(k2.stride(0)), c_ll(v2.stride(0)), c_float(eps), _st(q)), "gka_prep_fwd")
        ctx.save_for_backward(q2, k2, v2, bt, nq, nk)
        ctx.eps, ctx.shapes, ctx.beta_meta = eps, (q.shape, k.shape, v.shape), None if beta is None else (beta.shape, beta.dtype)
        return qn.view(q.shape), kn.view(k.shape), vn.view(v.shape)

    @staticmethod
    def backward(ctx, gq, gk, gv):
        q2, k2, v2, bt, nq, nk = ctx.saved_tensors
        N, D = q2.shape
        gq2, gk2, gv2 = (_lib.aligned(g.reshape(-1, D).to(BF16)) for g in (gq, gk, gv))
        dq, dk, dv = (torch.empty(N, D, device=q2.device, dtype=BF16) for _ in range(3))
        dbeta = torch.empty(N, device=q2.device, dtype=torch.float32) if bt is not None else None
        _lib.check(_K().hmf_gka_prep_bwd(_lib.ptr(q2), _lib.ptr(k2), _lib.ptr(v2), _lib.ptr(bt), _lib.ptr(nq), _lib.ptr(nk),
                                         _lib.ptr(gq2), _lib.ptr(gk2), _lib.ptr(gv2), _lib.ptr(dq), _lib.ptr(dk),
                                         _lib.ptr(dv), _lib.ptr(dbeta), c_ll(N), c_int(D), c_ll(q2.stride(0)),
                                         c_ll(k2.stride(0)), c_ll(v2.stride(0)), c_float(ctx.eps), _st(q2)),
                   "gka_prep_bwd")
        sq, sk, sv = ctx.shapes
        db = None
        if ctx.beta_meta is not None:
            db = dbeta.view(ctx.beta_meta[0]).to(ctx.beta_meta[1])
        return dq.view(sq), dk.view(sk), dv.view(sv), db, None


def gka_prepare(q, k, v, beta=None, eps=1e-6):
    """``(q / (|q| + eps), (beta + eps) k / (|k| + eps), (beta + eps) v)``; bf16 CUDA tensors with a head dimension that
    is a multiple of 8 up to 256 take the fused kernels, everything else the PyTorch formulation."""
    D = q.shape[-1]
    if not (_is_bf16(q, k, v) and D % 8 == 0 and D <= 256 and q.shape == k.shape == v.shape):
        return R.gka_prepare(q, k, v, beta, eps)
    return _apply(_GKAPrepare, q, k, v, beta, eps)


def gdn_gating(a, b, A_log, dt_bias, beta_scale=1.0):
    return R.gdn_gating(a, b, A_log, dt_bias, beta_scale)


# ----------------------------------------------------------------------------------------
# causal conv1d
# ----------------------------------------------------------------------------------------
class _Conv1d(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, bias, init, act, want_state):
        B, T, C = x.shape
        x = x.contiguous()
        w = weight.contiguous()
        K = w.shape[-1]
        init_c = None if init is None else init.to(BF16).contiguous()
        y = torch.empty_like(x)
        final = torch.empty(B, K - 1, C, device=x.device, dtype=x.dtype) if want_state else None
        _lib.check(_K().hmf_conv1d_fwd(_lib.ptr(x), _lib.ptr(w), _lib.ptr(bias), _lib.ptr(init_c), _lib.ptr(y),
                                       _lib.ptr(final), c_int(B), c_int(T), c_int(C), c_int(K), c_int(act), _st(x)),
                   "conv1d_fwd")
        ctx.save_for_backward(x, w, bias, init_c)
        ctx.act = act
        ctx.has_init = init is not None
        if want_state:
            ctx.mark_non_differentiable(final)
            return y, final
        return y, None

    @staticmethod
    def backward(ctx, dy, _dfinal):
        x, w, bias, init_c = ctx.saved_tensors
        B, T, C = x.shape
        K = w.shape[-1]
        dy = dy.contiguous()
        dx = torch.empty_like(x)
        dw = torch.zeros(C, K, device=x.device, dtype=torch.float32)
        db = torch.zeros(C, device=x.device, dtype=torch.float32) if bias is not None else None
        dinit = torch.empty(B, K - 1, C, device=x.device, dtype=torch.float32) if ctx.has_init else None
        _lib.check(_K().hmf_conv1d_bwd(_lib.ptr(x), _lib.ptr(w), _lib.ptr(bias), _lib.ptr(init_c), _lib.ptr(dy),
                                       _lib.ptr(dx), _lib.ptr(dinit), _lib.ptr(dw), _lib.ptr(db), c_int(B), c_int(T),
                                       c_int(C), c_int(K), c_int(ctx.act), _st(x)), "conv1d_bwd")
        return (dx, dw.to(w.dtype), None if db is None else db.to(bias.dtype),
                None if dinit is None else dinit.to(x.dtype), None, None)


def causal_conv1d(x, weight, bias=None, activation="silu", initial_state=None, return_final_state=False):
    if not _is_bf16(x, weight, bias) or weight.shape[-1] != 4 or x.shape[-1] % 8 != 0:
        return R.causal_conv1d(x, weight, bias, activation, initial_state, return_final_state)
    act = 1 if activation in ("silu", "swish") else 0
    y, final = _apply(_Conv1d, x, weight, bias, initial_state, act, return_final_state)
    return (y, final) if return_final_state else y


def causal_conv1d_update(x, conv_state, weight, bias=None, activation="silu", slots: Optional[Tensor] = None):
    """Decode step; ``conv_state`` is updated in place (and returned)."""
    if not _is_bf16(x, weight, bias, conv_state) or weight.shape[-1] != 4 or x.shape[-1] % 8 != 0:
        return R.causal_conv1d_update(x, conv_state, weight, bias, activation)
    B, C = x.shape
    y = torch.empty_like(x)
    state = conv_state if conv_state.is_contiguous() else conv_state.contiguous()
    x, weight = x.contiguous(), weight.contiguous()
    _lib.check(_K().hmf_conv1d_update(_lib.ptr(x), _lib.ptr(state), _lib.ptr(weight),
                                      _lib.ptr(bias), _lib.ptr(y), _lib.ptr(slots), c_int(B), c_int(C), c_int(4),
                                      c_int(1 if activation in ("silu", "swish") else 0), _st(x)), "conv1d_update")
    return y, state


# ----------------------------------------------------------------------------------------
# fused linear + cross entropy
# ----------------------------------------------------------------------------------------
class _LinearCE(torch.autograd.Function):
    """Forward computes the loss *and* the gradients chunk by chunk (logits of one chunk live at a
    time, in bf16); backward only rescales by the incoming gradient."""

    @staticmethod
    def forward(ctx, hidden, weight, labels, ignore_index, chunk):
        from .gemm import gemm
        N, Dm = hidden.shape
        V = weight.shape[0]
        hidden = hidden.contiguous()
        labels = labels.contiguous().to(torch.int64)
        loss = torch.zeros(1, device=hidden.device, dtype=torch.float32)
        nvalid = torch.zeros(1, device=hidden.device, dtype=torch.int32)
        need_dh = ctx.needs_input_grad[0]
        need_dw = ctx.needs_input_grad[1]
        dh = torch.empty_like(hidden) if need_dh else None
        dw = torch.zeros(V, Dm, device=hidden.device, dtype=torch.float32) if need_dw else None
        Vp = (V + 7) // 8 * 8
        buf = torch.empty(min(chunk, N), Vp, device=hidden.device, dtype=BF16)
        for s in range(0, N, chunk):
            n = min(chunk, N - s)
            h = hidden[s:s + n]
            logits = buf[:n, :V]
            own = V % 8 == 0 and Dm % 8 == 0 and n >= 128 and weight.is_contiguous()
            if own:
                gemm(h, weight, out=logits)
            else:
                torch.matmul(h, weight.t(), out=logits) if Vp == V else logits.copy_(h @ weight.t())
            _lib.check(_K().hmf_ce_fwd_bwd(_lib.ptr(logits), _lib.ptr(labels[s:s + n]), _lib.ptr(loss),
                                           _lib.ptr(nvalid), c_ll(n), c_int(V), c_ll(Vp), c_ll(ignore_index),
                                           _st(hidden)), "ce_fwd_bwd")
            if need_dh:
                if own:
                    gemm(logits, weight, b_mn_major=True, out=dh[s:s + n])
                else:
                    torch.matmul(logits, weight, out=dh[s:s + n])
            if need_dw:
                # dW[V, Dm] += dlogits^T[V, n] @ h[n, Dm]: both operands MN-major for the tcgen05 GEMM
                if V % 8 == 0 and Dm % 8 == 0:
                    gemm(logits, h, a_mn_major=True, b_mn_major=True, out=dw, out_mode="f32_accumulate")
                else:
                    dw.addmm_(logits.t().float(), h.float())
        ctx.save_for_backward(dh, dw)
        ctx.wdtype = weight.dtype
        ctx.mark_non_differentiable(nvalid)
        return loss[0], nvalid[0]

    @staticmethod
    def backward(ctx, dloss, _dn):
        dh, dw = ctx.saved_tensors
        gh = None if dh is None else dh * dloss.to(dh.dtype)
        gw = None if dw is None else (dw * dloss).to(ctx.wdtype)
        return gh, gw, None, None, None


def linear_cross_entropy(hidden, weight, labels, ignore_index=-100, chunk=8192):
    if not _is_bf16(hidden, weight):
        return R.linear_cross_entropy(hidden, weight, labels, ignore_index, "sum", chunk)
    return _LinearCE.apply(hidden, weight, labels, ignore_index, chunk)


# ----------------------------------------------------------------------------------------
# optimizer kernels
# ----------------------------------------------------------------------------------------
_DT = {torch.bfloat16: 0, torch.float32: 1}


def grad_sumsq(flat_grad: Tensor, out: Tensor) -> None:
    """``out[0] += sum(flat_grad ** 2)`` (fp32 accumulator on the device, no host sync)."""
    _lib.check(_K().hmf_sumsq(_lib.ptr(flat_grad), c_int(1 if flat_grad.dtype == BF16 else 0), c_ll(flat_grad.numel()),
                              _lib.ptr(out), _st(flat_grad)), "sumsq")


def adamw_step(p: Tensor, g: Tensor, m: Tensor, v: Tensor, *, lr: float, beta1: float, beta2: float, eps: float,
               weight_decay: float, step: int, master: Optional[Tensor] = None, norm_sq: Optional[Tensor] = None,
               max_norm: float = 0.0, grad_scale: float = 1.0) -> None:
    """Fused AdamW over flat buffers, with optional global-norm clipping read from ``norm_sq``."""
    bc1, bc2 = 1.0 - beta1 ** step, 1.0 - beta2 ** step
    _lib.check(_K().hmf_adamw(_lib.ptr(p), _lib.ptr(g), _lib.ptr(m), _lib.ptr(v), _lib.ptr(master), c_ll(p.numel()),
                              c_int(_DT[p.dtype]), c_int(_DT[g.dtype]), c_int(_DT[m.dtype]), c_float(lr), c_float(beta1),
                              c_float(beta2), c_float(eps), c_float(weight_decay), c_float(bc1), c_float(bc2),
                              _lib.ptr(norm_sq), c_float(max_norm), c_float(grad_scale), _st(p)), "adamw")


# ----------------------------------------------------------------------------------------
# flash attention (tcgen05)
# ----------------------------------------------------------------------------------------
_INT_MAX = 2 ** 31 - 1


def _mask_bounds(causal: bool, window: Optional[int], hollow: Optional[int]) -> Tuple[int, int]:
    """(lo, hi) with key visible iff ``lo <= q_pos - k_pos < hi``."""
    assert causal, "non-causal attention is not part of this library"
    lo, hi = 0, _INT_MAX
    if window is not None:
        hi = min(hi, int(window))
    if hollow is not None:
        lo, hi = max(lo, int(hollow)), min(hi, 2 * int(hollow))
    return lo, hi


def _bthd_strides(t: Tensor):
    assert t.stride(3) == 1, "head dimension must be contiguous"
    return c_ll(t.stride(0)), c_ll(t.stride(1)), c_ll(t.stride(2))


def _tma_ok(t: Tensor) -> bool:
    return (t.stride(3) == 1 and t.data_ptr() % 16 == 0 and all(s % 8 == 0 for s in t.stride()[:3]))


def attention_fwd_raw(q: Tensor, k: Tensor, v: Tensor, scale: float, lo: int, hi: int, q_off: int,
                      q_pos: Optional[Tensor] = None) -> Tuple[Tensor, Tensor]:
    """Launches the forward kernel; returns ``(o [B,Tq,Hq,D] bf16, lse [B,Hq,Tq] fp32)``."""
    B, Tq, Hq, D = q.shape
    Tk, Hkv = k.shape[1], k.shape[2]
    q = q if _tma_ok(q) else q.contiguous()
    k = k if _tma_ok(k) else k.contiguous()
    v = v if _tma_ok(v) else v.contiguous()
    o = torch.empty(B, Tq, Hq, D, device=q.device, dtype=BF16)
    lse = torch.empty(B, Hq, Tq, device=q.device, dtype=torch.float32)
    if q_pos is not None:
        q_pos = q_pos.to(torch.int32).contiguous()
    _lib.check(_K().hmf_attention_fwd(_lib.ptr(q), _lib.ptr(k), _lib.ptr(v), _lib.ptr(o), _lib.ptr(lse), _lib.ptr(q_pos),
                                      c_int(B), c_int(Tq), c_int(Tk), c_int(Hq), c_int(Hkv), c_int(D),
                                      *_bthd_strides(q), *_bthd_strides(k), *_bthd_strides(v), c_int(lo), c_int(hi),
                                      c_int(q_off), c_float(scale), _st(q)), "attention_fwd")
    return o, lse


_warned = set()


def warn_once(msg: str) -> None:
    """One warning per distinct message when a bf16 CUDA tensor leaves the kernel path (orders of magnitude slower)."""
    if msg not in _warned:
        _warned.add(msg)
        import warnings
        warnings.warn(msg, stacklevel=3)


def _attention_bwd_blocked(q, k, v, o, do, lse, scale, lo, hi, q_off, q_pos=None, dlse=None, block: int = 1024):
    """Attention backward for head dimensions without a backward kernel (256): recomputes the probabilities from the
    saved log-sum-exp one block of query rows at a time (memory O(block x Tk) per head) with library matrix products."""
    B, Tq, Hq, D = q.shape
    Tk, Hkv = k.shape[1], k.shape[2]
    G = Hq // Hkv
    dq = torch.empty_like(q)
    dk = torch.zeros(B, Tk, Hkv, D, device=q.device, dtype=torch.float32)
    dv = torch.zeros_like(dk)
    delta = (o.float() * do.float()).sum(-1)                              # [B, Tq, Hq]
    if dlse is not None:
        delta = delta - dlse.transpose(1, 2)
    kpos = torch.arange(Tk, device=q.device)
    kf, vf = k.float(), v.float()
    for s in range(0, Tq, block):
        e = min(Tq, s + block)
        pos = (q_pos[:, s:e].long() if q_pos is not None else (torch.arange(s, e, device=q.device) + q_off)[None].expand(B, -1))
        diff = pos[:, :, None] - kpos[None, None, :]
        vis = (diff >= lo) & (diff < hi)                                  # [B, n, Tk]
        qb = q[:, s:e].float().view(B, e - s, Hkv, G, D)
        dob = do[:, s:e].float().view(B, e - s, Hkv, G, D)
        sc = torch.einsum("bnhgd,bkhd->bhgnk", qb, kf) * scale
        lse_b = lse[:, :, s:e].view(B, Hkv, G, e - s)
        p = torch.exp(sc - lse_b[..., None]).masked_fill(~vis[:, None, None], 0.0)
        p = torch.nan_to_num(p, nan=0.0)
        dp = torch.einsum("bnhgd,bkhd->bhgnk", dob, vf)
        ds = p * (dp - delta[:, s:e].view(B, e - s, Hkv, G).permute(0, 2, 3, 1)[..., None]) * scale
        dq[:, s:e] = torch.einsum("bhgnk,bkhd->bnhgd", ds, kf).reshape(B, e - s, Hq, D).to(q.dtype)
        dk += torch.einsum("bhgnk,bnhgd->bkhd", ds, qb)
        dv += torch.einsum("bhgnk,bnhgd->bkhd", p, dob)
    return dq, dk.to(k.dtype), dv.to(v.dtype)


def deterministic_attention_backward() -> bool:
    """True when the attention backward must sum dQ in a fixed order (``torch.use_deterministic_algorithms`` or
    ``HMF_ATTN_BWD_DETERMINISTIC=1``): the two-kernel path, 7 GEMMs per tile pair, no atomics."""
    return os.environ.get("HMF_ATTN_BWD_DETERMINISTIC", "0") == "1" or torch.are_deterministic_algorithms_enabled()


def attention_bwd_raw(q, k, v, o, do, lse, scale, lo, hi, q_off, q_pos=None, dlse=None, deterministic=None):
    """Gradients of ``attention_fwd_raw``; returns ``(dq, dk, dv)`` (bf16, contiguous).

    Head dimension 128 runs the single fused kernel (S and dP computed once per tile pair, dQ summed into an fp32
    buffer with global reductions, then converted); head dimension 64, or ``deterministic``, runs the dQ and dK/dV
    kernels separately."""
    B, Tq, Hq, D = q.shape
    Tk, Hkv = k.shape[1], k.shape[2]
    if D not in (64, 128):
        warn_once(f"attention backward: head dimension {D} has a forward kernel only; the gradients are computed "
                  "block by block with library matrix products")
        return _attention_bwd_blocked(q, k, v, o, do, lse, scale, lo, hi, q_off, q_pos, dlse)
    q = q if _tma_ok(q) else q.contiguous()
    k = k if _tma_ok(k) else k.contiguous()
    v = v if _tma_ok(v) else v.contiguous()
    o, do = o.contiguous(), do.contiguous()
    dq = torch.empty(B, Tq, Hq, D, device=q.device, dtype=BF16)
    dk = torch.empty(B, Tk, Hkv, D, device=q.device, dtype=BF16)
    dv = torch.empty(B, Tk, Hkv, D, device=q.device, dtype=BF16)
    delta = torch.empty(B, Hq, Tq, device=q.device, dtype=torch.float32)
    if q_pos is not None:
        q_pos = q_pos.to(torch.int32).contiguous()
    if dlse is not None:
        dlse = dlse.float().contiguous()
    if deterministic is None:
        deterministic = deterministic_attention_backward()
    if D == 128 and not deterministic:
        dq_acc = torch.zeros(B, Tq, Hq, D, device=q.device, dtype=torch.float32)
        _lib.check(_K().hmf_attention_bwd_fused(
            _lib.ptr(q), _lib.ptr(k), _lib.ptr(v), _lib.ptr(o), _lib.ptr(do), _lib.ptr(lse), _lib.ptr(dlse),
            _lib.ptr(delta), _lib.ptr(dq_acc), _lib.ptr(dq), _lib.ptr(dk), _lib.ptr(dv), _lib.ptr(q_pos),
            c_int(B), c_int(Tq), c_int(Tk), c_int(Hq), c_int(Hkv), c_int(D),
            *_bthd_strides(q), *_bthd_strides(k), *_bthd_strides(v), c_int(lo), c_int(hi),
            c_int(q_off), c_float(scale), _st(q)), "attention_bwd_fused")
        _lib.add_launches(2)
        return dq, dk, dv
    _lib.check(_K().hmf_attention_bwd(_lib.ptr(q), _lib.ptr(k), _lib.ptr(v), _lib.ptr(o), _lib.ptr(do), _lib.ptr(lse),
                                      _lib.ptr(dlse), _lib.ptr(delta), _lib.ptr(dq), _lib.ptr(dk), _lib.ptr(dv), _lib.ptr(q_pos),
                                      c_int(B), c_int(Tq), c_int(Tk), c_int(Hq), c_int(Hkv), c_int(D),
                                      *_bthd_strides(q), *_bthd_strides(k), *_bthd_strides(v), c_int(lo), c_int(hi),
                                      c_int(q_off), c_float(scale), _st(q)), "attention_bwd")
    _lib.add_launches(2)
    return dq, dk, dv


class _Attention(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, scale, lo, hi, q_off, q_pos):
        o, lse = attention_fwd_raw(q, k, v, scale, lo, hi, q_off, q_pos)
        ctx.save_for_backward(q, k, v, o, lse, q_pos)
        ctx.cfg = (scale, lo, hi, q_off)
        ctx.set_materialize_grads(False)      # the lse output usually carries no gradient
        return o, lse

    @staticmethod
    def backward(ctx, do, dlse):
        q, k, v, o, lse, q_pos = ctx.saved_tensors
        scale, lo, hi, q_off = ctx.cfg
        if do is None:
            do = torch.zeros_like(o)
        dq, dk, dv = attention_bwd_raw(q, k, v, o, do, lse, scale, lo, hi, q_off, q_pos, dlse)
        return dq, dk, dv, None, None, None, None, None


class _AttentionFromSaved(torch.autograd.Function):
    """Re-registers the backward of an attention call whose forward result was stashed by the first run
    of a checkpointed layer (``utils/checkpointing.py``): no forward kernel is launched."""

    @staticmethod
    def forward(ctx, q, k, v, o, lse, scale, lo, hi, q_off, q_pos):
        ctx.save_for_backward(q, k, v, o, lse, q_pos)
        ctx.cfg = (scale, lo, hi, q_off)
        ctx.set_materialize_grads(False)
        return o.view_as(o), lse.view_as(lse)

    @staticmethod
    def backward(ctx, do, dlse):
        q, k, v, o, lse, q_pos = ctx.saved_tensors
        scale, lo, hi, q_off = ctx.cfg
        if do is None:
            do = torch.zeros_like(o)
        dq, dk, dv = attention_bwd_raw(q, k, v, o, do, lse, scale, lo, hi, q_off, q_pos, dlse)
        return dq, dk, dv, None, None, None, None, None, None, None


def _contiguous_positions(pos: Optional[Tensor], n: int) -> Optional[int]:
    """Offset ``c`` if ``pos[b, i] == i + c`` for every row, else ``None`` (host sync: small tensors only)."""
    if pos is None:
        return 0
    first = pos[:, :1]
    if bool((pos == first + torch.arange(n, device=pos.device)[None]).all()) and bool((first == first[0]).all()):
        return int(first[0, 0])
    return None


def attention(q, k, v, *, scale=None, causal=True, window=None, hollow=None, q_pos=None, k_pos=None,
              return_lse=False):
    """Softmax attention on the tcgen05 kernels.  ``q_pos`` / ``k_pos`` follow the reference contract;
    keys must sit at contiguous positions, queries either contiguous or ascending (query-sparse)."""
    D = q.shape[-1]
    if not _is_bf16(q, k, v) or D not in (64, 128, 256):
        if q.is_cuda and q.dtype == BF16:
            warn_once(f"attention: head dimension {D} has no kernel; evaluating the PyTorch formulation on the GPU")
        return R.attention(q, k, v, scale=scale, causal=causal, window=window, hollow=hollow, q_pos=q_pos,
                           k_pos=k_pos, return_lse=return_lse)
    Tq, Tk = q.shape[1], k.shape[1]
    scale = D ** -0.5 if scale is None else scale
    lo, hi = _mask_bounds(causal, window, hollow)
    k_off = _contiguous_positions(k_pos, Tk)
    if k_off is None:
        # keys at irregular positions (B'MOJO halo with padded negatives): shift is not expressible
        warn_once("attention: keys at irregular positions; evaluating the PyTorch formulation on the GPU")
        return R.attention(q, k, v, scale=scale, causal=causal, window=window, hollow=hollow, q_pos=q_pos,
                           k_pos=k_pos, return_lse=return_lse)
    qp = None
    if q_pos is None:
        q_off = Tk - Tq
    else:
        c = _contiguous_positions(q_pos, Tq)
        if c is not None:
            q_off = c - k_off
        else:
            q_off, qp = 0, (q_pos - k_off)
    from ..utils import checkpointing as _ckpt
    rd = _ckpt.stash_for_read()
    if rd is not None and torch.is_grad_enabled() and len(rd) > 0:
        o_saved, lse_saved = rd.pop(0)
        o, lse = _AttentionFromSaved.apply(q, k, v, o_saved, lse_saved, scale, lo, hi, q_off, qp)
    else:
        o, lse = _apply(_Attention, q, k, v, scale, lo, hi, q_off, qp)
        wr = _ckpt.stash_for_write()
        if wr is not None:
            wr.append((o.detach(), lse.detach()))
    return (o, lse) if return_lse else o


def qsparse_attention(q, k, v, q_index, scale=None):
    return attention(q, k, v, scale=scale, causal=True, q_pos=q_index)


# ----------------------------------------------------------------------------------------
# scan cores (Gated DeltaNet, GKA, SSD)
# ----------------------------------------------------------------------------------------
from .scan import TorchScanCore  # noqa: E402


def _gdn_state_shapes(inputs):
    q, v = inputs[0], inputs[2]
    return [((q.shape[0], q.shape[2], q.shape[3], v.shape[3]), torch.float32)]


def GDNCore(scale=None, chunk_size=64, use_qk_l2norm=True, recurrent=False):
    """Scan core of the gated delta rule on the GPU."""
    from . import gdn_cuda
    if gdn_cuda.available() and not recurrent and chunk_size == 64:
        return gdn_cuda.GDNChunkCore(scale=scale, use_qk_l2norm=use_qk_l2norm)
    fn = R.gated_delta_rule_recurrent if recurrent else R.gated_delta_rule_chunk
    kw = dict(scale=scale, use_qk_l2norm=use_qk_l2norm)
    if not recurrent:
        kw["chunk_size"] = chunk_size
    return TorchScanCore(fn, n_state=1, state_shape_fn=_gdn_state_shapes, **kw)
