"""Chunked gated delta rule on the GPU.

Pipeline of one segment (forward):
  1. chunk-parallel preparation (``_prep``): L2 norms, cumulative gates, the WY factors
     ``u = T (beta v)``, ``w = T (beta e^{G} k)`` with ``T = (I + tril(beta k k^T . decay))^{-1}``, the
     causal intra-chunk score matrix ``P`` and the decayed keys / queries, packed as the bf16
     operand tiles of the scan kernel;
  2. ``hmf_gdn_scan_fwd`` (``csrc/kernels/gdn_scan.cu``): the sequential inter-chunk recurrence
     *and* the output, on tcgen05 with the state in registers / tensor memory.
Backward: ``hmf_gdn_scan_bwd`` runs the reverse recurrence for the state gradient; the gradients
of the per-chunk factors are four batched products of saved tensors, and autograd carries them
through the preparation graph to ``q, k, v, g, beta``.

The preparation currently runs as batched PyTorch ops on the device.
"""
from __future__ import annotations

import ctypes
from typing import Optional

import torch

from . import _lib
from . import reference as R
from .scan import ScanCore, TorchScanCore

c_int, c_uint = ctypes.c_int, ctypes.c_uint
import os

BF16 = torch.bfloat16
C = 64
# debugging aid: evaluate the chunk preparation with batched PyTorch ops instead of the CUDA kernel
_FORCE_TORCH_PREP = os.environ.get("HMF_GDN_TORCH_PREP", "0") == "1"
_USE_BWD_KERNEL = os.environ.get("HMF_GDN_BWD_KERNEL", "1") == "1"
_GLA_SEGMENTS = os.environ.get("HMF_GLA_SEGMENTS", "1") == "1"      # segment-parallel inference scan (gla mode)


def available() -> bool:
    if not _lib.kernels_available():
        return False
    return hasattr(_lib.kernels(), "hmf_gdn_scan_fwd")


def _chunk(x: torch.Tensor, N: int) -> torch.Tensor:
    """``[B, T, H, ...] -> [B*H, N, C, ...]`` (zero padded to ``N*C`` tokens)."""
    B, T, H = x.shape[:3]
    rest = x.shape[3:]
    pad = N * C - T
    if pad:
        x = torch.cat([x, x.new_zeros(B, pad, H, *rest)], dim=1)
    x = x.reshape(B, N, C, H, *rest)
    perm = (0, 3, 1, 2) + tuple(range(4, 4 + len(rest)))
    return x.permute(*perm).reshape(B * H, N, C, *rest)


def _chunkf(x: torch.Tensor, N: int) -> torch.Tensor:
    """:func:`_chunk` fused with the conversion to fp32 (one pass over the data instead of two)."""
    B, T, H = x.shape[:3]
    if N * C != T:
        return _chunk(x, N).float()
    rest = x.shape[3:]
    perm = (0, 3, 1, 2) + tuple(range(4, 4 + len(rest)))
    return x.reshape(B, N, C, H, *rest).permute(*perm).float().reshape(B * H, N, C, *rest)


def _unchunk_into(dst: torch.Tensor, x: torch.Tensor) -> None:
    """``dst [B, T, H, ...]`` (any dtype / strides) <- ``x [B*H, N, C, ...]``; one strided pass when ``T = N*C``."""
    B, T, H = dst.shape[:3]
    N = x.shape[1]
    rest = x.shape[3:]
    if N * C != T:
        dst.copy_(_unchunk(x, B, H, T))
        return
    perm = (0, 3, 1, 2) + tuple(range(4, 4 + len(rest)))
    dst.unflatten(1, (N, C)).permute(*perm).copy_(x.reshape(B, H, N, C, *rest))


def _unchunk(x: torch.Tensor, B: int, H: int, T: int) -> torch.Tensor:
    """Inverse of :func:`_chunk`: ``[B*H, N, C, ...] -> [B, T, H, ...]``."""
    N = x.shape[1]
    rest = x.shape[3:]
    x = x.reshape(B, H, N, C, *rest)
    perm = (0, 2, 3, 1) + tuple(range(4, 4 + len(rest)))
    return x.permute(*perm).reshape(B, N * C, H, *rest)[:, :T]


class _tf32_matmul:
    """fp32 matmuls of the chunk-local backward on the tensor cores (TF32); restored on exit."""

    def __enter__(self):
        self.prev = torch.backends.cuda.matmul.allow_tf32
        torch.backends.cuda.matmul.allow_tf32 = True

    def __exit__(self, *exc):
        torch.backends.cuda.matmul.allow_tf32 = self.prev


class GDNChunkCore(ScanCore):
    n_state = 1

    def __init__(self, scale: Optional[float] = None, use_qk_l2norm: bool = True, gla: bool = False):
        """``gla=True``: plain gated linear attention ``S_t = e^{g_t} S_{t-1} + k_t v_t^T`` (no delta rule;
        ``beta`` is ignored).  Same kernels: the WY factors degenerate to ``w = 0``, ``u = v``."""
        self.scale, self.use_qk_l2norm, self.gla = scale, use_qk_l2norm, gla
        if gla:
            self._fallback = TorchScanCore(lambda q, k, v, g, beta, initial_state=None: R.simple_gla_chunk(
                q, k, v, g, scale=scale, initial_state=initial_state, chunk_size=C), n_state=1,
                state_shape_fn=self.state_shapes)
        else:
            self._fallback = TorchScanCore(R.gated_delta_rule_chunk, n_state=1, state_shape_fn=self.state_shapes,
                                           scale=scale, use_qk_l2norm=use_qk_l2norm, chunk_size=C)
        # sequence-parallel hooks filled in by parallel.peer.PeerStateTransport
        self.peer = None

    def state_shapes(self, inputs):
        q, v = inputs[0], inputs[2]
        return [((q.shape[0], q.shape[2], q.shape[3], v.shape[3]), torch.float32)]

    @staticmethod
    def _supported(q, k, v) -> bool:
        return (q.is_cuda and q.dtype == BF16 and k.dtype == BF16 and v.dtype == BF16 and q.shape[-1] == 128
                and v.shape[-1] == 128)

    # -- chunk-parallel preparation ------------------------------------------------------
    def _prep(self, q, k, v, g, beta):
        B, T, H, Dk = q.shape
        N = (T + C - 1) // C
        scale = Dk ** -0.5 if self.scale is None else self.scale
        qf, kf, vf = _chunk(q, N).float(), _chunk(k, N).float(), _chunk(v, N).float()
        gc = _chunk(g.float(), N)
        bc = torch.ones_like(gc) if self.gla else _chunk(beta.float(), N)
        if self.use_qk_l2norm:
            qf = qf * torch.rsqrt(qf.pow(2).sum(-1, keepdim=True) + 1e-6)
            kf = kf * torch.rsqrt(kf.pow(2).sum(-1, keepdim=True) + 1e-6)
        qf = qf * scale
        G = gc.cumsum(-1)
        glast = G[..., -1]
        idx = torch.arange(C, device=q.device)
        lower = idx[:, None] >= idx[None, :]
        strict = idx[:, None] > idx[None, :]
        diff = G[..., :, None] - G[..., None, :]
        decay = torch.exp(diff.masked_fill(~lower, 0.0)) * lower
        if self.gla:
            u, w = vf, torch.zeros_like(kf)
        else:
            A = (bc[..., None] * (kf @ kf.transpose(-1, -2)) * decay) * strict
            eye = torch.eye(C, device=q.device, dtype=torch.float32)
            Tm = torch.linalg.solve_triangular(eye + A, eye.expand_as(A), upper=False)
            u = Tm @ (vf * bc[..., None])
            w = Tm @ (kf * (bc * torch.exp(G))[..., None])
        P = (qf @ kf.transpose(-1, -2)) * decay
        qt = qf * torch.exp(G)[..., None]
        kt = kf * torch.exp(glast[..., None] - G)[..., None]
        return {"w": w, "qt": qt, "kt": kt, "P": P, "u": u, "glast": glast, "N": N}

    def _prep_backward(self, q, k, v, g, beta, d_w, d_qt, d_kt, d_P, d_u, d_gl):
        """Hand-written backward of :meth:`_prep` (no autograd graph, a third of the memory passes).
        ``q, k, v [B,T,h,D]``, ``g, beta [B,T,h]``; upstream gradients in chunk layout ``[B*h, N, C, .]`` (``d_P``
        lower triangular, ``d_gl [B*h, N]``).  Returns ``dq, dk, dv, dg, dbeta`` in the input layouts."""
        B, T, H, Dk = q.shape
        N = (T + C - 1) // C
        scale = Dk ** -0.5 if self.scale is None else self.scale
        qf, kf, vf = _chunkf(q, N), _chunkf(k, N), _chunkf(v, N)
        gc = _chunkf(g, N)
        if self.use_qk_l2norm:
            rq = torch.rsqrt(qf.pow(2).sum(-1, keepdim=True) + 1e-6)
            rk = torch.rsqrt(kf.pow(2).sum(-1, keepdim=True) + 1e-6)
            qn, kn = qf * (rq * scale), kf * rk
        else:
            qn, kn = qf * scale, kf
        G = gc.cumsum(-1)
        eG = torch.exp(G)
        eR = torch.exp(G[..., -1:] - G)
        idx = torch.arange(C, device=q.device)
        lower = idx[:, None] >= idx[None, :]
        strict = idx[:, None] > idx[None, :]
        Dm = torch.exp((G[..., :, None] - G[..., None, :]).masked_fill(~lower, 0.0)) * lower
        knT = kn.transpose(-1, -2)
        # intra-chunk scores P = (qn kn^T) . D
        Nm = d_P * Dm
        dqn = Nm @ kn
        dkn = Nm.transpose(-1, -2) @ qn
        sP = Nm * (qn @ knT)                        # d_P . P
        dG = sP.sum(-1) - sP.sum(-2)
        # decayed queries / keys
        dqn.addcmul_(d_qt, eG[..., None])
        dG += (d_qt * qn).sum(-1) * eG
        dkn.addcmul_(d_kt, eR[..., None])
        t = (d_kt * kn).sum(-1) * eR
        dG -= t
        dG[..., -1] += t.sum(-1) + d_gl
        dbeta = None
        if self.gla:
            dv = d_u
        else:
            bc = _chunkf(beta, N)
            KK = kn @ knT
            KD = KK * Dm * strict
            A = bc[..., None] * KD
            eye = torch.eye(C, device=q.device, dtype=torch.float32)
            Tm = torch.linalg.solve_triangular(eye + A, eye.expand_as(A), upper=False)
            TmT = Tm.transpose(-1, -2)
            be = bc * eG
            dbv, dbk = TmT @ d_u, TmT @ d_w
            dT = d_u @ (vf * bc[..., None]).transpose(-1, -2) + d_w @ (kn * be[..., None]).transpose(-1, -2)
            dA = -(TmT @ dT @ TmT) * strict
            Mm = dA * Dm * bc[..., None]
            dkn += Mm @ kn
            dkn += Mm.transpose(-1, -2) @ kn
            sA = dA * A
            dG += sA.sum(-1) - sA.sum(-2)
            dbeta = (dA * KD).sum(-1)
            dv = dbv * bc[..., None]
            dbeta += (dbv * vf).sum(-1)
            dkn.addcmul_(dbk, be[..., None])
            x = (dbk * kn).sum(-1) * eG
            dbeta += x
            dG += x * bc
        dg = dG.flip(-1).cumsum(-1).flip(-1)
        if self.use_qk_l2norm:
            dq = (dqn - qn * ((qn * dqn).sum(-1, keepdim=True) / (scale * scale))) * (rq * scale)
            dk = (dkn - kn * (kn * dkn).sum(-1, keepdim=True)) * rk
        else:
            dq, dk = dqn * scale, dkn
        return dq, dk, dv, dg, dbeta          # chunk layout [B*h, N, C, .]; the caller scatters them

    @staticmethod
    def _pack(f):
        wqT = torch.stack([f["w"].transpose(-1, -2), f["qt"].transpose(-1, -2)], dim=2).to(BF16).contiguous()
        kPT = torch.cat([f["kt"].transpose(-1, -2), f["P"]], dim=-2).to(BF16).contiguous()
        uT = f["u"].transpose(-1, -2).to(BF16).contiguous()
        return wqT, kPT, uT, f["glast"].float().contiguous()

    # -- ScanCore API ---------------------------------------------------------------------
    @staticmethod
    def _head_groups(B, T, H):
        """Head slices such that one fp32 ``[B, T, hs, 128]`` intermediate stays near 256 MB."""
        per_head = B * T * 128 * 4
        g = max(1, min(H, (256 << 20) // max(per_head, 1)))
        return [slice(i, min(H, i + g)) for i in range(0, H, g)]

    def _packed_buffers(self, B, H, N, Dk, Dv, device):
        wqT = torch.empty(B, H, N, 2, Dk, C, device=device, dtype=BF16)
        kPT = torch.empty(B, H, N, Dk + C, C, device=device, dtype=BF16)
        uT = torch.empty(B, H, N, Dv, C, device=device, dtype=BF16)
        glast = torch.empty(B, H, N, device=device, dtype=torch.float32)
        return wqT, kPT, uT, glast

    def _prep_packed(self, q, k, v, g, beta, want_u=True):
        """Runs the preparation head group by head group and returns the packed operand tiles."""
        B, T, H, Dk = q.shape
        Dv = v.shape[-1]
        N = (T + C - 1) // C
        wqT, kPT, uT, glast = self._packed_buffers(B, H, N, Dk, Dv, q.device)
        if hasattr(_lib.kernels(), "hmf_gdn_prep") and not _FORCE_TORCH_PREP:
            def tma_ok(t):
                return t.stride(3) == 1 and t.data_ptr() % 16 == 0 and all(s % 8 == 0 for s in t.stride()[:3])
            q, k, v = (t if tma_ok(t) else t.contiguous() for t in (q, k, v))
            scale = Dk ** -0.5 if self.scale is None else self.scale
            ll = ctypes.c_longlong
            g32 = g.float().contiguous()        # held in locals: a temporary's block could be reused before the launch
            b32 = None if self.gla else beta.float().contiguous()
            rc = _lib.kernels().hmf_gdn_prep(
                _lib.ptr(q), _lib.ptr(k), _lib.ptr(v), _lib.ptr(g32),
                _lib.ptr(b32), _lib.ptr(wqT), _lib.ptr(kPT), _lib.ptr(uT), _lib.ptr(glast),
                c_int(B), c_int(T), c_int(H), c_int(k.shape[2]), c_int(v.shape[2]), c_int(N),
                ll(q.stride(0)), ll(q.stride(1)), ll(q.stride(2)), ll(k.stride(0)), ll(k.stride(1)), ll(k.stride(2)),
                ll(v.stride(0)), ll(v.stride(1)), ll(v.stride(2)), ctypes.c_float(scale),
                c_int(int(self.use_qk_l2norm)), c_int(int(self.gla)), _lib.stream_ptr(q.device))
            _lib.check(rc, "hmf_gdn_prep")
            return wqT, kPT, uT, glast, N
        for hs in self._head_groups(B, T, H):
            f = self._prep(q[:, :, hs], k[:, :, hs], v[:, :, hs], g[:, :, hs],
                           None if beta is None else beta[:, :, hs])
            a, b_, c_, d_ = self._pack(f)
            nh = hs.stop - hs.start
            wqT[:, hs] = a.view(B, nh, N, 2, Dk, C)
            kPT[:, hs] = b_.view(B, nh, N, Dk + C, C)
            if want_u:
                uT[:, hs] = c_.view(B, nh, N, Dv, C)
            glast[:, hs] = d_.view(B, nh, N)
            del f, a, b_, c_, d_
        return wqT, kPT, uT, glast, N

    def peer_capable(self, inputs) -> bool:
        """The scan kernels can receive / push the state over peer memory for these inputs."""
        q, k, v = inputs[:3]
        return available() and self._supported(q, k, v)

    def forward(self, inputs, state0, peer=None):
        q, k, v, g, beta = inputs
        if not self._supported(q, k, v):
            assert peer is None
            out, sT, saved, meta = self._fallback.forward(inputs, state0)
            return out, sT, saved, ("fallback", meta)
        B, T, H, Dk = q.shape
        Dv = v.shape[-1]
        need_bwd = any(t is not None and t.requires_grad for t in inputs) or (
            state0 is not None and state0[0].requires_grad)
        if (self.gla and not need_bwd and peer is None and B == 1 and T >= 2048 and 2 * H <= 148 and _GLA_SEGMENTS
                and q.stride(3) == 1 and k.stride(3) == 1 and v.stride(3) == 1):
            P = min(8, 148 // H, T // 512)
            if P >= 2:
                return self._forward_segmented(q, k, v, g, state0, P)
        with torch.no_grad():
            wqT, kPT, uT, glast, N = self._prep_packed(q, k, v, g, beta)
            h0 = None if state0 is None else state0[0].float().contiguous()
            h0_flag, push_ptr, push_flag, epoch = None, None, None, 0
            if peer is not None:
                if peer.recv is not None:       # incoming state arrives in the symmetric buffer
                    h0, h0_flag = peer.recv, peer.recv_flag
                push_ptr = ctypes.c_void_p(peer.push_ptr) if peer.push_ptr else None
                push_flag = ctypes.c_void_p(peer.push_flag_ptr) if peer.push_ptr else None
                epoch = peer.epoch
            o = torch.empty(B, T, H, Dv, device=q.device, dtype=BF16)
            hT = torch.empty(B, H, Dk, Dv, device=q.device, dtype=torch.float32)
            vnT = torch.empty(B * H, N, Dv, C, device=q.device, dtype=BF16) if need_bwd else None
            h_all = torch.empty(B * H, N, Dv, Dk, device=q.device, dtype=BF16) if need_bwd else None
            rc = _lib.kernels().hmf_gdn_scan_fwd(
                _lib.ptr(wqT), _lib.ptr(kPT), _lib.ptr(uT), _lib.ptr(glast), _lib.ptr(h0), _lib.ptr(hT), _lib.ptr(o),
                _lib.ptr(vnT), _lib.ptr(h_all), c_int(B), c_int(H), c_int(T), c_int(N), _lib.ptr(h0_flag), push_ptr,
                push_flag, c_uint(epoch), _lib.stream_ptr(q.device))
            _lib.check(rc, "hmf_gdn_scan_fwd")
        # the incoming state itself is not needed again: the backward kernel reads the per-chunk states
        saved = [q, k, v, g, beta, None, vnT, h_all]
        return o, (hT,), saved, ("cuda", h0 is not None)

    def _scan(self, wqT, kPT, uT, glast, h0, hT, o, B, H, T, N, device):
        _lib.check(_lib.kernels().hmf_gdn_scan_fwd(
            _lib.ptr(wqT), _lib.ptr(kPT), _lib.ptr(uT), _lib.ptr(glast), _lib.ptr(h0), _lib.ptr(hT), _lib.ptr(o), None,
            None, c_int(B), c_int(H), c_int(T), c_int(N), None, None, None, c_uint(0), _lib.stream_ptr(device)),
            "hmf_gdn_scan_fwd")

    def _forward_segmented(self, q, k, v, g, state0, P):
        """Inference forward of plain gated linear attention (Mamba2 SSD, GLA) for one long sequence and few heads:
        the scan kernel runs one CTA per (batch, head), so 4 heads of a tensor-parallel shard would use 4 of 148 SMs.
        The sequence is cut into ``P`` equal segments scanned as a batch from a zero state, a prefix kernel turns the
        segment states into every segment's true incoming state, and the batch is scanned again from those; a tail
        shorter than a segment follows on its own."""
        _, T, H, Dk = q.shape
        Dv = v.shape[-1]
        L = (T // P) // C * C
        main, dev = P * L, q.device
        with torch.no_grad():
            def seg(t):         # [1, T, ...] -> [P, L, ...] without copying
                return t.as_strided((P, L) + tuple(t.shape[2:]), (L * t.stride(1),) + tuple(t.stride()[1:]),
                                    t.storage_offset())
            g32 = g.float()
            wqT, kPT, uT, glast, N = self._prep_packed(seg(q), seg(k), seg(v), seg(g32), None)
            o = torch.empty(1, T, H, Dv, device=dev, dtype=BF16)
            seg_state = torch.empty(P, H, Dk, Dv, device=dev, dtype=torch.float32)
            self._scan(wqT, kPT, uT, glast, None, seg_state, o, P, H, L, N, dev)           # pass 1: zero start
            h0 = None if state0 is None else state0[0].float().contiguous()
            s_in = torch.empty_like(seg_state)
            hT = torch.empty(1, H, Dk, Dv, device=dev, dtype=torch.float32)
            E, ll = Dk * Dv, ctypes.c_longlong
            _lib.check(_lib.kernels().hmf_gla_segment_prefix(
                _lib.ptr(seg_state), _lib.ptr(glast), _lib.ptr(h0), _lib.ptr(s_in), _lib.ptr(hT), c_int(P), c_int(H),
                c_int(N), c_int(E), ll(H * E), ll(E), ll(H * N), ll(N), ll(H * E), ll(E), ll(E),
                _lib.stream_ptr(dev)), "gla_segment_prefix")
            self._scan(wqT, kPT, uT, glast, s_in, seg_state, o, P, H, L, N, dev)          # pass 2: true states
            if main < T:
                tail = slice(main, T)
                wq2, kP2, u2, gl2, N2 = self._prep_packed(q[:, tail], k[:, tail], v[:, tail], g32[:, tail], None)
                hT2 = torch.empty_like(hT)
                self._scan(wq2, kP2, u2, gl2, hT, hT2, o[:, tail], 1, H, T - main, N2, dev)
                hT = hT2
        return o, (hT,), [q, k, v, g, None, None, None, None], ("cuda", state0 is not None)

    def backward(self, saved, meta, d_out, d_stateT, peer=None):
        kind, info = meta
        if kind == "fallback":
            assert peer is None
            return self._fallback.backward(saved, info, d_out, d_stateT)
        q, k, v, g, beta, h0, vnT, h_all = saved
        B, T, H, Dk = q.shape
        Dv = v.shape[-1]
        with torch.no_grad():
            wqT, kPT, _, glast, N = self._prep_packed(q, k, v, g, beta, want_u=False)
            do = d_out.to(BF16).contiguous()
            dhT = None
            if d_stateT is not None and d_stateT[0] is not None:
                dhT = d_stateT[0].float().contiguous()
            dhT_flag, push_ptr, push_flag, epoch = None, None, None, 0
            if peer is not None:
                if peer.recv is not None:       # gradient of the outgoing state arrives in the symmetric buffer
                    dhT, dhT_flag = peer.recv, peer.recv_flag
                push_ptr = ctypes.c_void_p(peer.push_ptr) if peer.push_ptr else None
                push_flag = ctypes.c_void_p(peer.push_flag_ptr) if peer.push_ptr else None
                epoch = peer.epoch
            dh0 = torch.empty(B, H, Dk, Dv, device=q.device, dtype=torch.float32) if info else None
            dvnT = torch.empty(B * H, N, Dv, C, device=q.device, dtype=BF16)
            dS_all = torch.empty(B * H, N, Dv, Dk, device=q.device, dtype=BF16)
            rc = _lib.kernels().hmf_gdn_scan_bwd(
                _lib.ptr(wqT), _lib.ptr(kPT), _lib.ptr(do), _lib.ptr(glast), _lib.ptr(dhT), _lib.ptr(dh0),
                _lib.ptr(dvnT), _lib.ptr(dS_all), c_int(B), c_int(H), c_int(T), c_int(N), _lib.ptr(dhT_flag), push_ptr,
                push_flag, c_uint(epoch), _lib.stream_ptr(q.device))
            _lib.check(rc, "hmf_gdn_scan_bwd")
            del wqT, kPT
            dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
            dg = torch.empty_like(g)
            dbeta = None if (beta is None or self.gla) else torch.empty_like(beta)
            vn5, h5 = vnT.view(B, H, N, Dv, C), h_all.view(B, H, N, Dv, Dk)
            dvn5, dS5 = dvnT.view(B, H, N, Dv, C), dS_all.view(B, H, N, Dv, Dk)
            gl5 = glast.view(B, H, N)
        if hasattr(_lib.kernels(), "hmf_gdn_prep_bwd") and not _FORCE_TORCH_PREP and _USE_BWD_KERNEL:
            # factor gradients by four batched GEMMs, then one kernel for the whole chunk-local backward
            with torch.no_grad():
                vnT_g, h_g = vnT.view(B * H, N, Dv, C), h_all.view(B * H, N, Dv, Dk)
                dS_g = dS_all.view(B * H, N, Dv, Dk)
                do_c = _chunk(do, N)                             # [BH, N, C, Dv]
                dvn = dvnT.transpose(-1, -2)
                d_w = None if self.gla else (dvn @ h_g).neg_()   # [C, Dv] @ [Dv, Dk]
                d_qt = do_c @ h_g
                d_P = (do_c @ vnT_g).float()
                d_kt = vnT_g.transpose(-1, -2) @ dS_g
                d_gl = torch.exp(glast.view(B * H, N)) * (dS_g * h_g).sum((-1, -2), dtype=torch.float32)
                del do_c, dS_g
                if not (dq.is_contiguous() and dk.is_contiguous() and dv.is_contiguous()):
                    dq, dk, dv = (torch.empty(t.shape, device=t.device, dtype=t.dtype) for t in (q, k, v))
                qq, kk, vv = (t if (t.stride(3) == 1 and all(s_ % 4 == 0 for s_ in t.stride()[:3])) else t.contiguous()
                              for t in (q, k, v))
                g32 = g.float().contiguous()
                b32 = None if self.gla else beta.float().contiguous()
                dg32 = torch.empty(B, T, H, device=q.device, dtype=torch.float32)
                db32 = None if self.gla else torch.empty(B, T, H, device=q.device, dtype=torch.float32)
                scale = Dk ** -0.5 if self.scale is None else self.scale
                ll = ctypes.c_longlong
                rc = _lib.kernels().hmf_gdn_prep_bwd(
                    _lib.ptr(qq), _lib.ptr(kk), _lib.ptr(vv), _lib.ptr(g32), _lib.ptr(b32), _lib.ptr(dvnT), _lib.ptr(d_w),
                    _lib.ptr(d_qt), _lib.ptr(d_kt), _lib.ptr(d_P), _lib.ptr(d_gl), _lib.ptr(dq), _lib.ptr(dk), _lib.ptr(dv),
                    _lib.ptr(dg32), _lib.ptr(db32), c_int(B), c_int(T), c_int(H), c_int(N),
                    ll(qq.stride(0)), ll(qq.stride(1)), ll(qq.stride(2)), ll(kk.stride(0)), ll(kk.stride(1)),
                    ll(kk.stride(2)), ll(vv.stride(0)), ll(vv.stride(1)), ll(vv.stride(2)), ctypes.c_float(scale),
                    c_int(int(self.use_qk_l2norm)), c_int(int(self.gla)), _lib.stream_ptr(q.device))
                _lib.check(rc, "hmf_gdn_prep_bwd")
                dg.copy_(dg32)
                if dbeta is not None:
                    dbeta.copy_(db32)
            return [dq, dk, dv, dg, dbeta], (None if dh0 is None else (dh0,))
        # gradients of the per-chunk factors, then the hand-written backward of the preparation, per head group
        for hs in self._head_groups(B, T, H):
            nh = hs.stop - hs.start
            with torch.no_grad():
                flat = lambda t: t[:, hs].reshape(B * nh, *t.shape[2:])  # noqa: E731
                vnT_g, h_g, dvnT_g, dS_g = flat(vn5), flat(h5), flat(dvn5), flat(dS5)
                do_c = _chunk(do[:, :, hs], N)               # [b*nh, N, C, Dv]
                dvn = dvnT_g.transpose(-1, -2)
                d_u = dvn.float()
                d_w = None if self.gla else -(dvn @ h_g).float()          # [C, Dv] @ [Dv, Dk]
                d_qt = (do_c @ h_g).float()
                d_P = torch.tril((do_c @ vnT_g).float())
                d_kt = (vnT_g.transpose(-1, -2) @ dS_g).float()
                d_gl = torch.exp(flat(gl5)) * (dS_g.float() * h_g.float()).sum((-1, -2))
                sub = [t[:, :, hs] if t is not None else None for t in (q, k, v, g, beta)]
                with _tf32_matmul():
                    gq, gk, gv, gg, gb = self._prep_backward(*sub, d_w, d_qt, d_kt, d_P, d_u, d_gl)
                for dst, src in ((dq, gq), (dk, gk), (dv, gv), (dg, gg), (dbeta, gb)):
                    if dst is not None:
                        _unchunk_into(dst[:, :, hs], src)
                del d_u, d_w, d_qt, d_P, d_kt, d_gl, gq, gk, gv, gg, gb
        return [dq, dk, dv, dg, dbeta], (None if dh0 is None else (dh0,))
