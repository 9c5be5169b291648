"""Gated delta rule on the GPU (chunk preparation + tcgen05 scan kernels) vs the fp32 reference."""
import pytest
import torch

from hybrid_model_factory_b200.ops import mixers
from hybrid_model_factory_b200.ops import reference as R

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _rel(a, b):
    return (a.float() - b.float()).abs().max().item() / max(b.float().abs().max().item(), 1e-6)


def _inputs(B, T, H, D=128):
    q = torch.randn(B, T, H, D, device=DEV).bfloat16()
    k = torch.randn(B, T, H, D, device=DEV).bfloat16()
    v = torch.randn(B, T, H, D, device=DEV).bfloat16()
    g = (-torch.rand(B, T, H, device=DEV) * 0.1).float()
    beta = torch.rand(B, T, H, device=DEV).float()
    return q, k, v, g, beta


@pytest.mark.parametrize("B,T,H,with_h0", [(1, 64, 1, False), (2, 256, 3, True), (1, 1000, 2, True), (1, 4096, 4, False)])
def test_gdn_forward_backward(B, T, H, with_h0):
    q, k, v, g, beta = _inputs(B, T, H)
    h0 = (torch.randn(B, H, 128, 128, device=DEV) * 0.1) if with_h0 else None
    leaves = [t.clone().requires_grad_(True) for t in (q, k, v, g, beta)]
    refs = [t.float().clone().requires_grad_(True) for t in (q, k, v, g, beta)]
    h0c = h0.clone().requires_grad_(True) if with_h0 else None
    h0r = h0.clone().requires_grad_(True) if with_h0 else None
    o, s = mixers.gated_delta_rule(*leaves, initial_state=h0c)
    orf, sr = R.gated_delta_rule_chunk(*refs, initial_state=h0r)
    assert _rel(o, orf) < 3e-2, f"o {_rel(o, orf)}"
    assert _rel(s, sr) < 3e-2, f"state {_rel(s, sr)}"
    do = torch.randn_like(orf)
    ds = torch.randn_like(sr) * 0.1
    (o.float() * do).sum().backward(retain_graph=True) if False else None
    torch.autograd.backward([o, s], [do.to(o.dtype), ds])
    torch.autograd.backward([orf, sr], [do, ds])
    names = ["q", "k", "v", "g", "beta"]
    for n, a, b in zip(names, leaves, refs):
        assert _rel(a.grad, b.grad) < 5e-2, f"d{n}: {_rel(a.grad, b.grad)}"
    if with_h0:
        assert _rel(h0c.grad, h0r.grad) < 5e-2, "dh0"


def test_gdn_state_split_equals_full():
    q, k, v, g, beta = _inputs(1, 512, 2)
    with torch.no_grad():
        o, s = mixers.gated_delta_rule(q, k, v, g, beta)
        oa, sa = mixers.gated_delta_rule(q[:, :256], k[:, :256], v[:, :256], g[:, :256], beta[:, :256])
        ob, sb = mixers.gated_delta_rule(q[:, 256:], k[:, 256:], v[:, 256:], g[:, 256:], beta[:, 256:], initial_state=sa)
    assert _rel(torch.cat([oa, ob], 1), o) < 2e-2
    assert _rel(sb, s) < 2e-2


def test_gdn_prep_kernel_matches_torch_prep():
    """The chunk-preparation kernel reproduces the batched PyTorch formulation of the same factors."""
    from hybrid_model_factory_b200.ops import gdn_cuda
    q, k, v, g, beta = _inputs(2, 300, 3)
    core = gdn_cuda.GDNChunkCore()
    a = core._prep_packed(q, k, v, g, beta)
    old = gdn_cuda._FORCE_TORCH_PREP
    gdn_cuda._FORCE_TORCH_PREP = True
    try:
        b = core._prep_packed(q, k, v, g, beta)
    finally:
        gdn_cuda._FORCE_TORCH_PREP = old
    for name, x, y in zip(["wqT", "kPT", "uT", "glast"], a[:4], b[:4]):
        assert _rel(x, y) < 2e-2, f"{name}: {_rel(x, y)}"


def test_simple_gla_kernel_mode():
    q, k, v, g, _ = _inputs(2, 500, 3)
    q = (q.float() * 0.3).bfloat16()
    h0 = torch.randn(2, 3, 128, 128, device=DEV) * 0.1
    leaves = [t.clone().requires_grad_(True) for t in (q, k, v, g)]
    refs = [t.float().clone().requires_grad_(True) for t in (q, k, v, g)]
    o, s = mixers.simple_gla(*leaves, scale=0.1, initial_state=h0)
    orf, sr = R.simple_gla_chunk(*refs, scale=0.1, initial_state=h0)
    assert _rel(o, orf) < 3e-2 and _rel(s, sr) < 3e-2
    do = torch.randn_like(orf)
    torch.autograd.backward([o], [do.to(o.dtype)])
    torch.autograd.backward([orf], [do])
    for n, a, b in zip("qkvg", leaves, refs):
        assert _rel(a.grad, b.grad) < 5e-2, f"d{n}: {_rel(a.grad, b.grad)}"


def test_ssd_matches_reference():
    B, T, H, P, G, N = 1, 700, 4, 128, 4, 128
    x = torch.randn(B, T, H, P, device=DEV).bfloat16()
    dt = torch.rand(B, T, H, device=DEV) * 0.3
    A = -torch.rand(H, device=DEV)
    Bm = (torch.randn(B, T, G, N, device=DEV) * 0.3).bfloat16()
    Cm = (torch.randn(B, T, G, N, device=DEV) * 0.3).bfloat16()
    Dp = torch.randn(H, device=DEV)
    h0 = torch.randn(B, H, P, N, device=DEV) * 0.1
    y, s = mixers.ssd(x, dt, A, Bm, Cm, Dp, initial_state=h0)
    yr, sr = R.ssd_chunk(x.float(), dt, A, Bm.float(), Cm.float(), Dp, initial_state=h0, chunk_size=64)
    assert _rel(y, yr) < 3e-2, _rel(y, yr)
    assert _rel(s, sr) < 3e-2, _rel(s, sr)


@pytest.mark.gpu
@pytest.mark.parametrize("P,N,H,G", [(64, 128, 8, 2), (128, 64, 4, 4), (32, 64, 4, 1)])
def test_ssd_narrow_heads_forward_backward(P, N, H, G):
    """Mamba2 shapes whose head_dim / d_state are not 128 (e.g. 64 heads x 64 with d_state 128 in groups): padded to
    the kernel width, forward and backward against the fp32 chunked formulation."""
    from hybrid_model_factory_b200.ops import _lib
    B, T = 2, 520
    x = torch.randn(B, T, H, P, device=DEV).bfloat16()
    dt = torch.rand(B, T, H, device=DEV) * 0.3
    A = -torch.rand(H, device=DEV)
    Bm = (torch.randn(B, T, G, N, device=DEV) * 0.3).bfloat16()
    Cm = (torch.randn(B, T, G, N, device=DEV) * 0.3).bfloat16()
    h0 = torch.randn(B, H, P, N, device=DEV) * 0.1
    xs, dts, Bs, Cs, hs = (t.clone().requires_grad_(True) for t in (x, dt, Bm, Cm, h0))
    xr, dtr, Br, Cr, hr = (t.float().clone().requires_grad_(True) for t in (x, dt, Bm, Cm, h0))
    before = _lib.launch_count()
    y, s = mixers.ssd(xs, dts, A, Bs, Cs, None, initial_state=hs)
    assert _lib.launch_count() > before, "the padded problem must run on the kernels"
    yr, sr = R.ssd_chunk(xr, dtr, A, Br, Cr, None, initial_state=hr, chunk_size=64)
    assert y.shape == (B, T, H, P) and s.shape == (B, H, P, N)
    assert _rel(y, yr) < 3e-2 and _rel(s, sr) < 3e-2
    dy, ds = torch.randn_like(yr), torch.randn_like(sr) * 0.1
    torch.autograd.backward([y.float(), s], [dy, ds])
    torch.autograd.backward([yr, sr], [dy, ds])
    for a, b, name in ((xs, xr, "dx"), (dts, dtr, "ddt"), (Bs, Br, "dB"), (Cs, Cr, "dC"), (hs, hr, "dh0")):
        assert _rel(a.grad, b.grad) < 6e-2, (name, _rel(a.grad, b.grad))


@pytest.mark.gpu
@pytest.mark.parametrize("T,with_state,with_gate", [(256, False, True), (200, True, True), (128, True, False)])
def test_gka_chebyshev_kernel_matches_fp32_formulation(T, with_state, with_gate):
    """The one-kernel Chebyshev solve (bf16 operands, fp32 accumulation) against the batched fp32 PyTorch solve."""
    from hybrid_model_factory_b200.ops import _lib
    from hybrid_model_factory_b200.ops import gka_parallel as GP
    torch.manual_seed(0)
    B, H, D = 2, 3, 128
    q = torch.randn(B, T, H, D, device="cuda")
    k = torch.nn.functional.normalize(torch.randn(B, T, H, D, device="cuda"), dim=-1)
    gk = -torch.rand(B, T, H, device="cuda") * 0.2 if with_gate else None
    h0 = None
    if with_state:
        a = torch.randn(B, H, D, 32, device="cuda") * 0.3
        h0 = a @ a.transpose(-1, -2)
    qb, kb = q.bfloat16(), k.bfloat16()
    with torch.no_grad():
        x_k, hT_k = GP.chebyshev_chunk_parallel(qb, kb, gk, ridge_ratio=0.02, num_iter=30, initial_state=h0)
        assert GP._kernel_ok(qb, kb, gk, 64)
        x_r, hT_r = GP.chebyshev_chunk_parallel(qb.float(), kb.float(), gk, ridge_ratio=0.02, num_iter=30,
                                                initial_state=h0)
    torch.cuda.synchronize()
    _lib.assert_status_ok()
    assert x_k.shape == x_r.shape and torch.isfinite(x_k).all()
    err = (x_k - x_r).norm() / x_r.norm()
    assert err < 2e-2, float(err)
    assert torch.allclose(hT_k, hT_r, atol=1e-4, rtol=1e-4)


@pytest.mark.gpu
def test_gka_chebyshev_implicit_backward_matches_autograd_through_the_iteration():
    """ChebyshevCore's backward (adjoint solve + GLA form + |H|_F closed form) against differentiating the fp32
    PyTorch iteration; enough iterations that both solves have converged."""
    from hybrid_model_factory_b200.ops import gka_parallel as GP
    from hybrid_model_factory_b200.ops.scan import ssm_scan
    torch.manual_seed(0)
    B, T, H, D = 1, 192, 2, 128
    q = torch.randn(B, T, H, D, device="cuda")
    k = torch.nn.functional.normalize(torch.randn(B, T, H, D, device="cuda"), dim=-1)
    gk = -torch.rand(B, T, H, device="cuda") * 0.2
    a = torch.randn(B, H, D, 16, device="cuda") * 0.3
    h0 = a @ a.transpose(-1, -2)
    w = torch.randn(B, T, H, D, device="cuda")
    wh = torch.randn(B, H, D, D, device="cuda") * 0.01
    wh = wh + wh.transpose(-1, -2)
    iters = 80
    # reference: fp32 autograd through the batched iteration
    qr, kr, gr, hr = (t.clone().requires_grad_(True) for t in (q, k, gk, h0))
    x_r, hT_r = GP.chebyshev_chunk_parallel(qr, kr, gr, ridge_ratio=0.05, num_iter=iters, initial_state=hr)
    ((x_r * w).sum() + (hT_r * wh).sum()).backward()
    # kernel core
    qk = q.bfloat16().requires_grad_(True)
    kk = k.bfloat16().requires_grad_(True)
    gkk = gk.clone().requires_grad_(True)
    hk = h0.clone().requires_grad_(True)
    core = GP.ChebyshevCore(0.05, iters)
    assert core.supported(qk, kk, gkk, 64)
    x_k, (hT_k,) = ssm_scan(core, [qk, kk, gkk], (hk,), None)
    ((x_k * w).sum() + (hT_k * wh).sum()).backward()

    def rel(a, b):
        return float((a.float() - b.float()).norm() / b.float().norm())
    assert rel(x_k, x_r) < 3e-2
    assert rel(qk.grad, qr.grad) < 5e-2, rel(qk.grad, qr.grad)
    assert rel(kk.grad, kr.grad) < 8e-2, rel(kk.grad, kr.grad)
    assert rel(gkk.grad, gr.grad) < 8e-2, rel(gkk.grad, gr.grad)
    assert rel(hk.grad, hr.grad) < 8e-2, rel(hk.grad, hr.grad)


@pytest.mark.gpu
@pytest.mark.parametrize("T,H,with_state", [(5000, 4, True), (4096, 8, False), (2500, 2, True)])
def test_gla_segment_parallel_inference_scan_matches_sequential(T, H, with_state):
    """Few heads, one long sequence: the segment-parallel forward (two batched scans + state prefix + tail) against
    the one-CTA-per-head scan of the same kernels."""
    from hybrid_model_factory_b200.ops import gdn_cuda
    torch.manual_seed(0)
    D = 128
    q, k, v = (torch.randn(1, T, H, D, device="cuda").bfloat16() * 0.5 for _ in range(3))
    g = -torch.rand(1, T, H, device="cuda") * 0.05
    s0 = (torch.randn(1, H, D, D, device="cuda") * 0.1,) if with_state else None
    core = gdn_cuda.GDNChunkCore(scale=D ** -0.5, use_qk_l2norm=False, gla=True)
    with torch.no_grad():
        o_seg, (h_seg,), _, _ = core.forward((q, k, v, g, None), s0)
        old = gdn_cuda._GLA_SEGMENTS
        gdn_cuda._GLA_SEGMENTS = False
        try:
            o_ref, (h_ref,), _, _ = core.forward((q, k, v, g, None), s0)
        finally:
            gdn_cuda._GLA_SEGMENTS = old
    torch.cuda.synchronize()
    assert (o_seg.float() - o_ref.float()).abs().max() < 2e-2 * o_ref.float().abs().max() + 1e-2
    assert (h_seg - h_ref).abs().max() < 2e-2 * h_ref.abs().max() + 1e-2


@pytest.mark.gpu
@pytest.mark.parametrize("with_h0", [False, True])
def test_gka_chunk_states_prefix_kernel_with_gradients(with_h0):
    """Chunk-start states of the key covariance: the decayed prefix-sum kernel (forward, and backward on the flipped
    sequence) against the quadratic weight-product formulation on the CPU in fp64."""
    from hybrid_model_factory_b200.ops import _lib
    from hybrid_model_factory_b200.ops.gka_parallel import chunk_states
    torch.manual_seed(3)
    B, H, N, C, D = 1, 3, 9, 16, 32
    k = (torch.randn(B, H, N, C, D) * 0.3)
    G = torch.cumsum(-torch.rand(B, H, N, C) * 0.1, dim=-1)
    H0 = torch.randn(B, H, D, D) * 0.2 if with_h0 else None
    leaves_ref = [t.double().requires_grad_(True) if t is not None else None for t in (k, G, H0)]
    ref = chunk_states(*leaves_ref)                      # CPU: the weight-product formulation
    w = torch.randn_like(ref)
    (ref * w).sum().backward()
    leaves = [t.cuda().requires_grad_(True) if t is not None else None for t in (k, G, H0)]
    before = _lib.launch_count()
    out = chunk_states(*leaves)
    (out * w.cuda().float()).sum().backward()
    assert _lib.launch_count() - before == 2             # one prefix pass each way
    assert (out.double().cpu() - ref).abs().max() < 1e-4 * ref.abs().max() + 1e-5
    for a, b in zip(leaves, leaves_ref):
        if a is not None:
            err = (a.grad.double().cpu() - b.grad).norm() / (b.grad.norm() + 1e-12)
            assert err < 1e-4, float(err)
    torch.cuda.synchronize()
    _lib.assert_status_ok()
