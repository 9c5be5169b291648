"""tcgen05 flash attention (forward and backward) vs the fp32 PyTorch reference."""
import pytest
import torch

from hybrid_model_factory_b200.ops import functional as F_ops
from hybrid_model_factory_b200.ops import reference as R

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _rel(a, b):
    return (a.float() - b.float()).abs().max().item() / max(b.float().abs().max().item(), 1e-6)


CASES = [
    # B, Tq, Tk, Hq, Hkv, D, window, hollow
    (1, 128, 128, 1, 1, 128, None, None),
    (2, 300, 300, 4, 2, 128, None, None),
    (1, 200, 500, 4, 4, 64, None, None),
    (1, 1024, 1024, 8, 2, 128, 100, None),
    (1, 700, 700, 2, 2, 128, None, 64),
    (1, 1000, 1000, 4, 1, 64, 129, None),
    (1, 2048, 2048, 4, 1, 128, None, None),
    (2, 1500, 1500, 4, 2, 256, None, None),       # Qwen3-Next head dimension: forward kernel, blocked backward
    (1, 640, 900, 2, 1, 256, 200, None),
]


@pytest.mark.parametrize("B,Tq,Tk,Hq,Hkv,D,window,hollow", CASES)
def test_attention_fwd_bwd(B, Tq, Tk, Hq, Hkv, D, window, hollow):
    q = torch.randn(B, Tq, Hq, D, device=DEV).bfloat16()
    k = torch.randn(B, Tk, Hkv, D, device=DEV).bfloat16()
    v = torch.randn(B, Tk, Hkv, D, device=DEV).bfloat16()
    qs, ks, vs = (t.clone().requires_grad_(True) for t in (q, k, v))
    qr, kr, vr = (t.float().clone().requires_grad_(True) for t in (q, k, v))
    o, lse = F_ops.attention(qs, ks, vs, window=window, hollow=hollow, return_lse=True)
    orf, lr = R.attention(qr, kr, vr, window=window, hollow=hollow, return_lse=True)
    assert _rel(o, orf) < 2e-2
    fin = torch.isfinite(lr)
    assert bool((torch.isfinite(lse) == fin).all())
    assert (lse[fin] - lr[fin]).abs().max().item() < 2e-2
    do = torch.randn_like(orf)
    # gradient through the log-sum-exp output as well (B'MOJO merges two attention results by their lse)
    dl = torch.where(fin, torch.randn_like(lr), torch.zeros_like(lr))
    torch.autograd.backward([o, lse], [do.bfloat16(), dl])
    torch.autograd.backward([orf, torch.where(fin, lr, torch.zeros_like(lr))], [do, dl])
    assert _rel(qs.grad, qr.grad) < 3e-2, "dq"
    assert _rel(ks.grad, kr.grad) < 3e-2, "dk"
    assert _rel(vs.grad, vr.grad) < 3e-2, "dv"


@pytest.mark.parametrize("Tq,Tk,window", [(2048, 2048, None), (700, 1500, 300), (333, 333, None)])
def test_attention_bwd_fused_matches_two_kernel_path(Tq, Tk, window):
    """D = 128: the single fused backward kernel (dQ by global fp32 reductions) against the dQ + dK/dV pair."""
    from hybrid_model_factory_b200.ops import cuda_ops
    B, Hq, Hkv, D = 2, 8, 2, 128
    q = torch.randn(B, Tq, Hq, D, device=DEV).bfloat16()
    k = torch.randn(B, Tk, Hkv, D, device=DEV).bfloat16()
    v = torch.randn(B, Tk, Hkv, D, device=DEV).bfloat16()
    hi = 2 ** 31 - 1 if window is None else window
    q_off = Tk - Tq
    o, lse = cuda_ops.attention_fwd_raw(q, k, v, D ** -0.5, 0, hi, q_off)
    do = torch.randn_like(o)
    a = cuda_ops.attention_bwd_raw(q, k, v, o, do, lse, D ** -0.5, 0, hi, q_off, deterministic=False)
    b = cuda_ops.attention_bwd_raw(q, k, v, o, do, lse, D ** -0.5, 0, hi, q_off, deterministic=True)
    torch.cuda.synchronize()
    from hybrid_model_factory_b200.ops import _lib
    _lib.assert_status_ok()
    for x, y, name in zip(a, b, ("dq", "dk", "dv")):
        assert _rel(x, y) < 1e-2, name


def test_attention_strided_qkv_views():
    """q, k, v as column slices of one fused projection output (no copies before the kernel)."""
    B, T, Hq, Hkv, D = 1, 512, 8, 2, 128
    qkv = torch.randn(B, T, (Hq + 2 * Hkv) * D, device=DEV).bfloat16()
    q = qkv[..., : Hq * D].view(B, T, Hq, D)
    k = qkv[..., Hq * D:(Hq + Hkv) * D].view(B, T, Hkv, D)
    v = qkv[..., (Hq + Hkv) * D:].view(B, T, Hkv, D)
    o = F_ops.attention(q, k, v)
    assert _rel(o, R.attention(q.float(), k.float(), v.float())) < 2e-2


def test_qsparse_attention():
    B, T, Hq, Hkv, D, Nq = 2, 600, 4, 2, 128, 200
    k = torch.randn(B, T, Hkv, D, device=DEV).bfloat16()
    v = torch.randn(B, T, Hkv, D, device=DEV).bfloat16()
    idx = torch.stack([torch.sort(torch.randperm(T, device=DEV)[:Nq]).values for _ in range(B)])
    q = torch.randn(B, Nq, Hq, D, device=DEV).bfloat16()
    qs, ks, vs = (t.clone().requires_grad_(True) for t in (q, k, v))
    qr, kr, vr = (t.float().clone().requires_grad_(True) for t in (q, k, v))
    o = F_ops.qsparse_attention(qs, ks, vs, idx)
    orf = R.qsparse_attention(qr, kr, vr, idx)
    assert _rel(o, orf) < 2e-2
    do = torch.randn_like(orf)
    o.backward(do.bfloat16())
    orf.backward(do)
    assert _rel(qs.grad, qr.grad) < 3e-2 and _rel(ks.grad, kr.grad) < 3e-2 and _rel(vs.grad, vr.grad) < 3e-2
