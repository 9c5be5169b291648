"""Memory-bound CUDA kernels vs fp32 PyTorch references (forward and backward)."""
import pytest
import torch

from hybrid_model_factory_b200.ops import functional as F_ops
from hybrid_model_factory_b200.ops import reference as R

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _close(a, b, rtol=2e-2, atol=2e-2, name=""):
    a, b = a.float(), b.float()
    err = (a - b).abs().max().item()
    ref = b.abs().max().item()
    assert err <= atol + rtol * ref, f"{name}: max err {err} vs ref max {ref}"


def _grad_pair(fn_cuda, fn_ref, inputs, names):
    """inputs: bf16 leaves. Runs both paths with the same upstream gradient."""
    xs = [t.clone().requires_grad_(True) for t in inputs]
    xr = [t.float().clone().requires_grad_(True) for t in inputs]
    y, yr = fn_cuda(*xs), fn_ref(*xr)
    _close(y, yr, name="forward")
    dy = torch.randn_like(yr)
    y.backward(dy.to(y.dtype))
    yr.backward(dy)
    for n, a, b in zip(names, xs, xr):
        _close(a.grad, b.grad, rtol=3e-2, atol=3e-2 * max(1.0, b.grad.abs().max().item()) * 0.5, name=f"d{n}")


@pytest.mark.parametrize("N,D,zc", [(1000, 4096, False), (4096 * 4, 128, False), (513, 2048, True), (2100, 4096, True), (3, 8192, False)])
def test_rms_norm(N, D, zc):
    x = torch.randn(N, D, device=DEV).bfloat16()
    w = (torch.randn(D, device=DEV) * 0.1 + (0 if zc else 1)).bfloat16()
    _grad_pair(lambda a, b: F_ops.rms_norm(a, b, 1e-6, zc), lambda a, b: R.rms_norm(a, b, 1e-6, zc), [x, w], ["x", "w"])


def test_fused_add_rms_norm():
    x, r = torch.randn(300, 1024, device=DEV).bfloat16(), torch.randn(300, 1024, device=DEV).bfloat16()
    w = torch.randn(1024, device=DEV).bfloat16()
    with torch.no_grad():
        y, ro = F_ops.fused_add_rms_norm(x, r, w, 1e-6)
        yr, rr = R.fused_add_rms_norm(x.float(), r.float(), w.float(), 1e-6)
    _close(ro, rr)
    _close(y, yr, atol=5e-2)


@pytest.mark.parametrize("D,H,mode,perhead", [(128, 32, True, False), (64, 8, False, True), (128, 4, False, True),
                                              (256, 2, True, False)])
def test_gated_norm(D, H, mode, perhead):
    x = torch.randn(2, 333, H, D, device=DEV).bfloat16()
    g = torch.randn(2, 333, H, D, device=DEV).bfloat16()
    w = (torch.randn((H, D) if perhead else (D,), device=DEV) * 0.2 + 1).bfloat16()
    _grad_pair(lambda a, b, c: F_ops.gated_rms_norm(a, b, c, 1e-5, mode),
               lambda a, b, c: R.gated_rms_norm(a, b, c, 1e-5, mode), [x, g, w], ["x", "gate", "w"])


def test_swiglu():
    g, u = torch.randn(777, 1536, device=DEV).bfloat16(), torch.randn(777, 1536, device=DEV).bfloat16()
    _grad_pair(F_ops.swiglu, R.swiglu, [g, u], ["g", "u"])


@pytest.mark.parametrize("D,Rr", [(128, 128), (256, 64), (64, 64)])
def test_rope(D, Rr):
    B, T, H = 2, 200, 6
    x = torch.randn(B, T, H, D, device=DEV).bfloat16()
    pos = torch.arange(T, device=DEV).expand(B, T)
    cos, sin = R.rope_tables(pos, Rr, 1e6)
    xs = x.clone().requires_grad_(True)
    xr = x.float().clone().requires_grad_(True)
    y = F_ops.apply_rope(xs, cos.bfloat16(), sin.bfloat16())
    yr = R.apply_rope(xr, cos.bfloat16().float(), sin.bfloat16().float())
    _close(y, yr)
    dy = torch.randn_like(yr)
    y.backward(dy.bfloat16())
    yr.backward(dy)
    _close(xs.grad, xr.grad)


def test_rope_strided_view():
    B, T, H, D = 1, 64, 4, 128
    big = torch.randn(B, T, H, 2 * D, device=DEV).bfloat16()
    x = big[..., :D].reshape(B, T, H * D)  # forces a copy; the kernel path sees contiguous data
    pos = torch.arange(T, device=DEV).expand(B, T)
    cos, sin = R.rope_tables(pos, D, 1e4)
    y = F_ops.apply_rope(x.view(B, T, H, D), cos.bfloat16(), sin.bfloat16())
    _close(y, R.apply_rope(x.view(B, T, H, D).float(), cos.bfloat16().float(), sin.bfloat16().float()))


@pytest.mark.parametrize("T,C,with_init,with_bias", [(200, 256, True, False), (64, 6144, False, True), (3, 64, True, True),
                                                     (1000, 1024, True, True)])
def test_conv1d(T, C, with_init, with_bias):
    B = 2
    x = torch.randn(B, T, C, device=DEV).bfloat16()
    w = (torch.randn(C, 4, device=DEV) * 0.5).bfloat16()
    ins, names = [x, w], ["x", "w"]
    if with_bias:
        ins.append(torch.randn(C, device=DEV).bfloat16())
        names.append("bias")
    if with_init:
        ins.append(torch.randn(B, 3, C, device=DEV).bfloat16())
        names.append("init")

    def unpack(args):
        a = list(args)
        xx, ww = a[0], a[1]
        bb = a[2] if with_bias else None
        ii = a[-1] if with_init else None
        return xx, ww, bb, ii

    def f_cuda(*a):
        xx, ww, bb, ii = unpack(a)
        return F_ops.causal_conv1d(xx, ww, bb, "silu", ii)

    def f_ref(*a):
        xx, ww, bb, ii = unpack(a)
        return R.causal_conv1d(xx, ww, bb, "silu", ii)

    _grad_pair(f_cuda, f_ref, ins, names)
    y, st = F_ops.causal_conv1d(x, w, None, "silu", None, True)
    yr, sr = R.causal_conv1d(x.float(), w.float(), None, "silu", None, True)
    _close(st, sr)


def test_conv1d_update():
    B, C = 5, 512
    x = torch.randn(B, C, device=DEV).bfloat16()
    st = torch.randn(B, 3, C, device=DEV).bfloat16()
    w, b = torch.randn(C, 4, device=DEV).bfloat16(), torch.randn(C, device=DEV).bfloat16()
    yr, sr = R.causal_conv1d_update(x.float(), st.float(), w.float(), b.float())
    y, s2 = F_ops.causal_conv1d_update(x, st.clone(), w, b)
    _close(y, yr)
    _close(s2, sr)


@pytest.mark.parametrize("N,V,Dm,chunk", [(300, 1024, 256, 128), (1000, 5000 - 8, 512, 4096)])
def test_linear_cross_entropy(N, V, Dm, chunk):
    h = (torch.randn(N, Dm, device=DEV) * 0.5).bfloat16().requires_grad_(True)
    w = (torch.randn(V, Dm, device=DEV) * 0.05).bfloat16().requires_grad_(True)
    y = torch.randint(0, V, (N,), device=DEV)
    y[::7] = -100
    loss, n = F_ops.linear_cross_entropy(h, w, y, chunk=chunk)
    hr, wr = h.detach().float().requires_grad_(True), w.detach().float().requires_grad_(True)
    lr = torch.nn.functional.cross_entropy(hr @ wr.t(), y, ignore_index=-100, reduction="sum")
    assert n.item() == (y != -100).sum().item()
    assert abs(loss.item() - lr.item()) / lr.item() < 5e-3
    (loss / n).backward()
    (lr / n).backward()
    _close(h.grad, hr.grad, rtol=5e-2, atol=1e-4)
    _close(w.grad, wr.grad, rtol=5e-2, atol=1e-4)


@pytest.mark.parametrize("pdt,sdt", [(torch.bfloat16, torch.bfloat16), (torch.bfloat16, torch.float32),
                                     (torch.float32, torch.float32)])
def test_adamw_and_norm(pdt, sdt):
    from hybrid_model_factory_b200.ops import cuda_ops
    n = 100003
    p0 = torch.randn(n, device=DEV)
    g = torch.randn(n, device=DEV) * 3
    p = p0.to(pdt).clone()
    gq = g.to(pdt)
    m, v = torch.zeros(n, device=DEV, dtype=sdt), torch.zeros(n, device=DEV, dtype=sdt)
    nsq = torch.zeros(1, device=DEV)
    cuda_ops.grad_sumsq(gq, nsq)
    assert abs(nsq.item() - gq.float().pow(2).sum().item()) / nsq.item() < 1e-3
    ref_p = p.float().clone().requires_grad_(True)
    opt = torch.optim.AdamW([ref_p], lr=1e-2, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1)
    coef = min(1.0, 1.0 / (nsq.sqrt().item() + 1e-6))
    for step in range(1, 4):
        ref_p.grad = gq.float() * coef
        opt.step()
        cuda_ops.adamw_step(p, gq, m, v, lr=1e-2, beta1=0.9, beta2=0.95, eps=1e-8, weight_decay=0.1, step=step,
                            norm_sq=nsq, max_norm=1.0)
    tol = 3e-2 if pdt == torch.bfloat16 else 1e-4
    _close(p, ref_p.detach(), rtol=tol, atol=tol)


@pytest.mark.gpu
def test_zero3_engine_on_gpu_uses_the_fused_adamw_and_matches_torch_adamw():
    """One rank on the GPU: ZeRO-3 hooks (gather / release around each layer, gradient flattening) with the fused
    AdamW kernel on the shards, against torch.optim.AdamW on a copy of the model."""
    import copy
    from hybrid_model_factory_b200.models.configuration import HybridConfig
    from hybrid_model_factory_b200.models.modeling_hybrid import build_model
    from hybrid_model_factory_b200.train.zero3 import Zero3Engine
    torch.manual_seed(0)
    cfg = HybridConfig("hybrid_qwen3", vocab_size=256, hidden_size=256, intermediate_size=512, num_hidden_layers=2,
                       num_attention_heads=2, num_key_value_heads=2, head_dim=128, hybrid_override_pattern="*-GDN")
    model = build_model(cfg).to("cuda", torch.float32)
    ref = copy.deepcopy(model)
    model.gradient_checkpointing_enable()
    eng = Zero3Engine(model, lr=1e-3, weight_decay=0.1, max_grad_norm=1.0)
    decay = [p for p in ref.parameters() if p.dim() >= 2 and not getattr(p, "_no_weight_decay", False)]
    rest = [p for p in ref.parameters() if not (p.dim() >= 2 and not getattr(p, "_no_weight_decay", False))]
    opt = torch.optim.AdamW([{"params": decay, "weight_decay": 0.1}, {"params": rest, "weight_decay": 0.0}], lr=1e-3)
    for _ in range(3):
        ids = torch.randint(0, 256, (2, 64), device="cuda")
        opt.zero_grad()
        ref.train()
        ref(input_ids=ids, labels=ids).loss.backward()
        torch.nn.utils.clip_grad_norm_(ref.parameters(), 1.0)
        opt.step()
        eng.zero_grad()
        model.train()
        model(input_ids=ids, labels=ids).loss.backward()
        assert eng.parameter_bytes_resident() == 0
        eng.step()
    eng.gather_full_state()
    for (n, p), q in zip(model.named_parameters(), ref.parameters()):
        assert torch.allclose(p, q, atol=5e-4, rtol=5e-3), (n, float((p - q).abs().max()))


@pytest.mark.gpu
@pytest.mark.parametrize("pattern", ["*-M2", "*-GDN"])
def test_inference_fusions_match_the_autograd_path(pattern):
    """Without an autograd graph the layers take fused kernels (per-head norm + rotary in one launch, residual add +
    norm, segment-parallel GLA scan); the logits must agree with the path that records a graph."""
    from hybrid_model_factory_b200.models.configuration import HybridConfig
    from hybrid_model_factory_b200.models.modeling_hybrid import build_model
    torch.manual_seed(0)
    cfg = HybridConfig("hybrid_qwen3", vocab_size=512, hidden_size=512, intermediate_size=1024, num_hidden_layers=2,
                       num_attention_heads=4, num_key_value_heads=2, head_dim=128, hybrid_override_pattern=pattern)
    model = build_model(cfg).to("cuda", torch.bfloat16).eval()
    ids = torch.randint(0, 512, (1, 2304), device="cuda")
    with torch.no_grad():
        fused = model(ids).logits.float()
    plain = model(ids).logits.float().detach()
    assert torch.isfinite(fused).all()
    err = (fused - plain).abs().max() / plain.abs().max()
    assert err < 3e-2, float(err)
    assert (fused.argmax(-1) == plain.argmax(-1)).float().mean() > 0.97


@pytest.mark.gpu
def test_device_timer_and_step_breakdown_on_gpu():
    from hybrid_model_factory_b200.models.configuration import HybridConfig
    from hybrid_model_factory_b200.models.modeling_hybrid import build_model
    from hybrid_model_factory_b200.utils import profiling
    cfg = HybridConfig("hybrid_qwen3", vocab_size=256, hidden_size=256, intermediate_size=512, num_hidden_layers=2,
                       num_attention_heads=2, num_key_value_heads=2, head_dim=128, hybrid_override_pattern="*-GDN")
    model = build_model(cfg).to("cuda", torch.bfloat16)
    sb = profiling.StepBreakdown(model)
    t = profiling.DeviceTimer()
    with t.time("forward"), profiling.nvtx_range("forward"):
        model(torch.randint(0, 256, (1, 256), device="cuda"))
    s = sb.summary()
    sb.remove()
    assert {"Attention", "GatedDeltaNetLayer", "MLP"} <= set(s) and s["MLP"]["calls"] == 2
    total = t.summary()["forward"]["total_ms"]
    assert total > 0 and sum(v["total_ms"] for v in s.values()) <= total * 1.05


@pytest.mark.gpu
@pytest.mark.parametrize("D,with_beta", [(128, True), (64, True), (256, False), (128, False)])
def test_gka_prepare_matches_reference(D, with_beta):
    """Fused q / k normalisation + beta scaling against the fp32 PyTorch formulation, values and gradients."""
    from hybrid_model_factory_b200.ops import _lib, cuda_ops
    from hybrid_model_factory_b200.ops import reference as R
    torch.manual_seed(D)
    B, T, H = 2, 300, 4
    q, k, v = (torch.randn(B, T, H, D, device="cuda").bfloat16().requires_grad_(True) for _ in range(3))
    beta = torch.rand(B, T, H, device="cuda").bfloat16().requires_grad_(True) if with_beta else None
    before = _lib.launch_count()
    outs = cuda_ops.gka_prepare(q, k, v, beta, 1e-6)
    gs = [torch.randn_like(o) for o in outs]
    torch.autograd.backward(outs, gs)
    assert _lib.launch_count() - before == 2
    got = [q.grad, k.grad, v.grad] + ([beta.grad] if with_beta else [])
    qf, kf, vf = (t.detach().float().requires_grad_(True) for t in (q, k, v))
    bf = beta.detach().float().requires_grad_(True) if with_beta else None
    refs = R.gka_prepare(qf, kf, vf, bf, 1e-6)
    torch.autograd.backward(refs, [g.float() for g in gs])
    want = [qf.grad, kf.grad, vf.grad] + ([bf.grad] if with_beta else [])
    for o, r in zip(outs, refs):
        assert (o.float() - r).abs().max() < 2e-2 * r.abs().max() + 1e-3
    for g, w in zip(got, want):
        rel = (g.float() - w).norm() / (w.norm() + 1e-12)
        assert rel < 2e-2, float(rel)
    torch.cuda.synchronize()
    _lib.assert_status_ok()
