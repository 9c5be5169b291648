"""tcgen05 GEMM vs an fp32 PyTorch reference of the same contraction."""
import pytest
import torch

from hybrid_model_factory_b200.ops.gemm import gemm


def _ref(a, b, a_mn, b_mn):
    am = a.float().t() if a_mn else a.float()
    bm = b.float() if b_mn else b.float().t()
    return am @ bm


def test_gemm_reference_cpu():
    a = torch.randn(33, 40).bfloat16()
    b = torch.randn(17, 40).bfloat16()
    out = gemm(a, b, out_mode="f32")
    torch.testing.assert_close(out, a.float() @ b.float().t())


@pytest.mark.gpu
@pytest.mark.parametrize("pair", [False, True], ids=["cta", "cta_pair"])
@pytest.mark.parametrize("a_mn,b_mn", [(False, False), (False, True), (True, False), (True, True)])
@pytest.mark.parametrize("M,N,K", [(128, 256, 64), (256, 512, 256), (304, 264, 200), (1024, 1024, 4096),
                                   (2048 + 256, 4096 + 40, 512)])
def test_gemm_layouts(a_mn, b_mn, M, N, K, pair):
    dev = "cuda"
    a = torch.randn((K, M) if a_mn else (M, K), device=dev).bfloat16()
    b = torch.randn((K, N) if b_mn else (N, K), device=dev).bfloat16()
    out = gemm(a, b, a_mn_major=a_mn, b_mn_major=b_mn, out_mode="f32", pair=pair)
    ref = _ref(a, b, a_mn, b_mn)
    err = (out - ref).abs().max().item()
    assert err <= 2e-2 * max(1.0, ref.abs().max().item()) * 0.05 + 1e-2, f"max err {err}"
    torch.testing.assert_close(out, ref, rtol=1e-3, atol=1e-2)


@pytest.mark.gpu
def test_gemm_bias_accumulate_bf16_out():
    dev = "cuda"
    a = torch.randn(512, 384, device=dev).bfloat16()
    b = torch.randn(768, 384, device=dev).bfloat16()
    bias = torch.randn(768, device=dev)
    ref = a.float() @ b.float().t() + bias
    out = gemm(a, b, bias=bias)
    torch.testing.assert_close(out.float(), ref, rtol=2e-2, atol=2e-1)
    acc = torch.ones(512, 768, device=dev)
    gemm(a, b, out=acc, out_mode="f32_accumulate")
    torch.testing.assert_close(acc, a.float() @ b.float().t() + 1.0, rtol=1e-3, atol=1e-2)


@pytest.mark.gpu
@pytest.mark.parametrize("T,E,k,Dm,Fi", [(300, 8, 2, 256, 128), (1000, 16, 4, 512, 256), (64, 32, 2, 128, 64)])
def test_moe_experts_grouped_gemm_forward_backward(T, E, k, Dm, Fi):
    """Routed SwiGLU experts on the grouped GEMMs (padded row layout) against the per-expert fp32 formulation,
    outputs and all three gradients; some experts receive no token at all."""
    from hybrid_model_factory_b200.ops import moe
    from hybrid_model_factory_b200.ops import reference as R
    dev = "cuda"
    g = torch.Generator().manual_seed(T + E)
    x = (torch.randn(T, Dm, generator=g) * 0.5).bfloat16().to(dev)
    wgu = (torch.randn(E, 2 * Fi, Dm, generator=g) * 0.05).bfloat16().to(dev)
    wd = (torch.randn(E, Dm, Fi, generator=g) * 0.05).bfloat16().to(dev)
    logits = torch.randn(T, E, generator=g).to(dev)
    logits[:, E - 1] = -1e4                                 # nobody routes to the last expert: an empty group
    w, idx = R.moe_router(logits, k)
    assert moe.grouped_experts_available(x, wgu, wd)
    xs, ws, ds = (t.clone().requires_grad_(True) for t in (x, wgu, wd))
    out = moe.experts_forward(xs, ws, ds, w.to(x.dtype), idx)
    xr, wr, dr = (t.float().clone().requires_grad_(True) for t in (x, wgu, wd))
    ref = R.moe_experts(xr, wr, dr, w, idx)
    rel = lambda a, b: ((a.float() - b.float()).norm() / (b.float().norm() + 1e-9)).item()  # noqa: E731
    assert rel(out, ref) < 2e-2
    do = torch.randn(T, Dm, generator=g).to(dev)
    out.backward(do.bfloat16())
    ref.backward(do)
    assert rel(xs.grad, xr.grad) < 3e-2, "dx"
    assert rel(ws.grad, wr.grad) < 3e-2, "d gate_up"
    assert rel(ds.grad, dr.grad) < 3e-2, "d down"
    assert float(ws.grad[E - 1].abs().max()) == 0.0 and float(ds.grad[E - 1].abs().max()) == 0.0


@pytest.mark.gpu
def test_linear_layer_runs_three_gemms_on_the_library_kernel():
    from hybrid_model_factory_b200.ops import _lib
    from hybrid_model_factory_b200.ops.gemm import Linear, use_own_linear
    lin = torch.nn.Linear(384, 520, bias=True).to("cuda", torch.bfloat16)
    ref = torch.nn.Linear(384, 520, bias=True).to("cuda", torch.float32)
    ref.load_state_dict({k: v.float() for k, v in lin.state_dict().items()})
    holder = torch.nn.Sequential(lin)
    assert use_own_linear(holder) == 1 and type(holder[0]) is Linear
    x = torch.randn(3, 100, 384, device="cuda").bfloat16().requires_grad_(True)
    xr = x.detach().float().requires_grad_(True)
    before = _lib.launch_count()
    y = holder(x)
    dy = torch.randn_like(y)
    y.backward(dy)
    assert _lib.launch_count() - before == 3
    yr = ref(xr)
    yr.backward(dy.float())
    torch.testing.assert_close(y.float(), yr, rtol=2e-2, atol=2e-2)
    torch.testing.assert_close(x.grad.float(), xr.grad, rtol=2e-2, atol=2e-2)
    torch.testing.assert_close(lin.weight.grad.float(), ref.weight.grad, rtol=2e-2, atol=1e-1)
    torch.testing.assert_close(lin.bias.grad.float(), ref.bias.grad, rtol=2e-2, atol=1e-1)


@pytest.mark.gpu
@pytest.mark.parametrize("M,N,K,bias", [(1, 4096, 4096, False), (7, 128, 64, True), (64, 4096, 12288, False),
                                        (100, 512, 4096, True), (16, 19072, 512, True), (127, 1024, 256, False)])
def test_skinny_gemm_decode_rows(M, N, K, bias):
    """Decode-sized products (fewer than 128 rows) run on the swap-AB kernel: direct store with one K split, the
    split reduction through local scratch otherwise; several calls in a row reuse the scratch."""
    from hybrid_model_factory_b200.ops import _lib, gemm as G
    torch.manual_seed(M + N)
    x = torch.randn(M, K, device="cuda").bfloat16()
    w = (torch.randn(N, K, device="cuda") * K ** -0.5).bfloat16()
    b = torch.randn(N, device="cuda").bfloat16() if bias else None
    ref = x.float() @ w.float().t() + (b.float() if bias else 0.0)
    before = _lib.launch_count()
    for _ in range(3):
        y = G.linear(x, w, b)
    torch.cuda.synchronize()
    _lib.assert_status_ok()
    assert _lib.launch_count() - before == 3
    assert ((y.float() - ref).norm() / ref.norm()).item() < 1e-2
    assert (y.float() - ref).abs().max().item() < 0.06 * ref.abs().max().item() + 0.05
