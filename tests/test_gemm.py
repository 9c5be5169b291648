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
@pytest.mark.parametrize("a_mn,b_mn", [(False, False), (False, True), (True, False), (True, True)])
@pytest.mark.parametrize("M,N,K", [(128, 256, 64), (256, 512, 256), (304, 264, 200), (1024, 1024, 4096)])
def test_gemm_layouts(a_mn, b_mn, M, N, K):
    dev = "cuda"
    a = torch.randn((K, M) if a_mn else (M, K), device=dev).bfloat16()
    b = torch.randn((K, N) if b_mn else (N, K), device=dev).bfloat16()
    out = gemm(a, b, a_mn_major=a_mn, b_mn_major=b_mn, out_mode="f32")
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
