"""Row-wise scaled float8 linear layers: quantisers and GEMM against their PyTorch formulation, the layer against
a bf16 / fp32 linear, and the ``fp8: true`` switch of the training workflow."""
import json

import pytest
import torch

from hybrid_model_factory_b200.ops import fp8


def test_fp8_reference_path_and_module_filter():
    torch.manual_seed(0)
    x = torch.randn(64, 128)
    q, s = fp8.quant_rows(x)
    assert q.dtype == torch.uint8 and (fp8.dequant(q, s) - x).abs().max() < 0.07 * x.abs().max()
    qt, st = fp8.quant_cols_t(x)
    assert qt.shape == (128, 64) and (fp8.dequant(qt, st).t() - x).abs().max() < 0.07 * x.abs().max()
    from hybrid_model_factory_b200.models.configuration import HybridConfig
    from hybrid_model_factory_b200.models.modeling_hybrid import build_model
    cfg = HybridConfig("hybrid_qwen3", vocab_size=128, hidden_size=64, intermediate_size=128, num_hidden_layers=2,
                       num_attention_heads=4, num_key_value_heads=2, head_dim=16, hybrid_override_pattern="*-GDN")
    model = build_model(cfg)
    n = fp8.use_fp8_linear(model)
    names = [k for k, m in model.named_modules() if isinstance(m, fp8.Fp8Linear)]
    assert n == len(names) > 0 and not any("lm_head" in k for k in names)
    assert not isinstance(model.model.layers[1].gdn.b_proj, fp8.Fp8Linear)      # 4 output features: not a multiple of 16
    ids = torch.randint(0, 128, (2, 32))
    out = model(ids, labels=ids)
    out.loss.backward()
    assert torch.isfinite(out.loss) and model.model.layers[0].mlp.up_proj.weight.grad.abs().sum() > 0


def test_fp8_flag_in_the_training_workflow(tmp_path):
    from hybrid_model_factory_b200.train.workflow import run_exp
    tiny = {"model_type": "hybrid_qwen3", "vocab_size": 259, "hidden_size": 32, "intermediate_size": 64,
            "num_hidden_layers": 2, "num_attention_heads": 2, "num_key_value_heads": 1, "head_dim": 16,
            "hybrid_override_pattern": "*-GDN", "torch_dtype": "float32"}
    tr = run_exp({"model_name_or_path": json.dumps(tiny), "stage": "pt", "synthetic": True, "cutoff_len": 32,
                  "max_steps": 2, "output_dir": str(tmp_path), "bf16": False, "pure_bf16": False, "fp8": True,
                  "per_device_train_batch_size": 2})
    assert tr.global_step == 2 and any(isinstance(m, fp8.Fp8Linear) for m in tr.model.modules())


@pytest.mark.gpu
@pytest.mark.parametrize("R,C", [(300, 512), (4096, 1024), (17, 48)])
def test_fp8_quantisers_match_reference(R, C):
    x = (torch.randn(R, C, device="cuda") * torch.rand(R, 1, device="cuda") * 3).bfloat16()
    for fmt in (fp8.E4M3, fp8.E5M2):
        q, s = fp8.quant_rows(x, fmt)
        qr, sr = fp8.quant_rows(x.float().cpu(), fmt)
        torch.testing.assert_close(s.cpu(), sr, rtol=1e-5, atol=0)
        # the kernel multiplies by the reciprocal scale, the formulation divides: values on a rounding boundary may
        # land one code apart (one step is 1/8 of the binade for e4m3, 1/4 for e5m2), the rest must agree exactly
        diff = (fp8.dequant(q, s, fmt).cpu() - fp8.dequant(qr, sr, fmt)).abs()
        assert (q.cpu() != qr).float().mean() < 0.01
        assert diff.max() <= (0.13 if fmt == fp8.E4M3 else 0.26) * x.abs().max().item()
        if R % 16 == 0:
            qt, st = fp8.quant_cols_t(x, fmt)
            qtr, str_ = fp8.quant_cols_t(x.float().cpu(), fmt)
            torch.testing.assert_close(st.cpu(), str_, rtol=1e-5, atol=0)
            assert (qt.cpu() != qtr).float().mean() < 0.01          # rounding ties aside, the same codes


@pytest.mark.gpu
@pytest.mark.parametrize("M,N,K", [(256, 256, 128), (1000, 520, 384), (4096, 4096, 4096)])
def test_fp8_gemm_matches_dequantised_product(M, N, K):
    a = torch.randn(M, K, device="cuda").bfloat16()
    b = (torch.randn(N, K, device="cuda") * 0.05).bfloat16()
    aq, sa = fp8.quant_rows(a)
    bq, sb = fp8.quant_rows(b, fp8.E5M2)
    out = fp8.gemm_fp8(aq, sa, bq, sb, fp8.E4M3, fp8.E5M2, out_dtype=torch.float32)
    ref = fp8.dequant(aq, sa) @ fp8.dequant(bq, sb, fp8.E5M2).t()
    torch.testing.assert_close(out, ref, rtol=2e-3, atol=2e-3 * ref.abs().max().item())


@pytest.mark.gpu
def test_fp8_linear_layer_forward_backward():
    torch.manual_seed(0)
    lin = torch.nn.Linear(1024, 768, bias=True).to("cuda", torch.bfloat16)
    ref = torch.nn.Linear(1024, 768, bias=True).to("cuda", torch.float32)
    ref.load_state_dict({k: v.float() for k, v in lin.state_dict().items()})
    lin.__class__ = fp8.Fp8Linear
    x = torch.randn(4, 512, 1024, device="cuda").bfloat16().requires_grad_(True)
    xr = x.detach().float().requires_grad_(True)
    y = lin(x)
    dy = torch.randn_like(y)
    y.backward(dy)
    yr = ref(xr)
    yr.backward(dy.float())
    rel = lambda a, b: ((a.float() - b).norm() / b.norm()).item()  # noqa: E731
    assert rel(y, yr) < 0.06 and rel(x.grad, xr.grad) < 0.08 and rel(lin.weight.grad, ref.weight.grad) < 0.08
    assert rel(lin.bias.grad, ref.bias.grad) < 0.02
