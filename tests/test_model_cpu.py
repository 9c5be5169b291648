"""Tiny hybrid models on CPU: every layer symbol builds, trains one step and decodes consistently."""
import pytest
import torch

from hybrid_model_factory_b200.models.configuration import HybridConfig
from hybrid_model_factory_b200.models.modeling_hybrid import build_model
from hybrid_model_factory_b200.models.cache import HybridCache


def tiny(pattern, model_type="hybrid_qwen3", **kw):
    n = len(pattern.split("-"))
    base = dict(vocab_size=256, hidden_size=64, intermediate_size=128, num_hidden_layers=n, num_attention_heads=4,
                num_key_value_heads=2, head_dim=16, hybrid_override_pattern=pattern, max_position_embeddings=512,
                bmojo_config={"window_size": 8, "ssm_mixer": "gdn", "tie_attn_weights": False},
                swa_config={"window_size": 8}, gka_config=None)
    base.update(kw)
    return HybridConfig(model_type, **base)


@pytest.mark.parametrize("pattern", ["*-GDN", "GKA-*", "M2-*", "BMF-SWA", "*-GDN-GKA-M2"])
def test_forward_backward(pattern):
    torch.manual_seed(0)
    cfg = tiny(pattern)
    model = build_model(cfg)
    ids = torch.randint(0, 256, (2, 48))
    out = model(ids, labels=ids)
    assert torch.isfinite(out.loss)
    out.loss.backward()
    missing = [n for n, p in model.named_parameters() if p.grad is None]
    assert not missing, f"params without grad: {missing[:5]}"
    assert all(torch.isfinite(p.grad).all() for p in model.parameters())


@pytest.mark.parametrize("pattern", ["*-GDN", "GKA-*", "M2-*", "BMF-SWA"])
def test_prefill_decode_matches_full_forward(pattern):
    torch.manual_seed(0)
    cfg = tiny(pattern)
    model = build_model(cfg).eval()
    ids = torch.randint(0, 256, (2, 40))
    with torch.no_grad():
        full = model(ids).logits
        cache = HybridCache()
        pre = model(ids[:, :33], past_key_values=cache, use_cache=True).logits
        steps = [pre]
        for t in range(33, 40):
            steps.append(model(ids[:, t:t + 1], past_key_values=cache, use_cache=True).logits)
        inc = torch.cat(steps, dim=1)
    torch.testing.assert_close(inc, full, rtol=2e-3, atol=2e-3)


def test_generate_and_param_names():
    cfg = tiny("*-GDN-GKA-M2")
    model = build_model(cfg)
    names = set(dict(model.named_parameters()))
    for n in ["model.layers.0.self_attn.q_norm.weight", "model.layers.1.gdn.A_log", "model.layers.1.gdn.q_conv1d.weight",
              "model.layers.2.gka.alpha_proj.bias", "model.layers.3.mamba.in_proj.weight", "model.layers.3.mamba.B_norm.weight",
              "model.layers.3.mamba.conv1d.weight", "model.norm.weight", "lm_head.weight"]:
        assert n in names, n
    out = model.generate(torch.randint(0, 256, (1, 5)), max_new_tokens=4)
    assert out.shape == (1, 9)


def test_moe_and_next_family():
    cfg = tiny("GDN-GDN-GDN-*", model_type="qwen3_next_hmf", num_experts=8, num_experts_per_tok=2,
               moe_intermediate_size=32, shared_expert_intermediate_size=32, linear_num_key_heads=2,
               linear_num_value_heads=4, linear_key_head_dim=16, linear_value_head_dim=16, router_aux_loss_coef=0.01)
    model = build_model(cfg)
    ids = torch.randint(0, 256, (2, 32))
    out = model(ids, labels=ids)
    assert out.aux_loss is not None and torch.isfinite(out.loss)
    out.loss.backward()
    assert model.model.layers[0].mlp.experts.gate_up_proj.grad is not None
    assert model.model.layers[3].self_attn.q_proj.weight.shape[0] == 2 * 4 * 16  # gated attention


def test_fused_layers_streams():
    cfg = tiny("*DA-GDN*-GKA*-GDN>GKA")
    model = build_model(cfg)
    h = torch.randn(2, 16, 64)
    pos = torch.arange(16).expand(2, 16)
    pe = model.model.rotary_emb(pos)
    outs = model.model.layers[1](h, h, position_embeddings=pe, position_ids=pos)
    assert len(outs) == 6 and not outs[1].requires_grad and outs[0].requires_grad


def test_layer_checkpoint_matches_plain_backward():
    torch.manual_seed(0)
    cfg = tiny("*-GDN-GKA-M2")
    m1 = build_model(cfg)
    import copy
    m2 = copy.deepcopy(m1)
    m2.gradient_checkpointing_enable()
    m1.train(), m2.train()
    ids = torch.randint(0, 256, (2, 40))
    m1(ids, labels=ids).loss.backward()
    m2(ids, labels=ids).loss.backward()
    for (n, a), (_, b) in zip(m1.named_parameters(), m2.named_parameters()):
        torch.testing.assert_close(a.grad, b.grad, rtol=1e-5, atol=1e-6, msg=n)


def test_offloaded_checkpoints_give_the_same_gradients():
    """Layer inputs parked in host memory between forward and backward (here: forced copies of CPU tensors)."""
    import copy
    from hybrid_model_factory_b200.utils import checkpointing
    torch.manual_seed(0)
    cfg = HybridConfig("hybrid_qwen3", vocab_size=128, hidden_size=64, intermediate_size=128, num_hidden_layers=3,
                       num_attention_heads=4, num_key_value_heads=2, head_dim=16, hybrid_override_pattern="*-GDN-M2")
    a = build_model(cfg)
    b = copy.deepcopy(a)
    ids = torch.randint(0, 128, (2, 24))
    a.gradient_checkpointing_enable()
    b.gradient_checkpointing_enable()
    a.train(), b.train()
    a(ids, labels=ids).loss.backward()
    moved = []
    orig = checkpointing._to_host
    checkpointing.set_offload(True, min_bytes=0, force_cpu_copy=True)
    checkpointing._to_host = lambda t: (moved.append(t.numel()) or orig(t))
    try:
        b(ids, labels=ids).loss.backward()
    finally:
        checkpointing._to_host = orig
        checkpointing.set_offload(False)
    assert len(moved) >= 3 and max(moved) == 2 * 24 * 64            # the hidden state of every layer went through a copy
    for (n, p), q in zip(a.named_parameters(), b.parameters()):
        assert torch.allclose(p.grad, q.grad, atol=1e-6), n
