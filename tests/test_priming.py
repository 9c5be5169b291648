"""Stage-0 priming, unfuse and checkpoint round trips on tiny models (CPU)."""
import json
import os

import torch

from hybrid_model_factory_b200.models.configuration import HybridConfig
from hybrid_model_factory_b200.models.modeling_hybrid import build_model
from hybrid_model_factory_b200.priming.fused_to_standard import unfuse_checkpoint, unfuse_model
from hybrid_model_factory_b200.priming.hybridize_model import hybridize_model, load_config
from hybrid_model_factory_b200.utils import checkpoint_io


def _base(tmp_path, n_layers=4):
    cfg = HybridConfig("qwen3", vocab_size=128, hidden_size=64, intermediate_size=128, num_hidden_layers=n_layers,
                       num_attention_heads=4, num_key_value_heads=2, head_dim=16, use_qk_norm=True)
    model = build_model(cfg)
    d = str(tmp_path / "base")
    checkpoint_io.save_pretrained(model, d, max_shard_size="200KB")
    raw = json.load(open(os.path.join(d, "config.json")))
    raw["model_type"] = "qwen3"
    json.dump(raw, open(os.path.join(d, "config.json"), "w"))
    return model, d


def test_sharded_roundtrip(tmp_path):
    model, d = _base(tmp_path)
    assert os.path.exists(os.path.join(d, "model.safetensors.index.json"))
    loaded = checkpoint_io.from_pretrained(d, dtype=torch.float32)
    for (n, a), (_, b) in zip(model.state_dict().items(), loaded.state_dict().items()):
        torch.testing.assert_close(a, b, msg=n)


def test_stage0_rules(tmp_path):
    base, d = _base(tmp_path)
    cfg = load_config({"base_model_name_or_path": d, "hybrid_override_pattern": "*-GDN-GKA-M2",
                       "output_dir": str(tmp_path / "hyb"), "dtype": "float32", "gka": {"num_iter": 5}})
    model, report = hybridize_model(cfg)
    sd, bsd = model.state_dict(), base.state_dict()
    # shared weights copied
    torch.testing.assert_close(sd["model.layers.0.self_attn.q_proj.weight"], bsd["model.layers.0.self_attn.q_proj.weight"])
    torch.testing.assert_close(sd["model.layers.2.mlp.up_proj.weight"], bsd["model.layers.2.mlp.up_proj.weight"])
    # GDN: q/k/v/o copied, g = 0.5 (o^T + repeat(v))
    wo, wv = bsd["model.layers.1.self_attn.o_proj.weight"], bsd["model.layers.1.self_attn.v_proj.weight"]
    torch.testing.assert_close(sd["model.layers.1.gdn.k_proj.weight"], bsd["model.layers.1.self_attn.k_proj.weight"])
    torch.testing.assert_close(sd["model.layers.1.gdn.g_proj.weight"], 0.5 * (wo.t() + wv.repeat_interleave(2, dim=0)))
    # GKA config knob propagated
    assert model.config.gka_config["num_iter"] == 5 and model.model.layers[2].gka.num_iter == 5
    # Mamba2: in_proj = [z, v, k, q, dt]
    w = sd["model.layers.3.mamba.in_proj.weight"]
    a = "model.layers.3.self_attn."
    torch.testing.assert_close(w[64:96], bsd[a + "v_proj.weight"])
    torch.testing.assert_close(w[96:128], bsd[a + "k_proj.weight"])
    torch.testing.assert_close(w[128:192], bsd[a + "q_proj.weight"])
    torch.testing.assert_close(w[:64], 0.5 * (bsd[a + "o_proj.weight"].t() + bsd[a + "v_proj.weight"].repeat_interleave(2, 0)))
    torch.testing.assert_close(sd["model.layers.3.mamba.B_norm.weight"], bsd[a + "k_norm.weight"])
    out_cfg = json.load(open(os.path.join(cfg.output_dir, "config.json")))
    assert out_cfg["hybrid_override_pattern"] == "*-GDN-GKA-M2" and "gdn_config" in out_cfg and "mamba2_config" in out_cfg
    # the saved hybrid checkpoint loads and runs
    m2 = checkpoint_io.from_pretrained(cfg.output_dir, dtype=torch.float32)
    out = m2(torch.randint(0, 128, (1, 16)))
    assert torch.isfinite(out.logits).all()


def test_fused_then_unfuse(tmp_path):
    base, d = _base(tmp_path)
    cfg = load_config({"base_model_name_or_path": d, "hybrid_override_pattern": "*DA-GDN*-GKA*-*DA",
                       "output_dir": str(tmp_path / "fused"), "dtype": "float32"})
    fused, _ = hybridize_model(cfg)
    # teacher attention weights are present next to the student mixer
    assert "model.layers.1.self_attn.q_proj.weight" in fused.state_dict()
    std, missing = unfuse_model(fused)
    assert std.config.hybrid_override_pattern == "*-GDN-GKA-*" and not missing
    torch.testing.assert_close(std.state_dict()["model.layers.1.gdn.g_proj.weight"],
                               fused.state_dict()["model.layers.1.gdn.g_proj.weight"])
    out = unfuse_checkpoint(cfg.output_dir)
    assert out.endswith("_unfused") and os.path.exists(os.path.join(out, "config.json"))
