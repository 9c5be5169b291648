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


def test_stage0_builds_an_l2a_model_and_trains_with_the_sparsity_term(tmp_path):
    """L2A construction: both attention streams and the second norm start from the layer they replace, the router at
    zero (every token takes global attention); ``hmf train`` with ``lambda_reg`` adds the router sparsity term."""
    from hybrid_model_factory_b200.train.workflow import run_exp
    base, d = _base(tmp_path)
    cfg = load_config({"base_model_name_or_path": d, "hybrid_override_pattern": "L2A-L2A-*-L2A",
                       "output_dir": str(tmp_path / "l2a"), "dtype": "float32",
                       "l2a": {"sliding_window": 8, "temperature": 0.1, "leak_prob": 0.0}})
    model, _ = hybridize_model(cfg)
    sd, bsd = model.state_dict(), base.state_dict()
    for name in ("q_proj", "k_proj", "v_proj", "o_proj", "q_norm", "k_norm"):
        src = bsd[f"model.layers.1.self_attn.{name}.weight"]
        torch.testing.assert_close(sd[f"model.layers.1.l2a.local.{name}.weight"], src)
        torch.testing.assert_close(sd[f"model.layers.1.l2a.global_attn.{name}.weight"], src)
    torch.testing.assert_close(sd["model.layers.3.l2a.global_norm.weight"], bsd["model.layers.3.input_layernorm.weight"])
    assert sd["model.layers.0.l2a.router.weight"].abs().sum() == 0
    assert model.config.l2a_config["sliding_window"] == 8
    model.eval()
    model(torch.randint(0, 128, (1, 24)))
    assert all(model.model.layers[i].l2a.last_routed_fraction == 1.0 for i in (0, 1, 3))
    out = str(tmp_path / "run")
    tr = run_exp({"model_name_or_path": cfg.output_dir, "stage": "pt", "synthetic": True, "cutoff_len": 32,
                  "max_steps": 4, "warmup_steps": 1, "output_dir": out, "bf16": False, "pure_bf16": False,
                  "learning_rate": 1e-3, "lr_scheduler_type": "constant", "per_device_train_batch_size": 2,
                  "lambda_reg": 0.5, "lambda_reg_scheduler": "constant", "hybrid_learnable_params": "l2a,norm"})
    from hybrid_model_factory_b200.train.l2a import L2ALoss
    assert isinstance(tr.loss_fn, L2ALoss) and tr.loss_fn.step >= 4 and tr.loss_fn.last_sparsity
    assert tr.model.model.layers[0].l2a.router.weight.abs().sum() > 0          # the router has started to move
