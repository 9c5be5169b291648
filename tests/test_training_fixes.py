"""Regression tests of the training stack: reference policy of DPO / KTO, reward scoring at the last real token,
ZeRO-3 save + resume, epoch wrap-around of the batch stream, loud failure after a recorded device-side timeout."""
import json
import math
import os
import types

import pytest
import torch

from hybrid_model_factory_b200.data import loader as L
from hybrid_model_factory_b200.models.configuration import HybridConfig
from hybrid_model_factory_b200.models.modeling_hybrid import build_model
from hybrid_model_factory_b200.train import preference as P
from hybrid_model_factory_b200.train.trainer import Trainer, TrainingArguments
from hybrid_model_factory_b200.train.workflow import run_exp

TINY = {"model_type": "hybrid_qwen3", "vocab_size": 259, "hidden_size": 32, "intermediate_size": 64,
        "num_hidden_layers": 2, "num_attention_heads": 2, "num_key_value_heads": 1, "head_dim": 16,
        "hybrid_override_pattern": "*-GDN", "torch_dtype": "float32"}


def _tiny(seed=0):
    torch.manual_seed(seed)
    return build_model(HybridConfig.from_dict(dict(TINY)))


def _pref_batch():
    g = torch.Generator().manual_seed(3)
    c = torch.randint(5, 250, (2, 12), generator=g)
    r = torch.randint(5, 250, (2, 12), generator=g)
    lab = lambda t: torch.cat([torch.full((2, 4), -100), t[:, 4:]], 1)
    return {"chosen_input_ids": c, "chosen_labels": lab(c), "rejected_input_ids": r, "rejected_labels": lab(r)}


def test_dpo_needs_and_uses_a_reference_policy():
    ft = types.SimpleNamespace(pref_beta=0.5, pref_loss="sigmoid", ref_model=None)
    model, batch = _tiny(0), _pref_batch()
    with pytest.raises(ValueError):                       # no reference anywhere: refuse, do not train unanchored
        P.make_preference_loss("dpo", ft)(model, batch)
    # reference = frozen copy of the starting policy: first loss is ln 2, and it moves once the policy does
    ref = P.ReferencePolicy.build(model, ft)
    loss_fn = P.make_preference_loss("dpo", ft, ref)
    l0 = loss_fn(model, batch)
    assert abs(l0.item() - math.log(2)) < 1e-5
    opt = torch.optim.SGD(model.parameters(), lr=0.5)
    for _ in range(3):
        opt.zero_grad()
        loss_fn(model, batch).backward()
        opt.step()
    l1 = loss_fn(model, batch).item()
    assert l1 < math.log(2) - 1e-3, l1                    # the KL-anchored margin really grows
    # another reference gives another loss for the same policy
    other = P.ReferencePolicy(_tiny(7))
    l2 = P.make_preference_loss("dpo", ft, other)(model, batch).item()
    assert abs(l2 - l1) > 1e-4
    # precomputed reference log-probabilities in the batch take precedence
    b2 = dict(batch, ref_chosen_logps=torch.zeros(2), ref_rejected_logps=torch.zeros(2))
    assert abs(P.make_preference_loss("dpo", ft)(model, b2).item() - l1) > 1e-6


def test_lora_policy_uses_its_base_weights_as_reference():
    from hybrid_model_factory_b200.train.adapters import LoRALinear, apply_lora
    ft = types.SimpleNamespace(pref_beta=0.5, pref_loss="sigmoid", ref_model=None)
    model, batch = _tiny(0), _pref_batch()
    apply_lora(model, rank=2)
    ref = P.ReferencePolicy.build(model, ft)
    assert ref.use_adapter_base and ref.model is None
    with torch.no_grad():
        for m in model.modules():
            if isinstance(m, LoRALinear):
                m.lora_B.normal_(std=0.2)
    loss = P.make_preference_loss("dpo", ft, ref)(model, batch).item()
    assert abs(loss - math.log(2)) > 1e-4                 # adapters moved the policy away from its own base
    assert all(m.enabled for m in model.modules() if isinstance(m, LoRALinear))


def test_kto_and_reward_scoring():
    ft = types.SimpleNamespace(pref_beta=0.1, pref_loss="sigmoid", ref_model=None)
    model = _tiny(0)
    ids = torch.randint(5, 250, (2, 10))
    batch = {"input_ids": ids, "labels": ids.clone(), "kto_tags": torch.tensor([1, 0])}
    with pytest.raises(ValueError):
        P.make_preference_loss("kto", ft)(model, batch)
    l = P.make_preference_loss("kto", ft, P.ReferencePolicy.build(model, ft))(model, batch)
    assert abs(l.item() - 0.5) < 1e-5                     # r = 0 against its own copy: sigmoid(0)
    # the reward is read at the last real token, not at the padded end of the row
    P.attach_value_head(model)
    pad = 0
    a = torch.tensor([[7, 8, 9, 10, 11, pad, pad, pad]])
    b = torch.tensor([[7, 8, 9, 10, 11, 55, 66, 77]])
    assert P.last_token_index(a, None, pad).tolist() == [4]
    sa = P.reward_scores(model, a, None, pad)
    sb = P.reward_scores(model, b[:, :5], None, pad)
    assert torch.allclose(sa, sb, atol=1e-5)              # causal model: same prefix, same score


def test_zero3_checkpoint_resume(tmp_path):
    out = str(tmp_path / "z3")
    (tmp_path / "ds.json").write_text(json.dumps({"zero_optimization": {"stage": 3}}))
    cfg = {"model_name_or_path": json.dumps(TINY), "stage": "pt", "synthetic": True, "cutoff_len": 32, "max_steps": 2,
           "save_steps": 2, "output_dir": out, "bf16": False, "pure_bf16": False, "learning_rate": 1e-3,
           "lr_scheduler_type": "constant", "per_device_train_batch_size": 2, "deepspeed": str(tmp_path / "ds.json")}
    tr = run_exp(cfg)
    assert tr.global_step == 2
    ck = os.path.join(out, "checkpoint-2")
    tr.optimizer.gather_full_state()
    want = {k: v.clone() for k, v in tr.model.state_dict().items()}
    tr.optimizer.release_all()
    # full resume (optimizer shards present) and model-only resume both restore the weights under ZeRO-3
    for model_only in (False, True):
        if model_only:
            os.remove(os.path.join(ck, "optimizer_rank00000.pt"))
        tr2 = run_exp(dict(cfg, max_steps=3, resume_from_checkpoint=ck, output_dir=str(tmp_path / f"r{int(model_only)}")))
        assert tr2.global_step == 3
    model = _tiny(1)
    targs = TrainingArguments(output_dir="", zero_stage=3, max_steps=1, logging_steps=0, bf16=False, pure_bf16=False,
                              resume_from_checkpoint=ck)
    tr3 = Trainer(model, targs, device=torch.device("cpu"))
    tr3.optimizer.gather_full_state()
    for k, v in tr3.model.state_dict().items():
        assert torch.allclose(v, want[k]), k
    tr3.optimizer.release_all()


def test_resume_refuses_a_checkpoint_that_lacks_model_parameters(tmp_path):
    from hybrid_model_factory_b200.utils import checkpoint_io
    model = _tiny(0)
    sd = {k: v for k, v in model.state_dict().items() if "q_proj" not in k}
    checkpoint_io.save_state_dict(checkpoint_io.to_hf_names(sd), str(tmp_path))
    model.config.save_pretrained(str(tmp_path))
    with pytest.raises(KeyError):
        checkpoint_io.from_pretrained(str(tmp_path))
    assert checkpoint_io.from_pretrained(str(tmp_path), allow_missing=True)._load_report["missing"]
    with pytest.raises(KeyError):
        Trainer(_tiny(0), TrainingArguments(output_dir="", max_steps=1, logging_steps=0, bf16=False, pure_bf16=False,
                                            resume_from_checkpoint=str(tmp_path)), device=torch.device("cpu"))


def test_batch_stream_wraps_epochs_and_is_rank_uniform():
    rows = [{"input_ids": [i] * 4, "labels": [i] * 4} for i in range(11)]      # 11 samples: not divisible by dp*B = 4
    ds = L.ListDataset(rows, False)
    assert L.steps_per_epoch(len(ds), 2, world=2, sp_size=1) == 2
    streams = []
    for rank in range(2):
        it = L.batch_iterator(ds, 2, rank, 2, 1, pin=False, num_epochs=2, shuffle=True, seed=5)
        streams.append([b["input_ids"][:, 0].tolist() for b in it])
    assert len(streams[0]) == len(streams[1]) == 4         # two epochs of two steps on every rank
    assert streams[0][:2] == [[0, 1], [4, 5]] and streams[1][:2] == [[2, 3], [6, 7]]
    second = sum(streams[0][2:] + streams[1][2:], [])
    assert len(set(second)) == 8 and second != [0, 1, 4, 5, 2, 3, 6, 7]          # reshuffled, no repeats
    # without an epoch limit the stream keeps going (the trainer stops at max_steps); resuming skips steps
    it = L.batch_iterator(ds, 2, 0, 2, 1, pin=False, start_step=3)
    assert next(it)["input_ids"][:, 0].tolist() == [4, 5]


def test_two_epochs_run_to_the_end_of_the_schedule(tmp_path):
    (tmp_path / "dataset_info.json").write_text(json.dumps({"d": {"file_name": "d.json", "columns": {"prompt": "text"}}}))
    (tmp_path / "d.json").write_text(json.dumps([{"text": "lorem ipsum dolor sit amet " * 6} for _ in range(6)]))
    cfg = {"model_name_or_path": json.dumps(TINY), "stage": "pt", "dataset": "d", "dataset_dir": str(tmp_path),
           "cutoff_len": 32, "num_train_epochs": 2, "output_dir": str(tmp_path / "run"), "bf16": False, "pure_bf16": False,
           "learning_rate": 1e-3, "per_device_train_batch_size": 2}
    tr = run_exp(cfg)
    assert tr.global_step == tr.args.max_steps and tr.args.max_steps >= 2 and tr.args.max_steps % 2 == 0


def test_recorded_timeout_makes_the_trainer_fail_loudly():
    from hybrid_model_factory_b200.ops._lib import KernelError
    tr = Trainer(_tiny(0), TrainingArguments(output_dir="", max_steps=1, logging_steps=0, bf16=False, pure_bf16=False),
                 device=torch.device("cpu"))
    tr.check_kernel_status(lambda: (0, 0, 0, 0))
    with pytest.raises(KernelError):
        tr.check_kernel_status(lambda: (2, 17, 0x350, 1))


# -- Qwen3-Next / Qwen3.5 converters ---------------------------------------------------------------------------
NEXT_TINY = {"model_type": "qwen3_next_hmf", "vocab_size": 97, "hidden_size": 32, "intermediate_size": 48,
             "num_hidden_layers": 4, "num_attention_heads": 2, "num_key_value_heads": 1, "head_dim": 16,
             "linear_num_key_heads": 2, "linear_num_value_heads": 4, "linear_key_head_dim": 8, "linear_value_head_dim": 8,
             "num_experts": 4, "num_experts_per_tok": 2, "moe_intermediate_size": 16,
             "shared_expert_intermediate_size": 16, "decoder_sparse_step": 1, "mlp_only_layers": [],
             "hybrid_override_pattern": "GDN-GDN-GDN-*", "torch_dtype": "float32",
             "layer_types": ["linear_attention"] * 3 + ["full_attention"]}


def _to_source_layout(model, layout: str):
    """State dict of a tiny hybrid model written the way the released Qwen checkpoints store it."""
    from hybrid_model_factory_b200.priming import convert_qwen_gdn as cv
    from hybrid_model_factory_b200.utils import checkpoint_io
    cfg = model.config
    Hk, Hv, dk, dv = (cfg.linear_num_key_heads, cfg.linear_num_value_heads, cfg.linear_key_head_dim,
                      cfg.linear_value_head_dim)
    prefix = "model.language_model." if layout == "qwen3_5" else "model."
    out = {}
    sd = checkpoint_io.to_hf_names(model.state_dict())
    for name, t in sd.items():
        if ".gdn." not in name:
            out[name.replace("model.", prefix, 1) if name.startswith("model.") else name] = t.clone()
    for i, layer in enumerate(model.model.layers):
        if layer.symbol != "GDN":
            continue
        g = {k: v.clone() for k, v in layer.gdn.state_dict().items()}
        p = f"{prefix}layers.{i}.linear_attn."
        if layout == "qwen3_next":
            out[p + "in_proj_qkvz.weight"] = cv.interleave_qkvz(g["q_proj.weight"], g["k_proj.weight"], g["v_proj.weight"],
                                                                 g["g_proj.weight"], Hk, Hv, dk, dv)
            out[p + "in_proj_ba.weight"] = cv.interleave_ba(g["b_proj.weight"], g["gk_proj.weight"], Hk, Hv)
        else:
            out[p + "in_proj_qkv.weight"] = torch.cat([g["q_proj.weight"], g["k_proj.weight"], g["v_proj.weight"]])
            out[p + "in_proj_z.weight"], out[p + "in_proj_b.weight"] = g["g_proj.weight"], g["b_proj.weight"]
            out[p + "in_proj_a.weight"] = g["gk_proj.weight"]
        out[p + "conv1d.weight"] = torch.cat([g["q_conv1d.weight"], g["k_conv1d.weight"], g["v_conv1d.weight"]])
        out[p + "A_log"], out[p + "dt_bias"] = g["A_log"], g["dt_bias"]
        out[p + "norm.weight"], out[p + "out_proj.weight"] = g["o_norm.weight"], g["o_proj.weight"]
    out["mtp.layers.0.input_layernorm.weight"] = torch.ones(cfg.hidden_size)        # dropped by the converter
    if layout == "qwen3_5":
        out["model.visual.patch_embed.proj.weight"] = torch.ones(4, 4)
    return out


@pytest.mark.parametrize("layout", ["qwen3_next", "qwen3_5"])
def test_qwen_gdn_checkpoint_converts_and_loads_strictly(tmp_path, layout):
    from hybrid_model_factory_b200.priming import convert_qwen_gdn as cv
    from hybrid_model_factory_b200.utils import checkpoint_io
    torch.manual_seed(0)
    model = build_model(HybridConfig.from_dict(dict(NEXT_TINY))).eval()
    src_dir, out_dir = str(tmp_path / "src"), str(tmp_path / "out")
    os.makedirs(src_dir)
    checkpoint_io.save_state_dict(_to_source_layout(model, layout), src_dir)
    src_cfg = dict(NEXT_TINY, model_type="qwen3_next" if layout == "qwen3_next" else "qwen3_5_moe_text")
    src_cfg.pop("hybrid_override_pattern")
    if layout == "qwen3_5":
        src_cfg = {"model_type": "qwen3_5_moe", "text_config": src_cfg}
    with open(os.path.join(src_dir, "config.json"), "w") as f:
        json.dump(src_cfg, f)
    rep = cv.convert_checkpoint(src_dir, out_dir, dtype=torch.float32)
    assert rep["missing"] == [] and any(k.startswith("mtp.") for k in rep["dropped"])
    assert rep["layers"][0] == "linear_attention -> GDN" and rep["layers"][3] == "full_attention -> *"
    loaded = checkpoint_io.from_pretrained(out_dir).eval()           # strict: raises on any missing parameter
    ids = torch.randint(0, 97, (2, 24))
    with torch.no_grad():
        a = model(ids, return_logits=True).logits
        b = loaded(ids, return_logits=True).logits
    assert torch.allclose(a, b, atol=1e-5), (a - b).abs().max()
    keys = set(checkpoint_io.load_state_dict(out_dir))
    assert "model.layers.0.gdn.q_proj.weight" in keys and not any("seq_mixer" in k or "linear_attn" in k for k in keys)


def test_qwen_gdn_to_gka_and_attention_to_ssm_targets(tmp_path):
    from hybrid_model_factory_b200.priming import convert_qwen_gdn as cv
    from hybrid_model_factory_b200.utils import checkpoint_io
    torch.manual_seed(0)
    # attention -> SSM copies q/k/v/o row for row, so it needs a source whose attention and linear-attention head
    # layouts coincide (the stage-0 rules raise on a shape mismatch)
    NEXT_TINY = dict(globals()["NEXT_TINY"], num_key_value_heads=2, head_dim=8, linear_num_value_heads=2)
    model = build_model(HybridConfig.from_dict(dict(NEXT_TINY))).eval()
    src_dir, out_dir = str(tmp_path / "src"), str(tmp_path / "out")
    os.makedirs(src_dir)
    checkpoint_io.save_state_dict(_to_source_layout(model, "qwen3_next"), src_dir)
    src_cfg = dict(NEXT_TINY, model_type="qwen3_next")
    src_cfg.pop("hybrid_override_pattern")
    with open(os.path.join(src_dir, "config.json"), "w") as f:
        json.dump(src_cfg, f)
    rep = cv.convert_checkpoint(src_dir, out_dir, pattern="GDN-GKA-GDN>GKA-GDN", dtype=torch.float32)
    assert rep["layers"] == {0: "linear_attention -> GDN", 1: "linear_attention -> GKA",
                             2: "linear_attention -> GDN>GKA", 3: "full_attention -> GDN"}
    assert all(any(m.startswith(p) for p in rep["fresh"]) for m in rep["missing"]) and rep["missing"]
    out = checkpoint_io.load_state_dict(out_dir)
    g0 = model.model.layers[1].gdn.state_dict()
    assert torch.equal(out["model.layers.1.gka.a_proj.weight"], g0["gk_proj.weight"])
    assert torch.equal(out["model.layers.1.gka.b_proj.weight"], g0["b_proj.weight"])
    assert torch.equal(out["model.layers.2.gdn.q_proj.weight"], model.model.layers[2].gdn.q_proj.weight)
    assert torch.equal(out["model.layers.2.gka.q_proj.weight"], model.model.layers[2].gdn.q_proj.weight)
    # attention -> GDN: query rows come out of the per-head [q | gate] blocks of the gated attention
    qg = model.model.layers[3].self_attn.q_proj.weight.view(2, 16, -1)
    assert torch.allclose(out["model.layers.3.gdn.q_proj.weight"], qg[:, :8].reshape(16, -1))
    assert cv.main([src_dir, str(tmp_path / "cli"), "--dtype", "float32"]) == 0
    # a naming mismatch is an error, not a silent random initialisation
    with pytest.raises(KeyError):
        cv.load_converted(build_model(HybridConfig.from_dict(dict(NEXT_TINY))), {"model.layers.0.seq_mixer.x": torch.ones(1)}, [])


def test_plot_loss_writes_curves(tmp_path):
    from hybrid_model_factory_b200.utils.ploting import plot_loss, smooth
    cfg = {"model_name_or_path": json.dumps(TINY), "stage": "pt", "synthetic": True, "cutoff_len": 32, "max_steps": 5,
           "output_dir": str(tmp_path / "run"), "bf16": False, "pure_bf16": False, "learning_rate": 1e-3,
           "per_device_train_batch_size": 2, "plot_loss": True}
    run_exp(cfg)
    files = [f for f in os.listdir(tmp_path / "run") if f.startswith("training_loss")]
    assert files and os.path.getsize(tmp_path / "run" / files[0]) > 200
    assert len(smooth([3.0, 2.0, 1.0])) == 3 and plot_loss(str(tmp_path / "nothing")) == []


def test_recompute_plan_keeps_layers_that_fit(tmp_path):
    """The activation probe records what each checkpointed layer's graph holds; the plan un-checkpoints layers from the
    last one backwards while they fit, and the un-checkpointed model gives the same loss and gradients."""
    import torch
    from hybrid_model_factory_b200.models.configuration import HybridConfig
    from hybrid_model_factory_b200.models.modeling_hybrid import build_model
    from hybrid_model_factory_b200.train.trainer import Trainer, TrainingArguments
    from hybrid_model_factory_b200.utils import checkpointing
    torch.manual_seed(0)
    cfg = HybridConfig("hybrid_qwen3", vocab_size=64, hidden_size=32, intermediate_size=64, num_hidden_layers=4,
                       num_attention_heads=2, num_key_value_heads=1, head_dim=16, hybrid_override_pattern="*-GDN-*-M2")
    model = build_model(cfg)
    tr = Trainer(model, TrainingArguments(output_dir="", learning_rate=0.0, max_steps=4, logging_steps=0,
                                          pure_bf16=False, bf16=False), device=torch.device("cpu"))
    ids = torch.randint(0, 64, (2, 24))
    batch = {"input_ids": ids, "labels": ids.clone()}
    live = {"n": 0}

    def fake_mem():            # every call reports 100 more bytes: each layer "holds" 100 bytes
        live["n"] += 100
        return live["n"]
    checkpointing.start_probe(fake_mem)
    model.train()
    model(input_ids=ids, labels=ids).loss.backward()
    sizes = checkpointing.stop_probe()
    assert sorted(sizes) == [0, 1, 2, 3] and all(v == 100 for v in sizes.values())
    g_ref = {n: p.grad.clone() for n, p in model.named_parameters() if p.grad is not None}
    # room for two and a half layers: total 1000, peak 600 -> (0.9 * 1000 - 600) * 0.8 = 240
    assert tr.plan_recompute(sizes, 1000, 600) == [2, 3]
    assert model.model.checkpoint_skip == frozenset({2, 3})
    model.zero_grad()
    loss2 = model(input_ids=ids, labels=ids).loss
    loss2.backward()
    for n, p in model.named_parameters():
        if n in g_ref:
            assert torch.allclose(p.grad, g_ref[n], atol=1e-6), n
    # a layer larger than the rest of the budget is passed over, smaller earlier ones still go in
    assert checkpointing.choose_unchecked_layers({0: 50, 1: 500, 2: 100}, 160) == [0, 2]
    assert tr.train_step(batch) is not None


def test_dft_and_eaft_losses_match_their_definitions():
    import torch
    import torch.nn.functional as F
    from hybrid_model_factory_b200.models.configuration import HybridConfig
    from hybrid_model_factory_b200.models.modeling_hybrid import build_model
    from hybrid_model_factory_b200.train.losses import make_weighted_sft_loss
    torch.manual_seed(0)
    cfg = HybridConfig("hybrid_qwen3", vocab_size=50, hidden_size=32, intermediate_size=64, num_hidden_layers=2,
                       num_attention_heads=2, num_key_value_heads=1, head_dim=16, hybrid_override_pattern="*-GDN")
    model = build_model(cfg)
    ids = torch.randint(0, 50, (2, 20))
    labels = ids.clone()
    labels[:, :5] = -100
    logits = model(input_ids=ids).logits.float()[:, :-1].reshape(-1, 50)
    y = labels[:, 1:].reshape(-1)
    ce = F.cross_entropy(logits, y, ignore_index=-100, reduction="none")[y != -100]
    lg = logits[y != -100]
    dft = (ce * torch.exp(-ce).detach()).mean()
    top = torch.topk(lg, 20, dim=-1).values
    lp = top - torch.logsumexp(top, -1, keepdim=True)
    ent = -(lp.exp() * lp).sum(-1)
    eaft = (ce * torch.pow(ent / 3.0, 2.0).detach()).mean()
    batch = {"input_ids": ids, "labels": labels}
    got_dft = make_weighted_sft_loss("dft", chunk=7)(model, batch)
    got_eaft = make_weighted_sft_loss("eaft", 2.0, chunk=7)(model, batch)
    assert torch.allclose(got_dft, dft, atol=1e-5) and torch.allclose(got_eaft, eaft, atol=1e-5)
    # gradients flow through the cross entropy only (the weights are constants)
    g1 = torch.autograd.grad(got_dft, model.lm_head.weight)[0]
    g2 = torch.autograd.grad(dft, model.lm_head.weight)[0]
    assert torch.allclose(g1, g2, atol=1e-6)


def test_tensorboard_event_file_neftune_and_callbacks(tmp_path):
    """The event writer's records carry valid checksums and read back; CRC-32C matches its published check value;
    ``report_to: tensorboard`` puts a callback on the run; NEFTune perturbs embeddings in training mode only."""
    from hybrid_model_factory_b200.train.adapters import add_neftune
    from hybrid_model_factory_b200.train.workflow import build_callbacks
    from hybrid_model_factory_b200.utils.tensorboard_writer import (EventWriter, TensorBoardCallback, crc32c,
                                                                    read_scalars)
    assert crc32c(b"123456789") == 0xE3069283
    w = EventWriter(str(tmp_path / "runs"))
    for step in range(3):
        w.add_scalars({"train/loss": 2.0 - 0.5 * step, "train/learning_rate": 1e-4}, step)
    w.close()
    got = list(read_scalars(w.path))
    assert len(got) == 6 and got[0] == ("train/loss", 2.0, 0) and got[4][0] == "train/loss" and got[4][2] == 2
    assert abs(got[5][1] - 1e-4) < 1e-9
    raw = bytearray(open(w.path, "rb").read())
    raw[-6] ^= 0xFF                                              # a flipped payload byte is caught
    open(w.path, "wb").write(bytes(raw))
    import pytest
    with pytest.raises(ValueError, match="checksum"):
        list(read_scalars(w.path))

    class Args:
        report_to, output_dir = "tensorboard", str(tmp_path)
    cbs = build_callbacks(Args())
    assert any(isinstance(c, TensorBoardCallback) for c in cbs)

    torch.manual_seed(0)
    cfg = HybridConfig("hybrid_qwen3", vocab_size=64, hidden_size=32, intermediate_size=64, num_hidden_layers=2,
                       num_attention_heads=2, num_key_value_heads=1, head_dim=16, hybrid_override_pattern="*-GDN")
    model = build_model(cfg)
    ids = torch.randint(0, 64, (1, 8))
    model.eval()
    clean = model.model.embed_tokens(ids)
    handle = add_neftune(model, alpha=5.0)
    assert torch.equal(model.model.embed_tokens(ids), clean)
    model.train()
    noisy = model.model.embed_tokens(ids)
    bound = 5.0 / (8 * 32) ** 0.5
    assert 0 < (noisy - clean).abs().max() <= bound + 1e-6
    handle.remove()
    assert torch.equal(model.model.embed_tokens(ids), clean)
