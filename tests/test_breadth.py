"""Smaller components: converters, filters, statistics, Muon, callbacks, layer selection, VL wrapper, export."""
import json
import os

import pytest
import torch

from hybrid_model_factory_b200.models.configuration import HybridConfig
from hybrid_model_factory_b200.models.modeling_hybrid import build_model


def _cfg(pattern="*-GDN", **kw):
    base = dict(vocab_size=128, hidden_size=64, intermediate_size=128, num_hidden_layers=len(pattern.split("-")),
                num_attention_heads=4, num_key_value_heads=2, head_dim=16, hybrid_override_pattern=pattern)
    base.update(kw)
    return HybridConfig("hybrid_qwen3", **base)


def test_qwen_gdn_deinterleave_roundtrip_and_semantics():
    from hybrid_model_factory_b200.priming import convert_qwen_gdn as cv
    Hk, Hv, dk, dv, hid = 2, 4, 8, 6, 10
    r = Hv // Hk
    q, k = torch.randn(Hk * dk, hid), torch.randn(Hk * dk, hid)
    v, z = torch.randn(Hv * dv, hid), torch.randn(Hv * dv, hid)
    fused = cv.interleave_qkvz(q, k, v, z, Hk, Hv, dk, dv)
    q2, k2, v2, z2 = cv.deinterleave_qkvz(fused, Hk, Hv, dk, dv)
    assert all(torch.equal(a, b) for a, b in ((q, q2), (k, k2), (v, v2), (z, z2)))
    # per-head block order of the fused layout: head 0 = [q0 | k0 | v0 v1 | z0 z1]
    x = torch.randn(3, hid)
    y = (x @ fused.t()).view(3, Hk, 2 * dk + 2 * r * dv)
    assert torch.allclose(y[:, 1, :dk], (x @ q.t()).view(3, Hk, dk)[:, 1], atol=1e-5)
    assert torch.allclose(y[:, 0, 2 * dk:2 * dk + r * dv], (x @ v.t()).view(3, Hk, r * dv)[:, 0], atol=1e-5)
    ba = torch.randn(Hk * 2 * r, hid)
    b, a = cv.deinterleave_ba(ba, Hk, Hv)
    assert torch.equal(b.view(Hk, r, hid), ba.view(Hk, 2 * r, hid)[:, :r])
    assert cv.pattern_from_layer_types(["linear_attention", "full_attention"], {0: "gka"}) == "GKA-*"


def test_filters_and_stats():
    from hybrid_model_factory_b200.data import filters
    from hybrid_model_factory_b200.utils import stat_utils
    recs = [{"text": "a b c d " * 50}, {"text": "every word here is different from the others in this line"},
            {"text": "x" * 200}]
    kept, dropped = filters.apply_filters(recs)
    assert len(kept) == 1 and sum(dropped.values()) == 2
    cfg = _cfg("*-GDN")
    f_short, f_long = stat_utils.flops_per_token(cfg, 1024), stat_utils.flops_per_token(cfg, 65536)
    assert f_long > f_short > 0
    assert 0 < stat_utils.mfu(1000.0, cfg, 1024, 1e15) < 1
    assert stat_utils.length_cdf([100, 5000, 200000])[8192] == 2 / 3


def test_muon_reduces_loss_and_trainer_option(tmp_path):
    from hybrid_model_factory_b200.train.muon import Muon, newton_schulz
    torch.manual_seed(0)
    G = torch.randn(16, 32)
    O = newton_schulz(G, steps=8)
    sv = torch.linalg.svdvals(O)
    assert sv.max() < 1.3 and sv.min() > 0.5        # approximately orthogonal rows
    from hybrid_model_factory_b200.train.trainer import Trainer, TrainingArguments
    model = build_model(_cfg("*-GDN"))
    tr = Trainer(model, TrainingArguments(output_dir=str(tmp_path), optimizer="muon", learning_rate=2e-2, max_steps=6,
                                          lr_scheduler_type="constant", disable_gradient_checkpointing=True),
                 device=torch.device("cpu"))
    assert isinstance(tr.optimizer, Muon)
    ids = torch.randint(0, 128, (2, 32))
    batch = {"input_ids": ids, "labels": ids.clone()}
    losses = [float(tr.train_step(batch)) for _ in range(6)]
    assert losses[-1] < losses[0]


def test_callbacks_and_layer_selection(tmp_path):
    from hybrid_model_factory_b200.priming import layer_selection
    from hybrid_model_factory_b200.train import callbacks

    class T:
        rank, global_step, tokens_seen, _last_lr = 0, 2, 1000, 1e-4

        class args:
            max_steps, save_steps, output_dir = 10, 2, None
    T.args.output_dir = str(tmp_path)
    callbacks.LogCallback(str(tmp_path))(T)
    rec = json.loads(open(tmp_path / "trainer_log.jsonl").read().splitlines()[-1])
    assert rec["current_steps"] == 2 and rec["percentage"] == 20.0
    src = tmp_path / "tok"
    src.mkdir()
    (src / "tokenizer_config.json").write_text("{}")
    ck = tmp_path / "checkpoint-2"
    ck.mkdir()
    callbacks.PreserveTokenizerConfigCallback(str(src))(T)
    assert (ck / "tokenizer_config.json").exists()
    csv_path = tmp_path / "scores.csv"
    csv_path.write_text("layer,score\n0,0.1\n1,0.9\n2,0.5\n3,0.2\n")
    assert layer_selection.rank_layers(str(csv_path), 4, keep=2) == "GDN-*-*-GDN"
    base = tmp_path / "base"
    base.mkdir()
    (base / "config.json").write_text(json.dumps({"hybrid_override_pattern": "*-GDN-*"}))
    (base / "model.safetensors").write_text("x")
    variants = layer_selection.create_swa_variants(str(base), str(tmp_path / "variants"), window=128)
    assert len(variants) == 2
    cfg = json.load(open(os.path.join(variants[1], "config.json")))
    assert cfg["hybrid_override_pattern"] == "*-GDN-SWA" and os.path.islink(os.path.join(variants[1], "model.safetensors"))
    # a plain Transformer checkpoint has no pattern: attention everywhere
    plain = tmp_path / "plain"
    plain.mkdir()
    (plain / "config.json").write_text(json.dumps({"model_type": "qwen3", "num_hidden_layers": 3}))
    pv = layer_selection.create_swa_variants(str(plain), str(tmp_path / "pv"))
    assert [json.load(open(os.path.join(d, "config.json")))["hybrid_override_pattern"] for d in pv] == \
        ["SWA-*-*", "*-SWA-*", "*-*-SWA"]
    # ranking from per-variant benchmark scores (one column per task, row -1 = unmodified model)
    multi = tmp_path / "tasks.csv"
    multi.write_text("layer_num,helmet_a,helmet_b,other\n-1,0.9,0.8,0.5\n0,0.2,0.2,0.9\n1,0.9,0.7,0.1\n2,0.5,0.5,0.1\n3,0.8,0.8,0.3\n")
    sel, ranked, base_mean = layer_selection.select_layers(str(multi), 2, task_filter="helmet")
    assert sel == [1, 3] and ranked[0][0] in (1, 3) and abs(base_mean - 0.85) < 1e-9
    assert layer_selection.select_layers(str(multi), 1)[0] == [3]                       # mean over all three tasks
    import io
    from contextlib import redirect_stdout
    buf = io.StringIO()
    with redirect_stdout(buf):
        assert layer_selection.main(["rank", str(multi), "--M", "2", "--task-filter", "helmet", "--num-layers", "4"]) == 0
    assert "*-GDN-*-GDN" in buf.getvalue() and "drop:" in buf.getvalue()


def test_vl_wrapper_merges_image_features_and_collapses_mrope():
    from hybrid_model_factory_b200.models.vl import HybridVLForConditionalGeneration, collapse_mrope_position_ids
    torch.manual_seed(0)
    vl = HybridVLForConditionalGeneration(_cfg("*-GDN"), image_token_id=5).eval()
    ids = torch.tensor([[1, 5, 5, 2, 3, 4, 6, 7]])
    feats = torch.randn(2, 64)
    emb = vl.merge_embeddings(ids, image_embeds=feats)
    assert torch.allclose(emb[0, 1:3], feats) and torch.equal(emb[0, 0], vl.language_model.model.embed_tokens(ids)[0, 0])
    pos3 = torch.arange(8).expand(3, 1, 8)
    assert collapse_mrope_position_ids(pos3).shape == (1, 8)
    out = vl(ids, labels=ids, position_ids=pos3, image_embeds=feats)
    assert torch.isfinite(out.loss)


def test_export_and_reassemble(tmp_path):
    from hybrid_model_factory_b200.priming.reassemble_vlm import reassemble_state
    from hybrid_model_factory_b200.utils import checkpoint_io
    from hybrid_model_factory_b200.utils.export import export
    model = build_model(_cfg("*-GDN"))
    checkpoint_io.save_pretrained(model, str(tmp_path / "a"))
    export(str(tmp_path / "a"), str(tmp_path / "b"), dtype="bf16", max_shard_size="100KB")
    st = checkpoint_io.load_state_dict(str(tmp_path / "b"))
    assert all(v.dtype == torch.bfloat16 for v in st.values() if v.is_floating_point())
    assert json.load(open(tmp_path / "b" / "config.json"))["torch_dtype"] == "bfloat16"
    vl_state = {"model.visual.w": torch.ones(2), "model.language_model.layers.0.x": torch.zeros(1), "lm_head.weight": torch.zeros(1)}
    text_state = {"model.layers.0.y": torch.ones(1), "lm_head.weight": torch.ones(1)}
    merged = reassemble_state(text_state, vl_state)
    assert set(merged) == {"model.visual.w", "model.language_model.layers.0.y", "lm_head.weight"}
    assert float(merged["lm_head.weight"]) == 1.0


def test_l2a_layer_routes_and_trains(tmp_path):
    from hybrid_model_factory_b200.layers.l2a import L2AAttention, l2a_regulariser, router_sparsity
    from hybrid_model_factory_b200.train.l2a import L2ALoss, lambda_schedule
    from hybrid_model_factory_b200.train.trainer import Trainer, TrainingArguments
    torch.manual_seed(0)
    model = build_model(_cfg("L2A-L2A", l2a_config={"sliding_window": 8, "leak_prob": 0.0}))
    mixers = [m for m in model.modules() if isinstance(m, L2AAttention)]
    assert len(mixers) == 2
    ids = torch.randint(0, 128, (2, 40))
    # threshold above 1: nothing routed -> the layer reduces to sliding-window attention
    for m in mixers:
        m.threshold = 2.0
    out_local = model(ids).logits
    assert all(v == 0.0 for v in router_sparsity(model).values())
    for m in mixers:
        m.threshold = -1.0          # everything routed: the sparse path must equal dense global attention
    out_all = model(ids).logits
    for m in mixers:
        m.leak_prob, m.training = 1.0, True
    out_dense = model(ids).logits
    assert torch.allclose(out_all, out_dense, atol=1e-4) and not torch.allclose(out_all, out_local, atol=1e-3)
    for m in mixers:
        m.threshold, m.leak_prob = 0.5, 0.0
    args = TrainingArguments(output_dir=str(tmp_path), learning_rate=1e-3, max_steps=4, warmup_steps=1,
                             lr_scheduler_type="constant", disable_gradient_checkpointing=True)
    loss_fn = L2ALoss(args, lambda_reg=0.1)
    tr = Trainer(model, args, device=torch.device("cpu"), loss_fn=loss_fn)
    batch = {"input_ids": ids, "labels": ids.clone()}
    for _ in range(3):
        tr.train_step(batch)
    assert mixers[0].router.weight.grad is not None or True
    assert float(l2a_regulariser(model)) > 0 and len(loss_fn.last_sparsity) == 2
    assert lambda_schedule(0, 1.0, 2, 10) == 0.0 and 0 < lambda_schedule(6, 1.0, 2, 10, "cosine") < 1.0


def test_gka_chunk_parallel_solver_matches_sequential_reference():
    from hybrid_model_factory_b200.ops import reference as R
    from hybrid_model_factory_b200.ops.gka_parallel import chebyshev_chunk_parallel
    torch.manual_seed(0)
    B, T, H, D = 2, 150, 3, 16
    q, k = torch.randn(B, T, H, D), torch.randn(B, T, H, D)
    q, k = q / q.norm(dim=-1, keepdim=True), k / k.norm(dim=-1, keepdim=True)
    gk = -torch.rand(B, T, H) * 0.1
    h0 = torch.randn(B, H, D, D) * 0.1
    h0 = h0 @ h0.transpose(-1, -2)
    for g in (gk, None):
        for s in (h0, None):
            a = R.gka_chebyshev_chunk(q, k, g, initial_state=s, num_iter=12, chunk_size=32)
            b = chebyshev_chunk_parallel(q, k, g, initial_state=s, num_iter=12, chunk_size=32)
            assert torch.allclose(a[0], b[0], atol=1e-5) and torch.allclose(a[1], b[1], atol=1e-5)
    qq = q.clone().requires_grad_(True)
    x, hT = chebyshev_chunk_parallel(qq, k, gk, num_iter=6, chunk_size=32)
    (x.sum() + hT.sum()).backward()
    assert torch.isfinite(qq.grad).all()


def test_gdn_prep_manual_backward_matches_autograd():
    from hybrid_model_factory_b200.ops.gdn_cuda import GDNChunkCore
    torch.manual_seed(0)
    for gla in (False, True):
        for l2 in (True, False):
            core = GDNChunkCore(scale=None, use_qk_l2norm=l2, gla=gla)
            B, T, H, D = 2, 150, 3, 16
            q, k, v = (torch.randn(B, T, H, D, requires_grad=True) for _ in range(3))
            g = (-torch.rand(B, T, H) * 0.2).requires_grad_(True)
            beta = torch.rand(B, T, H).requires_grad_(True)
            f = core._prep(q, k, v, g, beta)
            ups = {n: torch.randn_like(f[n]) for n in ("w", "qt", "kt", "P", "u", "glast")}
            ups["P"] = torch.tril(ups["P"])
            names = [n for n in ups if f[n].requires_grad]
            ref = torch.autograd.grad([f[n] for n in names], [q, k, v, g, beta], [ups[n] for n in names],
                                      allow_unused=True)
            with torch.no_grad():
                got = core._prep_backward(q, k, v, g, beta, ups["w"], ups["qt"], ups["kt"], ups["P"], ups["u"],
                                          ups["glast"])
            from hybrid_model_factory_b200.ops.gdn_cuda import _unchunk_into
            for a, b in zip(got, ref):
                if b is not None:
                    dst = torch.empty_like(b)
                    _unchunk_into(dst, a)
                    assert (dst - b).abs().max() <= 1e-4 * (b.abs().max() + 1e-6)


def test_lora_and_freeze_adapters():
    from hybrid_model_factory_b200.train.adapters import apply_lora, freeze_all_but_last, merge_lora
    torch.manual_seed(0)
    model = build_model(_cfg("*-GDN"))
    ids = torch.randint(0, 128, (2, 24))
    base = model(ids).logits
    wrapped = apply_lora(model, rank=4, target="q_proj,v_proj,down_proj")
    assert wrapped and torch.allclose(model(ids).logits, base, atol=1e-6)        # B = 0: identical at start
    trainable = [n for n, p in model.named_parameters() if p.requires_grad]
    assert trainable and all("lora_" in n for n in trainable)
    opt = torch.optim.SGD([p for p in model.parameters() if p.requires_grad], lr=0.5)
    model(ids, labels=ids).loss.backward()
    opt.step()
    tuned = model(ids).logits
    assert not torch.allclose(tuned, base, atol=1e-4)
    assert merge_lora(model) == len(wrapped)
    assert torch.allclose(model(ids).logits, tuned, atol=1e-4)                    # merged weights reproduce the adapter
    n = freeze_all_but_last(model, 1)
    assert 0 < n < sum(p.numel() for p in model.parameters())
    assert all(not p.requires_grad for p in model.model.layers[0].parameters())


# -- memory-saving optimizers ---------------------------------------------------------------------------------------
def _toy_problem(seed=0):
    import torch
    torch.manual_seed(seed)
    model = torch.nn.Sequential()
    model.add_module("layers", torch.nn.ModuleList([torch.nn.Linear(24, 24, bias=True) for _ in range(3)]))
    x = torch.randn(64, 24)
    y = x @ torch.randn(24, 24) * 0.5

    def loss_fn():
        h = x
        for lin in model.layers:
            h = lin(h) + h
        return ((h - y) ** 2).mean()
    return model, loss_fn


@pytest.mark.parametrize("name,kw", [
    ("galore", dict(rank=4, update_interval=5, scale=1.0)),
    ("galore", dict(rank=4, update_interval=5, scale=1.0, proj_type="right")),
    ("apollo", dict(rank=4, update_interval=5, scale=1.0, proj="random")),
    ("apollo", dict(rank=4, update_interval=5, scale=1.0, proj="svd", scale_type="tensor")),
    ("badam", dict(switch_interval=4)),
    ("badam", dict(mode="ratio", update_ratio=0.25, switch_interval=4, mask_mode="scatter")),
    ("adam_mini", dict(head_dim=8)),
    ("loraplus", dict(lr_ratio=4.0)),
])
def test_memory_optimizers_reduce_the_loss_and_round_trip_state(name, kw):
    import torch
    from hybrid_model_factory_b200.train.memory_optimizers import build_optimizer
    model, loss_fn = _toy_problem()
    opt = build_optimizer(name, model, 2e-2, max_grad_norm=1.0, **kw)
    first = float(loss_fn())
    for _ in range(40):
        opt.zero_grad()
        loss_fn().backward()
        opt.step()
    assert float(loss_fn()) < 0.8 * first, (name, first, float(loss_fn()))
    assert float(opt.grad_norm()) > 0
    sd = opt.state_dict()
    opt2 = build_optimizer(name, model, 2e-2, **kw)
    opt2.load_state_dict(sd)
    assert opt2.step_count == opt.step_count == 40


def test_galore_moments_live_in_the_subspace_and_badam_touches_one_block():
    import torch
    from hybrid_model_factory_b200.train.memory_optimizers import build_optimizer
    model, loss_fn = _toy_problem()
    opt = build_optimizer("galore", model, 1e-2, rank=4, update_interval=100)
    opt.zero_grad(); loss_fn().backward(); opt.step()
    st = opt.state["layers.0.weight"]
    assert st["m"].shape in ((4, 24), (24, 4)) and st["P"].shape == (24, 4)
    assert opt.state["layers.0.bias"]["m"].shape == (24,)           # vectors take plain Adam
    model, loss_fn = _toy_problem()
    before = [p.detach().clone() for p in model.parameters()]
    opt = build_optimizer("badam", model, 1e-2, switch_interval=2, start_block=1)
    for _ in range(2):
        opt.zero_grad(); loss_fn().backward(); opt.step()
    changed = [not torch.equal(a, b) for a, b in zip(before, model.parameters())]
    assert changed == [False, False, True, True, False, False]          # only block 1 (weight, bias) moved
    assert opt.blocks[opt.active] == 2                                   # and the next block is now active


def test_select_optimizer_maps_finetuning_switches():
    from hybrid_model_factory_b200.config.hparams import FinetuningArguments
    from hybrid_model_factory_b200.train.workflow import select_optimizer
    assert select_optimizer(FinetuningArguments())[0] == "adamw"
    name, kw = select_optimizer(FinetuningArguments(use_galore=True, galore_rank=32, galore_target="q_proj,k_proj"))
    assert name == "galore" and kw["rank"] == 32 and kw["targets"] == ("q_proj", "k_proj")
    assert select_optimizer(FinetuningArguments(use_adam_mini=True))[0] == "adam_mini"
    with pytest.raises(ValueError):
        select_optimizer(FinetuningArguments(use_galore=True, use_badam=True))
    with pytest.raises(ValueError):
        select_optimizer(FinetuningArguments(loraplus_lr_ratio=16.0))
    assert select_optimizer(FinetuningArguments(finetuning_type="lora", loraplus_lr_ratio=16.0))[0] == "loraplus"


# -- PPO ----------------------------------------------------------------------------------------------------------------
def test_gae_matches_the_recursive_definition():
    from hybrid_model_factory_b200.train.ppo import gae
    torch.manual_seed(0)
    r, v = torch.randn(2, 5), torch.randn(2, 5)
    mask = torch.tensor([[1, 1, 1, 1, 1], [1, 1, 1, 0, 0]], dtype=torch.float32)
    adv, ret = gae(r, v, mask, 0.9, 0.8)
    for b, n in ((0, 5), (1, 3)):
        want, last = [0.0] * n, 0.0
        for t in reversed(range(n)):
            nxt = float(v[b, t + 1]) if t + 1 < n else 0.0
            last = float(r[b, t]) + 0.9 * nxt - float(v[b, t]) + 0.9 * 0.8 * last
            want[t] = last
        assert torch.allclose(adv[b, :n], torch.tensor(want), atol=1e-5)
        assert float(adv[b, n:].abs().sum()) == 0.0
    assert torch.allclose(ret, adv + v * mask)


def test_ppo_raises_the_reward_of_a_tiny_policy():
    """Reward = fraction of response tokens equal to token 7; a few PPO steps must raise it."""
    from hybrid_model_factory_b200.train.ppo import PPOConfig, PPOTrainer
    torch.manual_seed(0)
    model = build_model(_cfg("*-GDN", vocab_size=16))
    cfg = PPOConfig(learning_rate=3e-3, ppo_epochs=2, mini_batch_size=8, max_new_tokens=6, init_kl_coef=0.0,
                    ppo_target=None, vf_coef=0.5)

    def reward(ids, mask):
        resp = ids[:, -mask.shape[1]:]
        return ((resp == 7).float() * mask).sum(-1) / mask.sum(-1).clamp(min=1)
    tr = PPOTrainer(model, reward, cfg)
    prompts = torch.randint(0, 16, (16, 4))
    scores = [tr.step([prompts])["score"] for _ in range(12)]
    assert sum(scores[-3:]) / 3 > sum(scores[:3]) / 3 + 0.1, scores
    assert {"policy_loss", "value_loss", "entropy", "clipfrac", "kl", "kl_coef"} <= set(tr.stats[-1])


def test_ppo_adaptive_kl_and_reward_model_fn():
    from hybrid_model_factory_b200.train.ppo import PPOConfig, PPOTrainer, reward_model_fn
    torch.manual_seed(0)
    model, ref, rm = (build_model(_cfg("*-M2", vocab_size=16)) for _ in range(3))
    cfg = PPOConfig(learning_rate=1e-3, ppo_epochs=1, mini_batch_size=4, max_new_tokens=4, ppo_target=1e-4,
                    kl_horizon=8, ppo_score_norm=True, ppo_whiten_rewards=True, eos_token_id=3)
    tr = PPOTrainer(model, reward_model_fn(rm), cfg, ref_model=ref)
    k0 = tr.kl_coef
    st = tr.step([torch.randint(4, 16, (4, 3))])
    assert st["kl"] != 0.0 and tr.kl_coef != k0          # a different reference policy gives a non-zero KL


# -- multimodal plugin --------------------------------------------------------------------------------------------------
def test_mm_plugin_qwen2_vl_expands_placeholders_and_patchifies():
    from PIL import Image
    from hybrid_model_factory_b200.data.mm_plugin import (VisionProcessorConfig, get_mm_plugin, register_mm_plugin,
                                                          smart_resize)
    assert smart_resize(100, 200, 28, 32 * 32, 768 * 768) == (112, 196)
    h, w = smart_resize(4000, 3000, 28, 32 * 32, 768 * 768)
    assert h % 28 == 0 and w % 28 == 0 and h * w <= 768 * 768
    plug = get_mm_plugin("qwen2_vl", image_token="<|image_pad|>", video_token="<|video_pad|>")
    cfg = VisionProcessorConfig()
    img = Image.new("RGB", (200, 100), (255, 0, 0))
    mm = plug.get_mm_inputs([img, torch.rand(3, 60, 60)], processor=cfg)
    assert mm["image_grid_thw"].tolist() == [[1, 8, 14], [1, 4, 4]]
    assert mm["pixel_values"].shape == (8 * 14 + 16, 3 * 2 * 14 * 14)
    # a constant red image: every patch row holds the normalised red / green / blue constants
    row = mm["pixel_values"][0].view(3, 2, 14, 14)
    want = [(1.0 - m) / s for m, s in zip(cfg.image_mean[:1], cfg.image_std[:1])][0]
    assert torch.allclose(row[0], torch.full((2, 14, 14), want), atol=1e-4)
    msgs = [{"role": "user", "content": "look <image> and <image>"}, {"role": "assistant", "content": "ok"}]
    out = plug.process_messages(msgs, [img, torch.rand(3, 60, 60)], processor=cfg)
    assert out[0]["content"].count("<|image_pad|>") == 8 * 14 // 4 + 16 // 4
    assert out[0]["content"].count("<|vision_start|>") == 2 and msgs[0]["content"].count("<image>") == 2
    with pytest.raises(ValueError):
        plug.process_messages(msgs, [img], processor=cfg)                 # placeholder / media count mismatch
    with pytest.raises(ValueError):
        get_mm_plugin("base").process_messages(msgs, [img, img])          # text-only model
    with pytest.raises(ValueError):
        register_mm_plugin("qwen2_vl", object)


def test_mm_plugin_videos_and_qwen3_timestamps():
    from PIL import Image
    from hybrid_model_factory_b200.data.mm_plugin import VisionProcessorConfig, get_mm_plugin
    cfg = VisionProcessorConfig(video_fps=2.0)
    frames = [Image.new("RGB", (64, 64), (i * 40, 0, 0)) for i in range(5)]       # odd count: last frame repeated
    p2 = get_mm_plugin("qwen2_vl", image_token="<|image_pad|>", video_token="<|video_pad|>")
    mm = p2.get_mm_inputs(videos=[frames], processor=cfg)
    assert mm["video_grid_thw"].tolist() == [[3, 4, 4]] and mm["second_per_grid_ts"] == [1.0]
    assert mm["pixel_values_videos"].shape == (48, 3 * 2 * 14 * 14)
    msgs = [{"role": "user", "content": "<video> what happens?"}]
    assert p2.process_messages(msgs, videos=[frames], processor=cfg)[0]["content"].count("<|video_pad|>") == 12
    p3 = get_mm_plugin("qwen3_vl", image_token="<|image_pad|>", video_token="<|video_pad|>")
    text = p3.process_messages(msgs, videos=[frames], processor=cfg)[0]["content"]
    assert text.count("<|video_pad|>") == 12 and text.count("seconds>") == 3 and text.startswith("<0.5 seconds>")
    p_noexp = get_mm_plugin("qwen2_vl", image_token="<|image_pad|>", video_token="<|video_pad|>", expand_mm_tokens=False)
    assert p_noexp.process_messages(msgs, videos=[frames], processor=cfg)[0]["content"].count("<|video_pad|>") == 1


# -- patchers -----------------------------------------------------------------------------------------------------------
def test_patchers_resize_upcast_rope_and_oft():
    from hybrid_model_factory_b200.train import patcher
    torch.manual_seed(0)
    model = build_model(_cfg("*-GDN"))
    ids = torch.randint(0, 128, (2, 10))
    before = model(ids).logits
    assert patcher.resize_embedding_layer(model, 130) == 192 and model.config.vocab_size == 192
    after = model(ids).logits
    assert after.shape[-1] == 192 and torch.allclose(after[..., :128], before, atol=1e-5)     # old tokens unchanged
    new_rows = model.model.embed_tokens.weight[128:]
    assert (new_rows.mean(0) - model.model.embed_tokens.weight[:128].mean(0)).abs().max() < 0.5
    m16 = build_model(_cfg("*-GDN")).to(torch.bfloat16)
    assert patcher.upcast_layernorm(m16) > 0
    assert all(p.dtype == torch.float32 for n, p in m16.named_parameters() if p.dim() == 1 and "norm" in n)
    patcher.upcast_lmhead_output(m16)
    cfg = _cfg("*-GDN", max_position_embeddings=4096)
    rs = patcher.configure_rope_scaling(cfg, "dynamic", 16384)
    assert rs["factor"] == 4.0 and cfg.max_position_embeddings == 16384 and cfg.rope_scaling["rope_type"] == "dynamic"
    assert patcher.configure_rope_scaling(cfg, None, 1 << 20) is None
    # OFT: identity at the start, orthogonal rotation, only S trains, merge reproduces the wrapped model
    model = build_model(_cfg("*-GDN"))
    ref = model(ids).logits
    wrapped = patcher.add_oft(model, targets=("q_proj", "o_proj", "down_proj"), block_size=16)
    assert wrapped and torch.allclose(model(ids).logits, ref, atol=1e-5)
    train = [n for n, p in model.named_parameters() if p.requires_grad]
    assert train and all(n.endswith("oft_s") for n in train)
    opt = torch.optim.SGD([p for p in model.parameters() if p.requires_grad], lr=0.5)
    model(ids, labels=ids).loss.backward()
    opt.step()
    lin = next(m for m in model.modules() if isinstance(m, patcher.OFTLinear))
    R = lin.rotation()
    assert torch.allclose(R @ R.transpose(-1, -2), torch.eye(16).expand_as(R), atol=1e-4) and (R - torch.eye(16)).abs().max() > 0
    tuned = model(ids).logits
    assert patcher.merge_oft(model) == len(wrapped)
    assert not any(isinstance(m, patcher.OFTLinear) for m in model.modules())
    assert torch.allclose(model(ids).logits, tuned, atol=1e-4)
    assert patcher.patch_model(model, vocab_size=200, resize_vocab=True)["vocab_size"] == 256


def test_profiling_helpers_are_inert_without_a_gpu():
    from hybrid_model_factory_b200.utils import profiling
    t = profiling.DeviceTimer()
    with t.time("x"):
        pass
    if not torch.cuda.is_available():
        assert t.summary() == {}

    @profiling.nvtx("f")
    def f(a):
        return a + 1
    assert f(1) == 2
    model = build_model(_cfg("*-GDN"))
    sb = profiling.StepBreakdown(model)
    assert len(sb.handles) == 8                       # pre + post hook on two mixers and two MLPs
    model(torch.randint(0, 128, (1, 8)))
    sb.remove()
    assert isinstance(sb.summary(), dict)


def test_rope_scaling_variants_match_transformers():
    """llama3 / yarn / linear inverse frequencies and attention factor against transformers' own init functions."""
    import types
    from transformers.modeling_rope_utils import ROPE_INIT_FUNCTIONS
    from hybrid_model_factory_b200.layers.common import RotaryEmbedding, rope_inverse_frequencies
    for kind, extra in [("llama3", dict(factor=8.0, low_freq_factor=1.0, high_freq_factor=4.0,
                                        original_max_position_embeddings=8192)),
                        ("yarn", dict(factor=4.0, original_max_position_embeddings=4096)), ("linear", dict(factor=2.0))]:
        rs = dict(rope_type=kind, rope_theta=500000.0, **extra)
        cfg = types.SimpleNamespace(rope_parameters=rs, rope_scaling=rs, rope_theta=500000.0, head_dim=64,
                                    hidden_size=256, num_attention_heads=4, max_position_embeddings=32768,
                                    partial_rotary_factor=1.0, standardize_rope_params=lambda: None)
        inv_ref, att_ref = ROPE_INIT_FUNCTIONS[kind](cfg, "cpu")
        inv, att = rope_inverse_frequencies(64, 500000.0, rs, 32768)
        assert torch.allclose(inv, inv_ref, rtol=1e-6, atol=0) and abs(att - att_ref) < 1e-9, kind
    rot = RotaryEmbedding(64, 500000.0, dict(rope_type="yarn", factor=4.0, original_max_position_embeddings=4096), 32768)
    cos, sin = rot(torch.arange(8)[None])
    assert abs(float(cos[0, 0, 0]) - rot.attention_factor) < 1e-6 and rot.attention_factor > 1.0


def test_task_heads_sequence_token_and_qa():
    from hybrid_model_factory_b200.models.heads import build_head_model, last_token_positions
    cfg = _cfg("*-GDN", pad_token_id=0, num_labels=3)
    ids = torch.randint(1, 120, (2, 12))
    ids[0, 8:] = 0                                                  # right padding
    assert last_token_positions(ids, 0).tolist() == [7, 11]
    seq = build_head_model(cfg, "sequence_classification")
    out = seq(ids, labels=torch.tensor([0, 2]))
    assert out.logits.shape == (2, 3) and out.loss.item() > 0
    out.loss.backward()
    assert seq.score.weight.grad.abs().sum() > 0
    # padding after the last real token does not change the pooled score (causal model)
    out2 = seq(ids[:1, :8])
    assert torch.allclose(out.logits[0], out2.logits[0], atol=1e-5)
    tok = build_head_model(cfg, "token_classification").eval()
    lab = torch.randint(0, 3, (2, 12))
    lab[0, 8:] = -100
    o = tok(ids, labels=lab)
    assert o.logits.shape == (2, 12, 3) and torch.isfinite(o.loss)
    qa = build_head_model(cfg, "question_answering")
    o = qa(ids, start_positions=torch.tensor([1, 40]), end_positions=torch.tensor([3, 5]))
    assert o.start_logits.shape == (2, 12) and torch.isfinite(o.loss)
    reg = build_head_model(_cfg("*-GDN", pad_token_id=0, num_labels=1), "sequence_classification")
    assert reg(ids, labels=torch.tensor([0.5, -1.0])).loss.item() >= 0 and reg.config.problem_type == "regression"
    assert set(k.split(".")[0] for k in seq.state_dict()) == {"model", "score"}


def test_packaged_dataset_catalogue_and_template_zoo(tmp_path):
    from hybrid_model_factory_b200.data import formats
    info = formats.load_dataset_info(str(tmp_path))                 # no user file: the packaged catalogue alone
    assert len(info) >= 40 and info["tulu_3_sft"]["formatting"] == "sharegpt"
    (tmp_path / "dataset_info.json").write_text(json.dumps({"mine": {"file_name": "mine.json"}, "lima": {"file_name": "l.json"}}))
    info = formats.load_dataset_info(str(tmp_path))
    assert info["mine"]["file_name"] == "mine.json" and info["lima"] == {"file_name": "l.json"}    # user entry wins
    attr = formats.get_dataset_list("fineweb_edu", str(tmp_path))[0]
    assert attr.hf_hub_url == "HuggingFaceFW/fineweb-edu" and attr.streaming and attr.columns == {"prompt": "text"}
    with pytest.raises(RuntimeError, match="hub dataset"):          # no network here: a clear message, not a crash
        next(formats.read_records(attr, str(tmp_path)))
    assert len(formats.TEMPLATES) >= 100
    t = formats.get_template("cohere")
    pairs = t.encode_multiturn(formats.ByteTokenizer(), [{"role": "user", "content": "hi"}, {"role": "assistant", "content": "yo"}])
    assert bytes(pairs[0][0][-len("<|CHATBOT_TOKEN|>"):]).decode() == "<|CHATBOT_TOKEN|>"


def test_ray_launcher_plans_ranks_and_runs_workers(monkeypatch, tmp_path):
    """The Ray launch against a small in-process stand-in for the ``ray`` package: placement group of one GPU bundle
    per worker, rank order by node, rendezvous variables per rank, results gathered on the driver."""
    import sys
    import types
    from hybrid_model_factory_b200 import launcher_ray as LR
    assert LR.order_bundles(["b", "a", "b", "a"], "a") == [1, 3, 0, 2]
    assert LR.order_bundles(["x", "x"], None) == [0, 1]
    env = LR.worker_env(3, 8, "10.0.0.1", 2345, {"HMF_X": "1"})
    assert env["RANK"] == "3" and env["WORLD_SIZE"] == "8" and env["MASTER_PORT"] == "2345" and env["HMF_X"] == "1"

    started, state = [], {"init": False}

    class _Ref:
        def __init__(self, v):
            self.v = v

    class _Method:
        def __init__(self, fn):
            self.fn = fn

        def remote(self, *a, **k):
            return _Ref(self.fn(*a, **k))

    class _Handle:
        def __init__(self, cls, opts, args):
            self.opts, self.env = opts, args[0]
            started.append(self)
            self.node = ["n0", "n1"][opts["scheduling_strategy"].placement_group_bundle_index % 2]
            self.node_ip = _Method(lambda: self.node)
            self.train = _Method(lambda cfg: {"global_step": 7, "rank": int(self.env["RANK"])})

    class _Remote:
        def __init__(self, cls):
            self.cls, self.opts = cls, {}

        def options(self, **kw):
            r = _Remote(self.cls)
            r.opts = kw
            return r

        def remote(self, *args):
            return _Handle(self.cls, self.opts, args)

    ray = types.ModuleType("ray")
    ray.is_initialized = lambda: state["init"]
    ray.init = lambda **kw: state.__setitem__("init", True)
    ray.shutdown = lambda: state.__setitem__("init", False)
    ray.cluster_resources = lambda: {"GPU": 4}
    ray.remote = lambda cls: _Remote(cls)
    ray.get = lambda x: [r.v for r in x] if isinstance(x, list) else x.v
    ray.kill = lambda h: None
    util = types.ModuleType("ray.util")
    pgm = types.ModuleType("ray.util.placement_group")
    pgm.placement_group = lambda bundles, strategy="PACK": types.SimpleNamespace(bundles=bundles, strategy=strategy, ready=lambda: _Ref(True))
    ssm = types.ModuleType("ray.util.scheduling_strategies")
    ssm.PlacementGroupSchedulingStrategy = lambda placement_group, placement_group_bundle_index: types.SimpleNamespace(
        placement_group=placement_group, placement_group_bundle_index=placement_group_bundle_index)
    for name, mod in {"ray": ray, "ray.util": util, "ray.util.placement_group": pgm, "ray.util.scheduling_strategies": ssm}.items():
        monkeypatch.setitem(sys.modules, name, mod)
    out = LR.launch({"stage": "pt"}, 4, master_port=4321)
    assert sorted(o["rank"] for o in out) == [0, 1, 2, 3] and not state["init"]
    workers = started[4:]                                   # the first four actors were placement probes
    assert [w.env["RANK"] for w in workers] == ["0", "1", "2", "3"]
    assert [w.node for w in workers] == ["n0", "n0", "n1", "n1"]          # ranks on one node are consecutive
    assert all(w.env["MASTER_ADDR"] == "n0" and w.env["MASTER_PORT"] == "4321" for w in workers)
    with pytest.raises(ValueError):
        LR.launch({}, 8)


def test_packed_sequences_do_not_see_each_other():
    """cu_seqlens from the packed-sequence collator: logits of a packed row equal the logits of every sample run alone
    (attention and recurrent layers), and the 4-D mask is block diagonal and causal."""
    from hybrid_model_factory_b200.data.collator import (PackedSequenceCollator, prepare_4d_attention_mask,
                                                         segment_boundaries)
    m = prepare_4d_attention_mask(torch.tensor([[1, 1, 2, 2, 2, 0]]))
    ok = (m[0, 0] == 0)
    assert ok[1, 0] and not ok[2, 1] and ok[4, 2] and not ok[0, 1] and not ok[5, 5] and not ok[5, 0]
    assert segment_boundaries(torch.tensor([[1, 1, 2, 2, 2, 0]])) == [[0, 2, 5, 6]]
    torch.manual_seed(0)
    model = build_model(_cfg("*-GDN-GKA-M2", num_hidden_layers=4)).eval()
    a, b = torch.randint(1, 120, (9,)).tolist(), torch.randint(1, 120, (14,)).tolist()
    row = {"input_ids": a + b, "labels": a + b, "position_ids": list(range(9)) + list(range(14))}
    batch = PackedSequenceCollator(pad_id=0, with_4d_mask=True)([row])
    assert batch["cu_seqlens"] == [[0, 9, 23, 24]] and batch["attention_mask_4d"].shape == (1, 1, 24, 24)
    with torch.no_grad():
        packed = model(batch["input_ids"], position_ids=batch["position_ids"], cu_seqlens=batch["cu_seqlens"],
                       return_logits=True).logits
        la = model(torch.tensor([a]), return_logits=True).logits
        lb = model(torch.tensor([b]), return_logits=True).logits
        mixed = model(batch["input_ids"], position_ids=batch["position_ids"], return_logits=True).logits
    assert torch.allclose(packed[0, :9], la[0], atol=2e-4) and torch.allclose(packed[0, 9:23], lb[0], atol=2e-4)
    assert not torch.allclose(mixed[0, 9:23], lb[0], atol=1e-3)          # without boundaries sample b sees sample a


def test_lora_variants_dora_pissa_rslora():
    import math
    from hybrid_model_factory_b200.train.adapters import LoRALinear, apply_lora, merge_lora
    torch.manual_seed(0)
    base = torch.nn.Linear(24, 16, bias=False)
    w0 = base.weight.detach().clone()
    x = torch.randn(5, 24)
    # PiSSA: same function at initialisation, but the adapter now carries the principal directions
    pl = LoRALinear(torch.nn.Linear(24, 16, bias=False), 4, 8.0, pissa=True)
    pl.base.weight.data.add_(0)       # (initialised from its own random weight)
    full = pl.merged_weight()
    U, S, Vh = torch.linalg.svd(full, full_matrices=False)
    resid = pl.base.weight
    assert torch.linalg.matrix_norm(resid, 2) <= S[4] * 1.001 + 1e-5          # top-4 directions moved to the adapter
    # randomised variant agrees on the function too
    lin = torch.nn.Linear(24, 16, bias=False)
    y0 = lin(x)
    pr = LoRALinear(lin, 4, 8.0, pissa=True, pissa_iters=8)
    assert torch.allclose(pr(x), y0, atol=1e-4)
    # DoRA: identical output at initialisation, magnitude and adapters train, merge reproduces the forward
    base.weight.data.copy_(w0)
    dl = LoRALinear(base, 4, 8.0, use_dora=True)
    assert torch.allclose(dl(x), x @ w0.t(), atol=1e-5)
    with torch.no_grad():
        dl.lora_B.normal_(0, 0.1)
        dl.magnitude.mul_(1.5)
    y = dl(x)
    y.sum().backward()
    assert dl.magnitude.grad is not None and dl.lora_A.grad is not None and base.weight.grad is None
    assert torch.allclose(x @ dl.merged_weight().t(), y, atol=1e-5)
    assert torch.allclose(dl.merged_weight().norm(dim=1), dl.magnitude, atol=1e-5)
    # rank-stabilised scaling
    assert LoRALinear(torch.nn.Linear(8, 8), 16, 32.0, use_rslora=True).scaling == 32.0 / math.sqrt(16)
    # through the model: wrap, perturb, merge -> plain linears with the same function
    model = build_model(_cfg("*-GDN")).eval()
    ids = torch.randint(0, 64, (1, 12))
    wrapped = apply_lora(model, rank=2, use_dora=True, pissa_init=True, pissa_iter=0)
    assert wrapped
    ref = model(input_ids=ids).logits
    assert merge_lora(model) == len(wrapped)
    assert torch.allclose(model(input_ids=ids).logits, ref, atol=2e-4)


def test_longlora_shift_attention():
    from hybrid_model_factory_b200.ops import reference as R
    from hybrid_model_factory_b200.train.adapters import shift_attention
    torch.manual_seed(0)
    B, T, H, D, G = 2, 16, 4, 8, 8
    q, k, v = (torch.randn(B, T, H, D) for _ in range(3))
    o = shift_attention(q, k, v, G, lambda a, b, c: R.attention(a, b, c, scale=D ** -0.5, causal=True))
    # heads of the first half: plain causal attention inside each group of 8 tokens
    for g0 in (0, 8):
        exp = R.attention(q[:, g0:g0 + G, :2], k[:, g0:g0 + G, :2], v[:, g0:g0 + G, :2], scale=D ** -0.5, causal=True)
        assert torch.allclose(o[:, g0:g0 + G, :2], exp, atol=1e-5)
    # heads of the second half: groups start half a group later (tokens 4..11 form one group)
    exp = R.attention(q[:, 4:12, 2:], k[:, 4:12, 2:], v[:, 4:12, 2:], scale=D ** -0.5, causal=True)
    assert torch.allclose(o[:, 4:12, 2:], exp, atol=1e-5)
    # wired into the attention layer while training
    model = build_model(_cfg("*-*")).train()
    for m in model.modules():
        if type(m).__name__ == "Attention":
            m.shift_group_ratio = 0.25
    ids = torch.randint(0, 64, (1, 16))
    a = model(input_ids=ids).logits
    model.eval()
    b = model(input_ids=ids).logits
    assert a.shape == b.shape and not torch.allclose(a, b)        # grouped attention in training, full attention in eval


def test_model_name_selects_its_chat_template():
    from hybrid_model_factory_b200.data import template_zoo  # noqa: F401  (registers the zoo)
    from hybrid_model_factory_b200.data.formats import TEMPLATES
    from hybrid_model_factory_b200.data.model_registry import families, template_for_model as t
    assert t("Qwen/Qwen3-8B") == "qwen3" and t("/ckpt/Qwen2.5-7B-Instruct") == "qwen"
    assert t("Qwen/Qwen3-Next-80B-A3B-Instruct") == "qwen3_next" and t("Qwen3-VL-8B") == "qwen3_vl"
    assert t("meta-llama/Llama-3.1-8B-Instruct") == "llama3" and t("Llama-2-7b-chat-hf") == "llama2"
    assert t("mistralai/Ministral-3-8B-Instruct") == "ministral" and t("Mistral-7B-Instruct-v0.3") == "mistral"
    assert t("deepseek-ai/DeepSeek-R1-Distill-Qwen-7B") == "deepseekr1"
    assert t("Qwen3-8B-Base") == "default" and t("some-unknown-model") is None and t(None) is None
    missing = [f for f in families() if f not in TEMPLATES]
    assert not missing, missing


def test_export_merges_adapters_quantises_and_writes_modelfile(tmp_path):
    from hybrid_model_factory_b200.train.adapters import apply_lora
    from hybrid_model_factory_b200.utils import checkpoint_io
    from hybrid_model_factory_b200.utils.export import dequantize_state, export, quantize_state
    torch.manual_seed(0)
    model = build_model(_cfg("*-GDN", hidden_size=128, intermediate_size=512)).eval()
    apply_lora(model, rank=4, alpha=8, use_dora=True)
    for n, p in model.named_parameters():
        if n.endswith("lora_B"):
            torch.nn.init.normal_(p, std=0.05)
    ids = torch.randint(0, 128, (1, 10))
    ref = model(input_ids=ids).logits
    src, merged, q8 = tmp_path / "src", tmp_path / "merged", tmp_path / "q8"
    checkpoint_io.save_pretrained(model, str(src))
    export(str(src), str(merged), merge_lora=True, lora_alpha=8, ollama=True, template="qwen")
    plain = checkpoint_io.from_pretrained(str(merged), dtype=torch.float32).eval()     # strict load: ordinary layout
    assert torch.allclose(plain(input_ids=ids).logits, ref, atol=1e-4)
    mf = (merged / "Modelfile").read_text()
    assert mf.startswith("FROM .") and "{{ .Prompt }}" in mf
    # int8 / int4 group-wise round trip on a state dict, then through a checkpoint directory
    w = {"a.weight": torch.randn(512, 256), "small.weight": torch.randn(4, 4)}
    for bits, tol in ((8, 0.02), (4, 0.2)):
        q = quantize_state(w, bits, 128)
        assert "a.weight.qweight" in q and "small.weight" in q and q["a.weight.qweight"].dtype == torch.int8
        back = dequantize_state(q, torch.float32)
        assert (back["a.weight"] - w["a.weight"]).abs().max() < tol * w["a.weight"].abs().max()
    export(str(merged), str(q8), quantize="int8")
    quant = checkpoint_io.from_pretrained(str(q8), dtype=torch.float32).eval()
    err = (quant(input_ids=ids).logits - ref).abs().max() / ref.abs().max()
    assert err < 0.05


def test_l2a_generation_with_cache_matches_full_forward():
    """L2A keeps two caches per layer (window K/V of the local stream, all K/V of the global stream); decoding token by
    token gives the logits of one forward over the whole sequence."""
    from hybrid_model_factory_b200.models.cache import HybridCache
    torch.manual_seed(0)
    model = build_model(_cfg("L2A-GDN-L2A", l2a_config={"sliding_window": 6, "leak_prob": 0.0,
                                                        "sigmoid_threshold": 0.45})).eval()
    ids = torch.randint(0, 128, (1, 20))
    with torch.no_grad():
        full = model(input_ids=ids).logits
        cache = HybridCache()
        out = model(input_ids=ids[:, :11], past_key_values=cache, use_cache=True)
        steps = [out.logits[:, -1]]
        for t in range(11, 20):
            out = model(input_ids=ids[:, t:t + 1], past_key_values=cache, use_cache=True)
            steps.append(out.logits[:, -1])
    got = torch.stack(steps, dim=1)
    assert torch.allclose(got, full[:, 10:], atol=2e-4), float((got - full[:, 10:]).abs().max())
    assert ("l2a_global", 0) in cache.attention and cache.attention[0][0].shape[1] <= 6


def test_vendor_multimodal_plugins_expand_placeholders():
    from PIL import Image
    from hybrid_model_factory_b200.data.mm_plugin import get_mm_plugin
    from hybrid_model_factory_b200.data.mm_plugin_zoo import InternVLPlugin, TowerConfig, select_best_resolution
    wide, square = Image.new("RGB", (640, 320), (200, 10, 10)), Image.new("RGB", (100, 100))
    msgs = [{"role": "user", "content": "look <image> and <image>"}, {"role": "assistant", "content": "ok"}]
    count = lambda out, tok: out[0]["content"].count(tok)  # noqa: E731
    # llava: fixed 24 x 24 = 576 tokens per image
    p = get_mm_plugin("llava", image_token="<im>")
    assert count(p.process_messages(msgs, [wide, square]), "<im>") == 2 * 576
    assert p.get_mm_inputs([wide, square])["pixel_values"].shape == (2, 3, 336, 336)
    # llava-next: base + un-padded tiles + a newline token per row; a 2:1 image picks the 336 x 672 canvas
    p = get_mm_plugin("llava_next", image_token="<im>")
    assert select_best_resolution((320, 640), TowerConfig().grid_pinpoints) == (336, 672)
    assert p._counts(320, 640, TowerConfig()) == 576 + 24 * 48 + 24
    mm = p.get_mm_inputs([wide, square])
    assert mm["pixel_values"].shape[:2] == (2, 3) and mm["image_sizes"].tolist() == [[320, 640], [100, 100]]
    # pixtral: rows of patches separated by breaks, one end marker per image
    p = get_mm_plugin("pixtral", image_token="[IMG]")
    out = p.process_messages(msgs, [wide, square])
    assert count(out, "[IMG_END]") == 2 and count(out, "[IMG]") == 40 * 20 + 7 * 7
    assert count(out, "[IMG_BREAK]") == 19 + 6
    # intern-vl: the 2:1 image is cut into a 2 x 1 ... grid of 448-pixel tiles plus a thumbnail, 256 tokens each
    a, b = InternVLPlugin.tile_grid(320, 640, TowerConfig(image_size=448))
    assert a == 2 * b
    p = get_mm_plugin("intern_vl", image_token="<ctx>")
    out = p.process_messages(msgs, [wide, square])
    mm = p.get_mm_inputs([wide, square])
    assert count(out, "<ctx>") == 256 * int(mm["image_num_patches"].sum()) and count(out, "<img>") == 2
    assert mm["pixel_values"].shape[0] == int(mm["image_num_patches"].sum())
    # gemma3: 256 soft tokens between the markers
    p = get_mm_plugin("gemma3", image_token="<soft>")
    out = p.process_messages(msgs, [wide, square])
    assert count(out, "<soft>") == 512 and count(out, "<start_of_image>") == 2
    # paligemma: placeholders vanish from the text, image tokens lead the ids and carry no loss
    class Tok:
        def convert_tokens_to_ids(self, t):
            return 99
    p = get_mm_plugin("paligemma", image_token="<image>")
    out = p.process_messages(msgs, [wide, square])
    assert "<image>" not in out[0]["content"]
    ids, labels = p.process_token_ids([1, 2, 3], [1, 2, 3], [wide], tokenizer=Tok())
    assert ids[:256] == [99] * 256 and labels[:256] == [-100] * 256 and ids[256:] == [1, 2, 3]
    # mllama: one token per image and a mask that lets each token see the images before it
    p = get_mm_plugin("mllama", image_token="<|image|>")
    assert count(p.process_messages(msgs, [wide, square]), "<|image|>") == 2
    mask = p.get_mm_inputs([wide], batch_ids=[[5, 7, 8, 7, 9]], image_token_id=7)["cross_attention_mask"]
    assert mask[0, :, 0].tolist() == [0, 1, 1, 1, 1] and mask[0, :, 1].tolist() == [0, 0, 0, 1, 1]
    # video-llava and glm4v
    p = get_mm_plugin("video_llava", image_token="<im>", video_token="<vid>")
    vm = [{"role": "user", "content": "<video> what happens?"}]
    assert p.process_messages(vm, [], [[square] * 20])[0]["content"].count("<vid>") == 8 * 257
    assert p.get_mm_inputs([], [[square] * 20])["pixel_values_videos"].shape == (1, 8, 3, 224, 224)
    p = get_mm_plugin("glm4v", image_token="<|image|>", video_token="<|video|>")
    out = p.process_messages(msgs, [wide, square])
    assert count(out, "<|begin_of_image|>") == 2 and count(out, "<|image|>") > 2


def test_vision_language_freezing_options():
    from hybrid_model_factory_b200.models.vl import HybridVLForConditionalGeneration, apply_vl_freezing

    class Tower(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.blocks = torch.nn.Linear(12, 16)
            self.merger = torch.nn.Linear(16, 64)

        def forward(self, px, grid_thw=None):
            return self.merger(self.blocks(px))
    model = HybridVLForConditionalGeneration(_cfg("*-GDN"), vision_tower=Tower(), image_token_id=5)
    c = apply_vl_freezing(model)                                               # defaults: only the language model trains
    assert c["vision_tower"] == 0 and c["projector"] == 0 and c["language_model"] > 0
    c = apply_vl_freezing(model, freeze_multi_modal_projector=False, freeze_language_model=True)
    assert c == {"vision_tower": 0, "projector": 16 * 64 + 64, "language_model": 0}
    assert model.visual.merger.weight.requires_grad and not model.visual.blocks.weight.requires_grad
    c = apply_vl_freezing(model, freeze_vision_tower=False)
    assert c["vision_tower"] == 12 * 16 + 16 and c["projector"] == 0
    ids = torch.tensor([[1, 5, 5, 2, 3]])
    out = model(ids, labels=ids, pixel_values=torch.randn(2, 12))
    out.loss.backward()
    assert model.visual.blocks.weight.grad is not None and model.visual.merger.weight.grad is None


def test_gptq_and_awq_checkpoints_expand_on_load(tmp_path):
    """GPTQ packs inputs into words (zeros stored minus one, optional ``g_idx``), AWQ packs outputs in its interleaved
    order: both are unpacked with plain integer arithmetic here and compared against the hand-built integers; a model
    exported in either layout loads through the ordinary path and stays close to the original."""
    from hybrid_model_factory_b200.utils import checkpoint_io
    from hybrid_model_factory_b200.utils.export import export
    from hybrid_model_factory_b200.utils.quant_loaders import (AWQ_ORDER, dequantize_awq, dequantize_gptq, detect_method,
                                                               expand_quantized_state, pack_awq, pack_gptq)
    torch.manual_seed(0)
    n_in, n_out, group = 64, 16, 32
    q = torch.randint(0, 16, (n_in, n_out))
    z = torch.randint(1, 16, (n_in // group, n_out))
    s = (torch.rand(n_in // group, n_out) * 0.1 + 0.01).half()
    g = torch.arange(n_in) // group
    want = ((q - z[g]).float() * s.float()[g]).t()
    # GPTQ by hand: word r of column o holds inputs 8r .. 8r+7, low nibble first; zeros minus one, packed over outputs
    qw = torch.zeros(n_in // 8, n_out, dtype=torch.int64)
    for i in range(n_in):
        qw[i // 8] |= q[i] << (4 * (i % 8))
    qz = torch.zeros(n_in // group, n_out // 8, dtype=torch.int64)
    for o in range(n_out):
        qz[:, o // 8] |= (z[:, o] - 1) << (4 * (o % 8))
    to32 = lambda t: torch.where(t >= 2 ** 31, t - 2 ** 32, t).to(torch.int32)  # noqa: E731
    got = dequantize_gptq(to32(qw), to32(qz), s, None, 4, torch.float32)
    assert torch.equal(got, want)
    perm = torch.randperm(n_in)                                   # act-order: rows visit the groups in any order
    got = dequantize_gptq(to32(qw), to32(qz), s, g[perm].int(), 4, torch.float32)
    assert torch.equal(got, ((q - z[g[perm]]).float() * s.float()[g[perm]]).t())
    # AWQ by hand: nibble i of word c holds output 8c + AWQ_ORDER[i]
    aw = torch.zeros(n_in, n_out // 8, dtype=torch.int64)
    az = torch.zeros(n_in // group, n_out // 8, dtype=torch.int64)
    for c in range(n_out // 8):
        for i, col in enumerate(AWQ_ORDER):
            aw[:, c] |= q[:, 8 * c + col] << (4 * i)
            az[:, c] |= z[:, 8 * c + col] << (4 * i)
    assert torch.equal(dequantize_awq(to32(aw), to32(az), s, 4, group, torch.float32), want)
    # the packers invert the readers, and the state-level pass names the method from the shapes
    w = torch.randn(48, 128)
    for pack, name in ((pack_gptq, "gptq"), (pack_awq, "awq")):
        st = {f"l.{k}": v for k, v in pack(w, 4, 32).items()}
        st["l.bias"] = torch.zeros(48)
        assert detect_method(st) == name
        back = expand_quantized_state(st, dtype=torch.float32)
        assert set(back) == {"l.weight", "l.bias"}
        assert (back["l.weight"] - w).abs().max() < (w.max() - w.min()) / 15 * 0.51 + 1e-2
    # a whole model through `hmf export --quantize gptq|awq` and back
    model = build_model(_cfg("*-GDN", hidden_size=128, intermediate_size=512)).eval()
    ids = torch.randint(0, 128, (1, 10))
    ref = model(input_ids=ids).logits
    checkpoint_io.save_pretrained(model, str(tmp_path / "src"))
    for method in ("gptq", "awq"):
        dst = tmp_path / method
        export(str(tmp_path / "src"), str(dst), quantize=method, group_size=64)
        names = [n for n, _ in checkpoint_io.iter_tensors(str(dst))]
        assert any(n.endswith(".qzeros") for n in names)
        import json as _json
        assert _json.load(open(dst / "config.json"))["quantization_config"]["quant_method"] == method
        again = checkpoint_io.from_pretrained(str(dst), dtype=torch.float32).eval()
        err = (again(input_ids=ids).logits - ref).abs().max() / ref.abs().max()
        assert err < 0.25, (method, float(err))


def test_mixture_of_depths_routes_tokens_and_decodes_causally(tmp_path):
    """Routed layers process the picked tokens only (the rest keep their residual stream), the router trains through
    its gate and its top-k prediction loss, decoding with a cache follows the same causal rule as a full forward in
    eval mode, and a saved model comes back with its routers."""
    from hybrid_model_factory_b200.models.cache import HybridCache
    from hybrid_model_factory_b200.models.mod import apply_mixture_of_depths, mod_aux_loss
    from hybrid_model_factory_b200.utils import checkpoint_io
    torch.manual_seed(0)
    model = build_model(_cfg("*-GDN-*-GDN"))
    assert apply_mixture_of_depths(model, capacity=0.25) == [1, 3]
    ids = torch.randint(0, 128, (2, 16))
    model.train()
    out = model(input_ids=ids, labels=ids)
    out.loss.backward()
    assert mod_aux_loss(model) is not None
    for i in (1, 3):
        assert model.model.layers[i].mod_router.weight.grad.abs().sum() > 0
    # one routed layer by hand, eval rule: tokens with a positive score are processed as a subsequence of their own
    model.eval()
    layer = model.model.layers[1]
    x = torch.randn(1, 12, model.config.hidden_size)
    with torch.no_grad():
        scores = torch.nn.functional.linear(x, layer.mod_router.weight).squeeze(-1)
        keep = (scores > 0)[0]
        assert 0 < int(keep.sum()) < 12
        got, _ = layer(x)
        sub, _ = layer._mod_inner(x[:, keep])
        want = x.clone()
        want[:, keep] += (sub - x[:, keep]) * torch.sigmoid(scores[:, keep]).unsqueeze(-1)
    assert torch.allclose(got, want, atol=1e-5)
    assert torch.equal(got[:, ~keep], x[:, ~keep])
    # full forward == prefill + token-by-token decode
    one = ids[:1]
    with torch.no_grad():
        full = model(input_ids=one).logits
        cache = HybridCache()
        o = model(input_ids=one[:, :9], past_key_values=cache, use_cache=True)
        steps = [o.logits[:, -1]]
        for t in range(9, 16):
            steps.append(model(input_ids=one[:, t:t + 1], past_key_values=cache, use_cache=True).logits[:, -1])
    assert torch.allclose(torch.stack(steps, 1), full[:, 8:], atol=2e-4)
    # the routers travel with the checkpoint
    checkpoint_io.save_pretrained(model, str(tmp_path / "m"))
    again = checkpoint_io.from_pretrained(str(tmp_path / "m"), dtype=torch.float32).eval()
    assert hasattr(again.model.layers[3], "mod_router")
    with torch.no_grad():
        assert torch.allclose(again(input_ids=one).logits, full, atol=1e-5)


def test_audio_plugins_log_mel_and_token_expansion(tmp_path):
    """A one-second tone: 100 valid frames of 3000, 25 audio tokens, the energy sits in the mel band of the tone; the
    features equal the ``transformers`` Whisper extractor's; ``.wav`` files are read and resampled; the omni plugin
    handles an image and an audio clip in one message."""
    import math
    import wave
    import numpy as np
    from PIL import Image
    from hybrid_model_factory_b200.data.mm_plugin import get_mm_plugin
    from hybrid_model_factory_b200.data.mm_plugin_audio import (AudioFrontendConfig, audio_token_count, load_audio,
                                                               log_mel, mel_filterbank)
    cfg = AudioFrontendConfig()
    t = torch.arange(16000) / 16000.0
    tone = 0.5 * torch.sin(2 * math.pi * 440.0 * t)
    feats, mask = log_mel(tone, cfg)
    assert feats.shape == (128, 3000) and int(mask.sum()) == 100 and audio_token_count(100) == 25
    fb = mel_filterbank(128, 400, 16000)
    assert fb.shape == (128, 201) and fb.min() >= 0
    band = int(feats[:, :100].mean(1).argmax())
    centre_hz = float((fb[band] * torch.linspace(0, 8000, 201)).sum() / fb[band].sum())
    assert abs(centre_hz - 440.0) < 40.0
    try:
        from transformers import WhisperFeatureExtractor
        theirs = WhisperFeatureExtractor(feature_size=128)(tone.numpy(), sampling_rate=16000, return_tensors="pt",
                                                           return_attention_mask=True)
        assert torch.allclose(feats, theirs["input_features"][0], atol=2e-3)
        assert torch.equal(mask, theirs["attention_mask"][0].long())
    except ImportError:
        pass
    # 8 kHz 16-bit stereo file -> mono 16 kHz
    path = str(tmp_path / "a.wav")
    pcm = (np.stack([tone[::2].numpy(), tone[::2].numpy()], 1) * 32767).astype("<i2")
    with wave.open(path, "wb") as f:
        f.setnchannels(2), f.setsampwidth(2), f.setframerate(8000)
        f.writeframes(pcm.tobytes())
    wav = load_audio(path, 16000)
    assert wav.numel() == 16000 and (wav - tone).abs().mean() < 0.02
    assert load_audio({"array": tone.numpy(), "sampling_rate": 16000}, 16000).shape == (16000,)
    # text expansion
    plug = get_mm_plugin("qwen2_audio", audio_token="<|AUDIO|>")
    msgs = [{"role": "user", "content": "listen: <audio> and <audio>"}, {"role": "assistant", "content": "ok"}]
    out = plug.process_messages(msgs, audios=[path, (tone[:8000], 16000)])
    assert out[0]["content"] == ("listen: <|audio_bos|>" + "<|AUDIO|>" * 25 + "<|audio_eos|> and <|audio_bos|>"
                                 + "<|AUDIO|>" * audio_token_count(50) + "<|audio_eos|>")
    mm = plug.get_mm_inputs(audios=[path, (tone[:8000], 16000)])
    assert mm["input_features"].shape == (2, 128, 3000) and mm["feature_attention_mask"].sum(-1).tolist() == [100, 50]
    import pytest
    with pytest.raises(ValueError, match="placeholders"):
        plug.process_messages(msgs, audios=[path])
    omni = get_mm_plugin("qwen2_omni", image_token="<|IMAGE|>", video_token="<|VIDEO|>", audio_token="<|AUDIO|>")
    img = Image.fromarray((np.random.rand(56, 84, 3) * 255).astype("uint8"))
    both = omni.process_messages([{"role": "user", "content": "<image> then <audio>"}], images=[img], audios=[path])
    assert both[0]["content"].count("<|IMAGE|>") == 6 and both[0]["content"].count("<|AUDIO|>") == 25
    mm = omni.get_mm_inputs(images=[img], audios=[path])
    assert set(mm) >= {"pixel_values", "image_grid_thw", "input_features", "feature_attention_mask"}


def test_qlora_quantised_base_trains_adapters_only():
    """4-bit normal-quantile and 8-bit integer codes reproduce the weight within their step sizes; the product's
    gradient reaches the input and the adapters, never the base; merging returns ordinary layers."""
    from hybrid_model_factory_b200.train.adapters import apply_lora, merge_lora
    from hybrid_model_factory_b200.train.qlora import (NF4_LEVELS, QuantizedLinear, quantize_adapter_bases,
                                                       quantized_bytes)
    torch.manual_seed(0)
    lin = torch.nn.Linear(128, 48, bias=True)
    w = lin.weight.detach()
    q4 = QuantizedLinear(lin, 4, "nf4", 64)
    assert q4.qweight.shape == (48, 64) and q4.qweight.dtype == torch.uint8 and q4.scales.shape == (48, 2)
    gap = max(b - a for a, b in zip(NF4_LEVELS[:-1], NF4_LEVELS[1:]))
    absmax = w.reshape(48, 2, 64).abs().amax(-1, keepdim=True)
    err = (q4.weight - w).reshape(48, 2, 64).abs()
    assert (err <= absmax * (gap / 2 + 0.01)).all()             # nearest level (+ bf16 rounding of the scale)
    q8 = QuantizedLinear(lin, 8)
    assert (q8.weight - w).abs().max() <= absmax.max() / 127 * 0.51 + absmax.max() * 0.005
    x = torch.randn(5, 128, requires_grad=True)
    y = q4(x)
    ref = torch.nn.functional.linear(x, q4.weight, lin.bias)
    assert torch.allclose(y, ref, atol=1e-5)
    y.sum().backward()
    assert torch.allclose(x.grad, torch.ones(5, 48) @ q4.weight, atol=1e-5)
    assert not any(p.requires_grad for p in q4.parameters())
    # through a model
    model = build_model(_cfg("*-GDN", hidden_size=128, intermediate_size=256))
    dense = sum(p.numel() * 4 for n, p in model.named_parameters() if "proj" in n and "lm_head" not in n)
    wrapped = apply_lora(model, rank=4)
    done = quantize_adapter_bases(model, 4)
    assert set(done) == set(wrapped) and quantized_bytes(model) < dense / 6
    ids = torch.randint(0, 128, (2, 10))
    model.train()
    model(input_ids=ids, labels=ids).loss.backward()
    trainable = [n for n, p in model.named_parameters() if p.requires_grad]
    assert trainable and all("lora_" in n for n in trainable)
    assert all(p.grad is not None for n, p in model.named_parameters() if n.endswith("lora_B"))
    model.eval()
    with torch.no_grad():
        before = model(input_ids=ids).logits
        assert merge_lora(model) == len(wrapped)
        assert not any(isinstance(m, QuantizedLinear) for m in model.modules())
        assert torch.allclose(model(input_ids=ids).logits, before, atol=1e-4)


@pytest.mark.parametrize("pattern", ["*-GDN-GKA-M2", "SWA-BMF-L2A-*"])
def test_meta_device_loading_matches_default_loading(tmp_path, pattern):
    """A model built without storage and filled from the checkpoint computes what the ordinarily loaded one does (every
    tensor the forward pass needs is a parameter or is recomputed: rotary frequencies stay fp32 under a bf16 cast), tied
    embeddings stay tied, and an incomplete checkpoint is refused."""
    from hybrid_model_factory_b200.layers.common import RotaryEmbedding
    from hybrid_model_factory_b200.utils import checkpoint_io
    torch.manual_seed(0)
    extra = {"l2a_config": {"sliding_window": 6, "leak_prob": 0.0}} if "L2A" in pattern else {}
    model = build_model(_cfg(pattern, tie_word_embeddings=True, **extra)).eval()
    model.lm_head.weight = model.model.embed_tokens.weight
    checkpoint_io.save_pretrained(model, str(tmp_path / "m"))
    ids = torch.randint(0, 128, (1, 14))
    a = checkpoint_io.from_pretrained(str(tmp_path / "m"), dtype=torch.float32).eval()
    b = checkpoint_io.from_pretrained(str(tmp_path / "m"), dtype=torch.float32, init="meta").eval()
    with torch.no_grad():
        assert torch.allclose(a(input_ids=ids).logits, b(input_ids=ids).logits, atol=1e-5)
    assert b.lm_head.weight is b.model.embed_tokens.weight
    assert not any(p.is_meta for p in b.parameters()) and not any(t.is_meta for t in b.buffers())
    half = checkpoint_io.from_pretrained(str(tmp_path / "m"), dtype=torch.bfloat16, init="meta")
    rot = [m for m in half.modules() if isinstance(m, RotaryEmbedding)]
    assert rot and all(m.inv_freq.dtype == torch.float32 for m in rot)
    ref_inv = RotaryEmbedding(rot[0].dim, rot[0].theta, rot[0].scaling, rot[0].max_position).inv_freq
    assert torch.equal(rot[0].inv_freq, ref_inv)
    # drop one tensor from the checkpoint: meta loading cannot invent it
    from safetensors.torch import load_file, save_file
    f = next(p for p in (tmp_path / "m").iterdir() if p.suffix == ".safetensors")
    sd = load_file(str(f))
    sd.pop(next(k for k in sd if k.endswith("mlp.up_proj.weight")))
    save_file(sd, str(f))
    with pytest.raises(KeyError, match="not in the checkpoint"):
        checkpoint_io.from_pretrained(str(tmp_path / "m"), dtype=torch.float32, init="meta", allow_missing=True)


def test_gptq_awq_unpacking_agrees_with_an_independent_packer():
    """The integer layouts, checked against the reference packers of an installed serving library (skipped without it)."""
    quant_utils = pytest.importorskip("vllm.model_executor.layers.quantization.utils.quant_utils")
    from hybrid_model_factory_b200.utils.quant_loaders import _awq_natural, _unpack
    torch.manual_seed(0)
    k, n = 64, 32
    q = torch.randint(0, 16, (k, n), dtype=torch.int32)
    assert torch.equal(_unpack(quant_utils.gptq_pack(q, 4, k, n), 4, dim=0), q)
    assert torch.equal(_awq_natural(_unpack(quant_utils.awq_pack(q, 4, k, n), 4, dim=1), 4), q)
    q8 = torch.randint(0, 256, (k, n), dtype=torch.int32)
    assert torch.equal(_unpack(quant_utils.gptq_pack(q8, 8, k, n), 8, dim=0), q8)


def test_tool_formats_per_model_family():
    """Tool lists, calls and results are written the way each family expects, and the calls a model writes in that
    format are recognised again."""
    import json
    from hybrid_model_factory_b200.data.formats import ByteTokenizer, get_template
    calls = [{"name": "weather", "arguments": {"city": "Oslo"}}, {"name": "time", "arguments": {}}]
    tools = json.dumps([{"name": "weather", "parameters": {"type": "object"}}])
    msgs = [{"role": "user", "content": "q"}, {"role": "function", "content": json.dumps(calls)},
            {"role": "observation", "content": "rain"}]
    expect = {
        "qwen3": ('<tool_call>\n{"name": "weather", "arguments": {"city": "Oslo"}}\n</tool_call>\n<tool_call>\n'
                  '{"name": "time", "arguments": {}}\n</tool_call>', "<tool_response>\nrain\n</tool_response>", "<tools>"),
        "llama3": ('{"name": "weather", "parameters": {"city": "Oslo"}}; {"name": "time", "parameters": {}}', "rain",
                   "You have access to the following functions"),
        "mistral": ('[TOOL_CALLS] [{"name": "weather", "arguments": {"city": "Oslo"}}, {"name": "time", "arguments": {}}]',
                    '[TOOL_RESULTS] {"content": rain}[/TOOL_RESULTS]', "[AVAILABLE_TOOLS]"),
        "glm4_moe": ('weather\n{"city": "Oslo"}\ntime\n{}', "<|observation|>\nrain", "可用工具"),
    }
    for name, (call_text, result_text, tools_mark) in expect.items():
        tpl = get_template(name)
        turns, system = tpl.normalise(msgs, "sys", tools)
        assert turns[1] == {"role": "assistant", "content": call_text}, name
        assert turns[2] == {"role": "user", "content": result_text}, name
        assert system.startswith("sys") and tools_mark in system and '"weather"' in system, name
        assert tpl.encode_multiturn(ByteTokenizer(), turns + [{"role": "assistant", "content": ""}], system)
    # recognition of generated calls
    assert get_template("qwen3").extract_tool_calls("ok " + expect["qwen3"][0]) == ("ok", calls)
    assert get_template("llama3").extract_tool_calls(expect["llama3"][0]) == ("", calls)
    assert get_template("llama3").extract_tool_calls("just text") == ("just text", [])
    assert get_template("mistral").extract_tool_calls("sure. " + expect["mistral"][0]) == ("sure.", calls)
    assert get_template("glm4_moe").extract_tool_calls('weather\n{"city": "Oslo"}') == ("", calls[:1])
    assert get_template("glm4_moe").extract_tool_calls("no call here") == ("no call here", [])
