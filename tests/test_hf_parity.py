"""Checkpoints written by the Hugging Face implementations of the base architectures load into this package's models
and give the same logits (fp32, CPU, tiny random models).  Covers the config dialects of recent ``transformers``
(``rope_parameters``, ``num_local_experts``, ``layer_types`` with native sliding-window layers) and every rotary scaling
rule the base families use."""
import pytest
import torch

from hybrid_model_factory_b200.utils import checkpoint_io

T = pytest.importorskip("transformers")

COMMON = dict(vocab_size=160, hidden_size=64, intermediate_size=128, num_hidden_layers=3, num_attention_heads=4,
              num_key_value_heads=2, max_position_embeddings=512)

CASES = {
    "qwen3": ("Qwen3Config", "Qwen3ForCausalLM", dict(head_dim=16, rope_theta=10000.0)),
    "qwen3_tied": ("Qwen3Config", "Qwen3ForCausalLM", dict(head_dim=16, tie_word_embeddings=True)),
    "qwen3_yarn": ("Qwen3Config", "Qwen3ForCausalLM", dict(head_dim=16, rope_parameters={
        "rope_type": "yarn", "rope_theta": 10000.0, "factor": 4.0, "original_max_position_embeddings": 128})),
    "qwen3_native_sliding_layers": ("Qwen3Config", "Qwen3ForCausalLM", dict(
        head_dim=16, sliding_window=8, use_sliding_window=True, max_window_layers=1,
        layer_types=["full_attention", "sliding_attention", "sliding_attention"])),
    "qwen2": ("Qwen2Config", "Qwen2ForCausalLM", dict(rope_theta=20000.0)),
    "qwen2_window_switched_off": ("Qwen2Config", "Qwen2ForCausalLM", dict(sliding_window=8, use_sliding_window=False)),
    "llama3_rope": ("LlamaConfig", "LlamaForCausalLM", dict(rope_parameters={
        "rope_type": "llama3", "rope_theta": 50000.0, "factor": 8.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
        "original_max_position_embeddings": 64})),
    "llama_with_biases": ("LlamaConfig", "LlamaForCausalLM", dict(attention_bias=True, mlp_bias=True, rope_theta=10000.0)),
    "llama_linear_rope": ("LlamaConfig", "LlamaForCausalLM", dict(rope_parameters={
        "rope_type": "linear", "rope_theta": 10000.0, "factor": 2.0})),
    "qwen3_attention_bias": ("Qwen3Config", "Qwen3ForCausalLM", dict(head_dim=16, attention_bias=True)),
    "mistral_sliding": ("MistralConfig", "MistralForCausalLM", dict(head_dim=16, sliding_window=8)),
    "qwen3_moe": ("Qwen3MoeConfig", "Qwen3MoeForCausalLM", dict(
        head_dim=16, num_experts=4, num_experts_per_tok=2, moe_intermediate_size=32, decoder_sparse_step=1,
        norm_topk_prob=True, mlp_only_layers=[])),
    "qwen3_moe_mixed_dense": ("Qwen3MoeConfig", "Qwen3MoeForCausalLM", dict(
        head_dim=16, num_experts=4, num_experts_per_tok=2, moe_intermediate_size=32, decoder_sparse_step=2,
        norm_topk_prob=False, mlp_only_layers=[])),
}


@pytest.mark.parametrize("name", sorted(CASES))
def test_logits_equal_the_hugging_face_model(tmp_path, name):
    cfg_name, model_name, extra = CASES[name]
    if not hasattr(T, cfg_name) or not hasattr(T, model_name):
        pytest.skip(f"this transformers has no {model_name}")
    torch.manual_seed(0)
    try:
        hf = getattr(T, model_name)(getattr(T, cfg_name)(**{**COMMON, **extra})).eval()
    except TypeError as e:                      # a config dialect this transformers version does not speak
        pytest.skip(str(e))
    hf.save_pretrained(str(tmp_path / "hf"), safe_serialization=True)
    own = checkpoint_io.from_pretrained(str(tmp_path / "hf"), dtype=torch.float32).eval()      # strict: every tensor used
    assert not own._load_report["unexpected"]
    ids = torch.randint(0, COMMON["vocab_size"], (2, 40))
    with torch.no_grad():
        want, got = hf(input_ids=ids).logits, own(input_ids=ids).logits
    assert torch.allclose(got, want, atol=2e-5), float((got - want).abs().max())
    # the checkpoint written by this package reloads to the same function (native windows, rotary settings kept)
    checkpoint_io.save_pretrained(own, str(tmp_path / "own"))
    again = checkpoint_io.from_pretrained(str(tmp_path / "own"), dtype=torch.float32, init="meta").eval()
    with torch.no_grad():
        assert torch.allclose(again(input_ids=ids).logits, want, atol=2e-5)
    # and decoding with the cache follows the same function (windowed layers included)
    with torch.no_grad():
        gen = own.generate(ids[:1, :20], max_new_tokens=4)
        ref = hf.generate(ids[:1, :20], max_new_tokens=4, do_sample=False)
    assert gen[0, 20:].tolist() == ref[0, 20:24].tolist()


def test_converted_qwen3_next_equals_the_hugging_face_model(tmp_path):
    """A Qwen3-Next checkpoint (Gated DeltaNet layers with fewer key than value heads, gated attention with partial
    rotary embedding, zero-centred norms, experts + shared expert) through ``hmf convert-qwen-gdn``: same logits, same
    greedy continuation with the recurrent cache."""
    if not hasattr(T, "Qwen3NextForCausalLM"):
        pytest.skip("this transformers has no Qwen3-Next")
    from hybrid_model_factory_b200.priming.convert_qwen_gdn import convert_checkpoint
    torch.manual_seed(0)
    cfg = T.Qwen3NextConfig(
        vocab_size=160, hidden_size=64, intermediate_size=128, num_hidden_layers=4, num_attention_heads=4,
        num_key_value_heads=2, head_dim=16, max_position_embeddings=512, linear_num_key_heads=2,
        linear_num_value_heads=4, linear_key_head_dim=16, linear_value_head_dim=16, linear_conv_kernel_dim=4,
        num_experts=4, num_experts_per_tok=2, moe_intermediate_size=32, shared_expert_intermediate_size=32,
        decoder_sparse_step=1, norm_topk_prob=True, full_attention_interval=4, partial_rotary_factor=0.25,
        mlp_only_layers=[])
    hf = T.Qwen3NextForCausalLM(cfg).eval()
    with torch.no_grad():                       # norms, biases and decay parameters away from their initial values
        for _, p in hf.named_parameters():
            if p.dim() == 1:
                p.add_(torch.randn_like(p) * 0.1)
    hf.save_pretrained(str(tmp_path / "hf"), safe_serialization=True)
    report = convert_checkpoint(str(tmp_path / "hf"), str(tmp_path / "own"), None, False, torch.float32)
    assert not report["dropped"] and not report["missing"]
    own = checkpoint_io.from_pretrained(str(tmp_path / "own"), dtype=torch.float32).eval()
    assert own.config.hybrid_override_pattern == "GDN-GDN-GDN-*"
    ids = torch.randint(0, 160, (2, 40))
    with torch.no_grad():
        want, got = hf(input_ids=ids).logits, own(input_ids=ids).logits
    assert torch.allclose(got, want, atol=2e-5), float((got - want).abs().max())
    with torch.no_grad():
        gen = own.generate(ids[:1, :24], max_new_tokens=5)
        ref = hf.generate(ids[:1, :24], max_new_tokens=5, do_sample=False)
    assert gen[0, 24:].tolist() == ref[0, 24:29].tolist()


def test_ministral3_long_context_temperature_in_model_and_engine(tmp_path):
    """Ministral 3: YaRN with equal magnitude corrections (attention factor 1) and a query temperature that grows past
    the original context.  A tiny original context makes both matter; the forward pass equals Hugging Face's, and the
    serving engine's decode path generates what the model's own generation does."""
    if not hasattr(T, "Ministral3ForCausalLM"):
        pytest.skip("this transformers has no Ministral 3")
    from hybrid_model_factory_b200.serving.engine import SamplingParams, ServingEngine
    torch.manual_seed(0)
    cfg = T.Ministral3Config(**COMMON, head_dim=16, sliding_window=None, rope_parameters={
        "rope_type": "yarn", "rope_theta": 1e6, "factor": 16.0, "original_max_position_embeddings": 16,
        "beta_fast": 32.0, "beta_slow": 1.0, "mscale_all_dim": 1.0, "mscale": 1.0, "llama_4_scaling_beta": 0.1})
    hf = T.Ministral3ForCausalLM(cfg).eval()
    hf.save_pretrained(str(tmp_path / "hf"), safe_serialization=True)
    own = checkpoint_io.from_pretrained(str(tmp_path / "hf"), dtype=torch.float32).eval()
    ids = torch.randint(0, COMMON["vocab_size"], (2, 60))
    with torch.no_grad():
        want, got = hf(input_ids=ids).logits, own(input_ids=ids).logits
    assert torch.allclose(got, want, atol=2e-5), float((got - want).abs().max())
    prompt = ids[0, :40].tolist()
    with torch.no_grad():
        ref = hf.generate(ids[:1, :40], max_new_tokens=6, do_sample=False)[0, 40:].tolist()
    eng = ServingEngine(own, block_size=8, num_blocks=32, max_num_seqs=2, max_num_batched_tokens=64, max_model_len=128)
    assert eng.generate([prompt], SamplingParams(max_new_tokens=6))[0] == ref


def test_image_sizing_and_patch_layout_agree_with_transformers():
    """The pixel-budget resize, the any-resolution canvas choice, the LLaVA-NeXT token count and the Qwen2-VL patch
    layout against the ``transformers`` processors (each part skipped when that processor is not importable)."""
    import random
    import numpy as np
    from PIL import Image
    from hybrid_model_factory_b200.data.mm_plugin import get_mm_plugin, smart_resize
    from hybrid_model_factory_b200.data.mm_plugin_zoo import LlavaNextPlugin, TowerConfig, select_best_resolution
    random.seed(0)
    checked = 0
    try:
        from transformers.models.qwen2_vl.image_processing_qwen2_vl import smart_resize as hf_resize
        for _ in range(500):
            h, w = random.randint(28, 3000), random.randint(28, 3000)
            if max(h, w) / min(h, w) <= 200:
                assert tuple(smart_resize(h, w, 28, 56 * 56, 28 * 28 * 1280)) == tuple(hf_resize(h, w, 28, 56 * 56, 28 * 28 * 1280))
        checked += 1
    except ImportError:
        pass
    pins = [(336, 672), (672, 336), (672, 672), (1008, 336), (336, 1008)]
    try:
        from transformers.image_processing_utils import select_best_resolution as hf_best
        for _ in range(500):
            size = (random.randint(50, 2000), random.randint(50, 2000))
            assert tuple(select_best_resolution(size, pins)) == tuple(hf_best(size, pins))
        checked += 1
    except ImportError:
        pass
    try:
        from transformers import LlavaNextProcessor
        proc = LlavaNextProcessor.__new__(LlavaNextProcessor)
        proc.patch_size, proc.num_additional_image_tokens, proc.vision_feature_select_strategy = 14, 0, "default"
        proc.image_processor = type("IP", (), {"image_grid_pinpoints": [list(p) for p in pins],
                                               "size": {"shortest_edge": 336}, "crop_size": {"height": 336, "width": 336}})()
        plug, tower = LlavaNextPlugin("<image>", None, None), TowerConfig()
        for _ in range(300):
            h, w = random.randint(40, 2500), random.randint(40, 2500)
            assert plug._counts(h, w, tower) == proc._get_number_of_features(h, w, 336, 336), (h, w)
        checked += 1
    except (ImportError, AttributeError):
        pass
    try:
        from transformers.models.qwen2_vl.image_processing_qwen2_vl import Qwen2VLImageProcessor
        img = Image.fromarray((np.random.default_rng(0).random((173, 311, 3)) * 255).astype("uint8"))
        mine = get_mm_plugin("qwen2_vl", image_token="<|image_pad|>", video_token="<|video_pad|>").get_mm_inputs(images=[img])
        theirs = Qwen2VLImageProcessor()(images=[img], return_tensors="pt")
        assert mine["image_grid_thw"].tolist() == theirs["image_grid_thw"].tolist()
        assert mine["pixel_values"].shape == theirs["pixel_values"].shape
        assert float((mine["pixel_values"] - theirs["pixel_values"]).abs().max()) < 0.05        # one 8-bit level of the resize
        checked += 1
    except ImportError:
        pass
    try:
        from types import SimpleNamespace
        from transformers.models.pixtral.image_processing_pixtral import get_resize_output_image_size
        from hybrid_model_factory_b200.data.mm_plugin_zoo import PixtralPlugin
        pix, pcfg = PixtralPlugin("[IMG]", None, None), TowerConfig(image_size=1024, patch_size=16)
        for _ in range(500):
            h, w = random.randint(8, 4000), random.randint(8, 4000)
            want = get_resize_output_image_size(np.zeros((h, w, 3), dtype=np.uint8), size=(1024, 1024),
                                                patch_size=(16, 16), input_data_format="channels_last")
            gh, gw = pix._grid(SimpleNamespace(height=h, width=w), pcfg)
            assert (gh * 16, gw * 16) == tuple(want), (h, w)
        checked += 1
    except ImportError:
        pass
    try:
        from transformers.models.got_ocr2.image_processing_got_ocr2 import get_optimal_tiled_canvas
        from hybrid_model_factory_b200.data.mm_plugin_zoo import InternVLPlugin
        icfg = TowerConfig(image_size=448)
        for _ in range(500):
            h, w = random.randint(30, 4000), random.randint(30, 4000)
            assert tuple(InternVLPlugin.tile_grid(h, w, icfg)) == tuple(get_optimal_tiled_canvas((h, w), (448, 448), 1, 12))
        checked += 1
    except ImportError:
        pass
    if not checked:
        pytest.skip("no transformers processor to compare with")


@pytest.mark.parametrize("name", ["qwen3", "qwen3_moe", "mistral_sliding"])
def test_loss_and_gradients_equal_the_hugging_face_model(tmp_path, name):
    """Same next-token loss and the same gradients (fused linear + cross-entropy, attention / MoE backward of this
    package's reference ops against autograd through the Hugging Face modules)."""
    cfg_name, model_name, extra = CASES[name]
    if not hasattr(T, model_name):
        pytest.skip(f"this transformers has no {model_name}")
    torch.manual_seed(0)
    hf = getattr(T, model_name)(getattr(T, cfg_name)(**{**COMMON, **extra})).train()
    hf.save_pretrained(str(tmp_path / "hf"), safe_serialization=True)
    own = checkpoint_io.from_pretrained(str(tmp_path / "hf"), dtype=torch.float32).train()
    ids = torch.randint(0, COMMON["vocab_size"], (2, 24))
    own.config.router_aux_loss_coef = 0.0   # the language-model loss alone (the routers' balancing term is an extra)
    loss_hf = hf(input_ids=ids, labels=ids).loss
    loss_own = own(input_ids=ids, labels=ids).loss
    assert abs(float(loss_hf) - float(loss_own)) < 1e-5
    loss_hf.backward()
    loss_own.backward()
    theirs = dict(hf.named_parameters())
    checked = 0
    for n, p in own.named_parameters():
        if n in theirs and p.grad is not None and theirs[n].grad is not None:
            assert torch.allclose(p.grad, theirs[n].grad, atol=2e-5), (n, float((p.grad - theirs[n].grad).abs().max()))
            checked += 1
    assert checked >= 20


def test_converted_qwen3_next_gradients_equal_the_hugging_face_model(tmp_path):
    """Gated DeltaNet backward (chunked delta rule, gates, short convolutions, gated head norm) and gated attention
    backward against autograd through the Hugging Face modules, parameter by parameter where the names coincide."""
    if not hasattr(T, "Qwen3NextForCausalLM"):
        pytest.skip("this transformers has no Qwen3-Next")
    from hybrid_model_factory_b200.priming.convert_qwen_gdn import convert_checkpoint
    torch.manual_seed(0)
    cfg = T.Qwen3NextConfig(
        vocab_size=160, hidden_size=64, intermediate_size=128, num_hidden_layers=4, num_attention_heads=4,
        num_key_value_heads=2, head_dim=16, max_position_embeddings=512, linear_num_key_heads=2,
        linear_num_value_heads=4, linear_key_head_dim=16, linear_value_head_dim=16, linear_conv_kernel_dim=4,
        num_experts=4, num_experts_per_tok=2, moe_intermediate_size=32, shared_expert_intermediate_size=32,
        decoder_sparse_step=1, norm_topk_prob=True, full_attention_interval=4, partial_rotary_factor=0.25,
        mlp_only_layers=[])
    hf = T.Qwen3NextForCausalLM(cfg).train()
    with torch.no_grad():
        for _, p in hf.named_parameters():
            if p.dim() == 1:
                p.add_(torch.randn_like(p) * 0.1)
    hf.save_pretrained(str(tmp_path / "hf"), safe_serialization=True)
    convert_checkpoint(str(tmp_path / "hf"), str(tmp_path / "own"), None, False, torch.float32)
    own = checkpoint_io.from_pretrained(str(tmp_path / "own"), dtype=torch.float32).train()
    own.config.router_aux_loss_coef = 0.0
    ids = torch.randint(0, 160, (2, 40))
    loss_hf, loss_own = hf(input_ids=ids, labels=ids).loss, own(input_ids=ids, labels=ids).loss
    assert abs(float(loss_hf) - float(loss_own)) < 1e-5
    loss_hf.backward()
    loss_own.backward()
    theirs, mine = dict(hf.named_parameters()), dict(own.named_parameters())
    same = [n for n in mine if n in theirs and mine[n].grad is not None and theirs[n].grad is not None
            and mine[n].shape == theirs[n].shape]
    assert len(same) >= 15
    for n in same:
        assert torch.allclose(mine[n].grad, theirs[n].grad, atol=3e-5), (n, float((mine[n].grad - theirs[n].grad).abs().max()))
    # the Gated DeltaNet layer's own parameters are renamed by the conversion: decay and output projection by hand
    for i in range(3):
        g_hf, g_own = hf.model.layers[i].linear_attn, own.model.layers[i].seq_mixer
        assert torch.allclose(g_own.A_log.grad, g_hf.A_log.grad, atol=3e-5)
        assert torch.allclose(g_own.dt_bias.grad, g_hf.dt_bias.grad, atol=3e-5)
        assert torch.allclose(g_own.o_proj.weight.grad, g_hf.out_proj.weight.grad, atol=3e-5)
        assert torch.allclose(g_own.o_norm.weight.grad, g_hf.norm.weight.grad, atol=3e-5)


def test_serving_engine_generates_what_hugging_face_generates(tmp_path):
    """Continuous batching, paged attention cache, recurrent-state slots, chunked prefill and speculative decoding of
    the serving engine on a converted Qwen3-Next checkpoint: three prompts of different lengths come out token for
    token as Hugging Face ``generate`` produces them one by one."""
    if not hasattr(T, "Qwen3NextForCausalLM"):
        pytest.skip("this transformers has no Qwen3-Next")
    from hybrid_model_factory_b200.priming.convert_qwen_gdn import convert_checkpoint
    from hybrid_model_factory_b200.serving.engine import SamplingParams, ServingEngine
    torch.manual_seed(0)
    cfg = T.Qwen3NextConfig(
        vocab_size=160, hidden_size=64, intermediate_size=128, num_hidden_layers=4, num_attention_heads=4,
        num_key_value_heads=2, head_dim=16, max_position_embeddings=512, linear_num_key_heads=2,
        linear_num_value_heads=4, linear_key_head_dim=16, linear_value_head_dim=16, linear_conv_kernel_dim=4,
        num_experts=4, num_experts_per_tok=2, moe_intermediate_size=32, shared_expert_intermediate_size=32,
        decoder_sparse_step=1, norm_topk_prob=True, full_attention_interval=4, partial_rotary_factor=0.25,
        mlp_only_layers=[])
    hf = T.Qwen3NextForCausalLM(cfg).eval()
    with torch.no_grad():
        for _, p in hf.named_parameters():
            if p.dim() == 1:
                p.add_(torch.randn_like(p) * 0.1)
    hf.save_pretrained(str(tmp_path / "hf"), safe_serialization=True)
    convert_checkpoint(str(tmp_path / "hf"), str(tmp_path / "own"), None, False, torch.float32)
    own = checkpoint_io.from_pretrained(str(tmp_path / "own"), dtype=torch.float32, init="meta").eval()
    g = torch.Generator().manual_seed(3)
    prompts = [torch.randint(0, 160, (n,), generator=g).tolist() for n in (37, 9, 21)]
    want = []
    with torch.no_grad():
        for p in prompts:
            want.append(hf.generate(torch.tensor([p]), max_new_tokens=8, do_sample=False)[0, len(p):].tolist())
    for kwargs, spec in (({"max_num_batched_tokens": 64}, 0), ({"max_num_batched_tokens": 16, "whole_prompts": False}, 0),
                         ({"max_num_batched_tokens": 64}, 3)):
        eng = ServingEngine(own, block_size=8, num_blocks=64, max_num_seqs=4, max_model_len=128, **kwargs)
        got = eng.generate(prompts, SamplingParams(max_new_tokens=8, speculative_tokens=spec))
        assert got == want, (kwargs, spec)
