"""Model-level paths on a GPU in bf16 at kernel-sized shapes: cached generation for every mixer, state composition,
task heads, L2A routing, packed rows.  Each compares the kernel path with the same model's PyTorch path
(``HMF_FORCE_REFERENCE``-style oracle through a float32 CPU copy) or checks internal consistency."""
import copy

import pytest
import torch

from hybrid_model_factory_b200.models.configuration import HybridConfig
from hybrid_model_factory_b200.models.modeling_hybrid import build_model

pytestmark = pytest.mark.gpu


def _cfg(pattern, **kw):
    base = dict(vocab_size=512, hidden_size=512, intermediate_size=1024, num_hidden_layers=len(pattern.split("-")),
                num_attention_heads=4, num_key_value_heads=2, head_dim=128, hybrid_override_pattern=pattern,
                swa_config={"window_size": 64}, bmojo_config={"window_size": 64, "ssm_mixer": "gdn", "tie_attn_weights": False},
                l2a_config={"sliding_window": 64, "leak_prob": 0.0})
    base.update(kw)
    return HybridConfig("hybrid_qwen3", **base)


def _status_ok():
    from hybrid_model_factory_b200.ops import _lib
    torch.cuda.synchronize()
    _lib.assert_status_ok()


@pytest.mark.parametrize("pattern", ["*-GDN", "M2-GKA", "SWA-BMF", "L2A-*"])
def test_cached_generation_matches_full_forward(pattern):
    """Prefill + token-by-token decoding through the hybrid cache gives the logits of one forward over the sequence
    (bf16 tolerance), for every mixer family."""
    torch.manual_seed(0)
    model = build_model(_cfg(pattern)).to("cuda", torch.bfloat16).eval()
    ids = torch.randint(0, 512, (1, 200), device="cuda")
    from hybrid_model_factory_b200.models.cache import HybridCache
    with torch.no_grad():
        full = model(input_ids=ids).logits.float()
        cache = HybridCache()
        out = model(input_ids=ids[:, :160], past_key_values=cache, use_cache=True)
        steps = [out.logits[:, -1].float()]
        for t in range(160, 199):
            out = model(input_ids=ids[:, t:t + 1], past_key_values=cache, use_cache=True)
            steps.append(out.logits[:, -1].float())
    got = torch.stack(steps, 1)
    want = full[:, 159:199]
    rel = (got - want).norm() / want.norm()
    assert rel < 5e-2, float(rel)
    _status_ok()


def test_state_composition_modes_run_on_kernels():
    from hybrid_model_factory_b200.models import composition as C
    torch.manual_seed(0)
    model = build_model(_cfg("*-GDN-M2-GKA")).to("cuda", torch.bfloat16).eval()
    ctx = torch.randint(0, 512, (1, 256), device="cuda")
    q = torch.randint(0, 512, (1, 16), device="cuda")
    ref = model.generate(torch.cat([ctx, q], 1), max_new_tokens=4)[:, 272:]
    one = C.generate_composed(model, ctx, q, num_chunks=1, compose_type="concat_fuse", max_new_tokens=4)
    assert one.shape == ref.shape and one[0, 0] == ref[0, 0]
    for kv in C.KV_MODES:
        for ssm in C.SSM_MODES:
            out = C.generate_composed(model, ctx, q, num_chunks=4, compose_type=f"{kv}_{ssm}", max_new_tokens=3)
            assert out.shape == (1, 3)
    _status_ok()


def test_task_heads_and_packed_rows():
    from hybrid_model_factory_b200.models.heads import build_head_model
    torch.manual_seed(0)
    cfg = _cfg("*-GDN", num_labels=3)
    ids = torch.randint(1, 512, (2, 160), device="cuda")
    for task in ("sequence_classification", "token_classification", "question_answering"):
        m = build_head_model(cfg, task).to("cuda", torch.bfloat16)
        out = m(input_ids=ids)
        first = out.logits if out.logits is not None else out.start_logits
        assert torch.isfinite(first.float()).all(), task
    # a packed row of three samples equals the three samples run on their own (per-sample mixers, shared MLPs)
    model = build_model(_cfg("*-GDN-M2")).to("cuda", torch.bfloat16).eval()
    parts = [torch.randint(0, 512, (1, n), device="cuda") for n in (130, 200, 150)]
    row = torch.cat(parts, 1)
    pos = torch.cat([torch.arange(p.shape[1], device="cuda") for p in parts])[None]
    with torch.no_grad():
        packed = model(input_ids=row, position_ids=pos, cu_seqlens=[0, 130, 330, 480]).logits.float()
        alone = torch.cat([model(input_ids=p).logits.float() for p in parts], 1)
    assert (packed - alone).norm() / alone.norm() < 3e-2
    _status_ok()
