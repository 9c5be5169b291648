"""Serving engine: continuous batching over the native scheduler reproduces plain greedy generation."""
import pytest
import torch

from hybrid_model_factory_b200.models.configuration import HybridConfig
from hybrid_model_factory_b200.models.modeling_hybrid import build_model
from hybrid_model_factory_b200.serving.engine import SamplingParams, ServingEngine
from hybrid_model_factory_b200.serving.scheduler import NativeScheduler


def tiny(pattern, **kw):
    n = len(pattern.split("-"))
    base = dict(vocab_size=128, hidden_size=64, intermediate_size=128, num_hidden_layers=n, num_attention_heads=4,
                num_key_value_heads=2, head_dim=16, hybrid_override_pattern=pattern, swa_config={"window_size": 8})
    base.update(kw)
    return HybridConfig("hybrid_qwen3", **base)


def test_scheduler_chunked_prefill_and_decode_first():
    s = NativeScheduler(num_blocks=64, block_size=4, num_slots=4, max_num_seqs=4, max_num_batched_tokens=10)
    s.add_request(0, list(range(17)), 3)
    b = s.step()
    assert [(x.req_id, x.num_tokens, x.start_pos) for x in b] == [(0, 8, 0)]   # chunk aligned to the block size
    s.advance(0, 8)
    s.add_request(1, list(range(5)), 2)
    b = s.step()
    # the running prefill takes 9 of the 10-token budget (to the end of its prompt); request 1 cannot get a
    # block-aligned chunk out of the single token left and stays queued
    assert [(x.req_id, x.num_tokens, x.start_pos) for x in b] == [(0, 9, 8)]
    s.advance(0, 9)
    s.append_token(0, 99)
    b = s.step()
    # decode of request 0 comes first, then the new prefill
    assert [(x.req_id, x.num_tokens, x.start_pos) for x in b] == [(0, 1, 17), (1, 5, 0)]
    assert b[0].is_decode and not b[1].is_decode
    s.advance(0, 1); s.advance(1, 5)
    s.append_token(0, 98); s.append_token(1, 97)
    b = s.step()
    assert all(x.num_tokens == 1 and x.is_decode for x in b) and len(b) == 2   # both decoding now
    assert len(s.block_table(0)) == 5
    s.finish(0); s.finish(1)
    assert s.stats()["free_slots"] == 4


def test_prefix_cache_hit_reuses_blocks():
    s = NativeScheduler(num_blocks=32, block_size=4, num_slots=4, max_num_seqs=4, max_num_batched_tokens=64,
                        enable_prefix_caching=True)
    prompt = list(range(13))
    s.add_request(0, prompt, 1)
    b = s.step()
    s.advance(0, b[0].num_tokens)
    first_blocks = s.block_table(0)
    s.finish(0)
    s.add_request(1, prompt[:12] + [77], 1)
    b = s.step()
    assert b[0].start_pos == 12 and b[0].num_tokens == 1
    assert s.block_table(1)[:3] == first_blocks[:3]
    assert s.stats()["prefix_hits"] == 1


@pytest.mark.parametrize("pattern", ["*-GDN", "M2-*", "GKA-SWA"])
def test_engine_matches_generate(pattern):
    torch.manual_seed(0)
    model = build_model(tiny(pattern)).eval()
    prompts = [torch.randint(0, 128, (n,)).tolist() for n in (5, 19, 11)]
    ref = [model.generate(torch.tensor([p]), max_new_tokens=6)[0, len(p):].tolist() for p in prompts]
    eng = ServingEngine(model, block_size=4, num_blocks=64, max_num_seqs=4, max_num_batched_tokens=8, max_model_len=64)
    out = eng.generate(prompts, SamplingParams(max_new_tokens=6))
    assert out == ref
    m = eng.request_metrics()
    assert m["finished"] == 3 and m["output_tokens"] == 18 and m["free_slots"] == 4


def test_engine_prefix_caching_with_state_snapshots():
    torch.manual_seed(0)
    model = build_model(tiny("*-GDN")).eval()
    shared = torch.randint(0, 128, (16,)).tolist()
    p1, p2 = shared + [1, 2, 3], shared + [4, 5]
    ref2 = model.generate(torch.tensor([p2]), max_new_tokens=4)[0, len(p2):].tolist()
    eng = ServingEngine(model, block_size=4, num_blocks=64, max_num_seqs=2, max_num_batched_tokens=8, max_model_len=64,
                        enable_prefix_caching=True)
    eng.generate([p1], SamplingParams(max_new_tokens=2))
    out2 = eng.generate([p2], SamplingParams(max_new_tokens=4))[0]
    assert out2 == ref2
    assert eng.sched.stats()["prefix_hits"] >= 1
