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


def test_scheduler_whole_prompt_policy():
    """A prompt that fits a step of its own is not split to fill the rest of the current step; one that exceeds the
    step budget still is."""
    s = NativeScheduler(num_blocks=64, block_size=4, num_slots=4, max_num_seqs=4, max_num_batched_tokens=16,
                        whole_prompts=True)
    s.add_request(0, list(range(10)), 1)
    s.add_request(1, list(range(12)), 1)
    s.add_request(2, list(range(24)), 1)
    b = s.step()
    assert [(x.req_id, x.num_tokens) for x in b] == [(0, 10)]          # request 1 (12 tokens) waits for its own step
    s.advance(0, 10)
    s.append_token(0, 7)
    b = s.step()
    # request 0 is done (one new token); request 1 runs whole; request 2 exceeds any step and takes what is left
    assert [(x.req_id, x.num_tokens) for x in b] == [(1, 12), (2, 4)]
    split = NativeScheduler(num_blocks=64, block_size=4, num_slots=4, max_num_seqs=4, max_num_batched_tokens=16)
    split.add_request(0, list(range(10)), 1)
    split.add_request(1, list(range(12)), 1)
    assert [(x.req_id, x.num_tokens) for x in split.step()] == [(0, 10), (1, 4)]


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


@pytest.mark.parametrize("pattern", ["*-GDN", "M2-*", "GKA-SWA", "BMF-*"])
def test_engine_matches_generate(pattern):
    torch.manual_seed(0)
    model = build_model(tiny(pattern, bmojo_config={"window_size": 4, "ssm_mixer": "gdn", "tie_attn_weights": False})).eval()
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


# ---------------------------------------------------------------------------------------------
# GPU: decode kernels against fp32 PyTorch references, and the engine in bf16 with head_dim 128
# ---------------------------------------------------------------------------------------------
def _kernels():
    import ctypes
    from hybrid_model_factory_b200.ops import _lib
    return _lib, _lib.kernels(), ctypes


@pytest.mark.gpu
@pytest.mark.parametrize("window", [0, 300])
def test_paged_attention_decode_kernel(window):
    _lib, K, ct = _kernels()
    torch.manual_seed(0)
    dev = "cuda"
    Rn, H, Hkv, D, bs = 5, 32, 8, 128, 64
    lens = torch.tensor([1, 63, 700, 5000, 129], dtype=torch.int32, device=dev)
    mb = int((lens.max() + bs - 1) // bs)
    nb = Rn * mb + 3
    kc = torch.randn(nb, bs, Hkv, D, device=dev, dtype=torch.bfloat16)
    vc = torch.randn(nb, bs, Hkv, D, device=dev, dtype=torch.bfloat16)
    perm = torch.randperm(nb, device=dev)[:Rn * mb].to(torch.int32).view(Rn, mb).contiguous()
    q = torch.randn(Rn, H, D, device=dev, dtype=torch.bfloat16)
    for splits, tc in ((1, False), (4, False), (1, True), (4, True), (8, True)):
        o = torch.empty(Rn, H, D, device=dev, dtype=torch.bfloat16)
        po = torch.empty(Rn, H, splits, D, device=dev, dtype=torch.float32)
        pml = torch.empty(Rn, H, splits, 2, device=dev, dtype=torch.float32)
        if tc:
            _lib.check(K.hmf_paged_attention_decode_tc(
                _lib.ptr(q), _lib.ptr(kc), _lib.ptr(vc), _lib.ptr(perm), _lib.ptr(lens), _lib.ptr(o), _lib.ptr(po),
                _lib.ptr(pml), ct.c_int(Rn), ct.c_int(H), ct.c_int(Hkv), ct.c_int(D), ct.c_int(bs), ct.c_int(nb),
                ct.c_int(mb), ct.c_int(splits), ct.c_int(window), ct.c_float(D ** -0.5), _lib.stream_ptr(q.device)), "pa")
            _lib.assert_status_ok()
        else:
            _lib.check(K.hmf_paged_attention_decode(
                _lib.ptr(q), _lib.ptr(kc), _lib.ptr(vc), _lib.ptr(perm), _lib.ptr(lens), _lib.ptr(o), _lib.ptr(po),
                _lib.ptr(pml), ct.c_int(Rn), ct.c_int(H), ct.c_int(Hkv), ct.c_int(D), ct.c_int(bs), ct.c_int(mb),
                ct.c_int(splits), ct.c_int(window), ct.c_float(D ** -0.5), _lib.stream_ptr(q.device)), "pa")
        for r in range(Rn):
            L = int(lens[r])
            p = torch.arange(L, device=dev)
            flat = perm[r].long()[p // bs] * bs + p % bs
            kk = kc.view(-1, Hkv, D)[flat].float()
            vv = vc.view(-1, Hkv, D)[flat].float()
            if window:
                kk, vv = kk[max(0, L - window):], vv[max(0, L - window):]
            kk = kk.repeat_interleave(H // Hkv, dim=1)
            vv = vv.repeat_interleave(H // Hkv, dim=1)
            s = torch.einsum("hd,lhd->hl", q[r].float(), kk) * D ** -0.5
            ref = torch.einsum("hl,lhd->hd", torch.softmax(s, -1), vv)
            assert (o[r].float() - ref).abs().max() < 2e-2, (splits, tc, r)


@pytest.mark.gpu
def test_gdn_and_ssd_decode_kernels():
    from hybrid_model_factory_b200.ops import reference as R
    _lib, K, ct = _kernels()
    torch.manual_seed(0)
    dev = "cuda"
    Rn, H, Hk, D = 6, 8, 4, 128
    q = torch.randn(Rn, H * D, device=dev, dtype=torch.bfloat16)
    k = torch.randn(Rn, Hk * D, device=dev, dtype=torch.bfloat16)
    v = torch.randn(Rn, Hk * D, device=dev, dtype=torch.bfloat16)
    g = -torch.rand(Rn, H, device=dev)
    beta = torch.rand(Rn, H, device=dev)
    slots = torch.tensor([7, 2, 5, 0, 3, 9], dtype=torch.int32, device=dev)
    st = torch.randn(10, H, D, D, device=dev) * 0.1
    st0 = st.clone()
    o = torch.empty(Rn, H, D, device=dev, dtype=torch.bfloat16)
    _lib.check(K.hmf_gdn_decode(_lib.ptr(q), _lib.ptr(k), _lib.ptr(v), _lib.ptr(g), _lib.ptr(beta), _lib.ptr(st),
                                _lib.ptr(slots), _lib.ptr(o), ct.c_int(Rn), ct.c_int(H), ct.c_int(H), ct.c_int(Hk),
                                ct.c_int(Hk), ct.c_int(D), ct.c_int(D), ct.c_float(D ** -0.5), ct.c_int(1),
                                _lib.stream_ptr(q.device)), "gdn_decode")
    rep = H // Hk
    qh = q.view(Rn, 1, H, D)
    kh = k.view(Rn, 1, Hk, D).repeat_interleave(rep, dim=2)
    vh = v.view(Rn, 1, Hk, D).repeat_interleave(rep, dim=2)
    ro, rs = R.gated_delta_rule_recurrent(qh, kh, vh, g[:, None], beta[:, None], initial_state=st0[slots.long()])
    assert (o.float() - ro[:, 0].float()).abs().max() < 2e-2
    assert (st[slots.long()] - rs).abs().max() < 2e-3
    untouched = [i for i in range(10) if i not in slots.tolist()]
    assert torch.equal(st[untouched], st0[untouched])

    # Mamba2 state update: x [R,Hx*P] B [R,Hx*N] C [R,H*N]
    Hh, Hx, P, N = 8, 2, 64, 128
    x = torch.randn(Rn, Hx * P, device=dev, dtype=torch.bfloat16)
    Bm = torch.randn(Rn, Hx * N, device=dev, dtype=torch.bfloat16)
    Cm = torch.randn(Rn, Hh * N, device=dev, dtype=torch.bfloat16)
    dt = torch.rand(Rn, Hh, device=dev)
    A = -torch.rand(Hh, device=dev)
    Dp = torch.randn(Hh, device=dev)
    st = torch.randn(10, Hh, P, N, device=dev) * 0.1
    st0 = st.clone()
    y = torch.empty(Rn, Hh, P, device=dev, dtype=torch.bfloat16)
    _lib.check(K.hmf_ssd_decode(_lib.ptr(x), _lib.ptr(dt), _lib.ptr(A), _lib.ptr(Bm), _lib.ptr(Cm), _lib.ptr(Dp),
                                _lib.ptr(st), _lib.ptr(slots), _lib.ptr(y), ct.c_int(Rn), ct.c_int(Hh), ct.c_int(Hx),
                                ct.c_int(Hx), ct.c_int(P), ct.c_int(N), _lib.stream_ptr(x.device)), "ssd_decode")
    rep = Hh // Hx
    xh = x.view(Rn, Hx, P).repeat_interleave(rep, dim=1)
    Bh = Bm.view(Rn, Hx, N).repeat_interleave(rep, dim=1)
    ry, rs = R.selective_state_update(st0[slots.long()], xh, dt, A, Bh, Cm.view(Rn, Hh, N), Dp)
    assert ((y.float() - ry.float()).abs() / (ry.float().abs() + 1.0)).max() < 1e-2
    assert (st[slots.long()] - rs).abs().max() < 2e-3


@pytest.mark.gpu
@pytest.mark.parametrize("pattern", ["*-GDN", "M2-*", "GKA-*"])
def test_engine_bf16_kernels_match_torch_path(pattern):
    """The kernel decode path and the PyTorch decode path of the engine agree on (almost) all greedy tokens."""
    torch.manual_seed(0)
    cfg = tiny(pattern, hidden_size=512, intermediate_size=1024, num_attention_heads=4, num_key_value_heads=2,
               head_dim=128, vocab_size=512)
    model = build_model(cfg).to("cuda", torch.bfloat16).eval()
    prompts = [torch.randint(0, 512, (n,)).tolist() for n in (70, 200, 33, 129)]
    outs = []
    for use_kernels in (True, False):
        eng = ServingEngine(model, block_size=64, num_blocks=64, max_num_seqs=4, max_num_batched_tokens=128,
                            max_model_len=512, use_cuda_graphs=use_kernels)
        assert eng._cuda
        eng._cuda = use_kernels
        outs.append(eng.generate(prompts, SamplingParams(max_new_tokens=12)))
        assert (eng.stats["graph_replays"] > 0) == use_kernels
    agree = sum(a == b for x, y in zip(*outs) for a, b in zip(x, y))
    first = sum(x[0] == y[0] for x, y in zip(*outs))
    assert first == len(prompts) and agree >= 0.75 * 12 * len(prompts), (agree, outs)


@pytest.mark.gpu
def test_moe_engine_decodes_from_cuda_graphs():
    """A bf16 MoE model: the expert path has static shapes on the device, so the decode step is captured and replayed;
    the tokens agree with the eager engine."""
    torch.manual_seed(0)
    base = tiny("*-GDN", hidden_size=512, intermediate_size=1024, num_attention_heads=4, num_key_value_heads=2,
                head_dim=128, vocab_size=512, num_experts=8, num_experts_per_tok=2, moe_intermediate_size=256)
    cfg = HybridConfig("hybrid_qwen3_moe", **{k: v for k, v in base.to_dict().items() if k != "model_type"})
    model = build_model(cfg).to("cuda", torch.bfloat16).eval()
    prompts = [torch.randint(0, 512, (n,)).tolist() for n in (70, 33, 129)]
    outs = []
    for graphs in (True, False):
        eng = ServingEngine(model, block_size=64, num_blocks=64, max_num_seqs=4, max_num_batched_tokens=128,
                            max_model_len=512, use_cuda_graphs=graphs)
        outs.append(eng.generate(prompts, SamplingParams(max_new_tokens=10)))
        assert (eng.stats["graph_replays"] > 0) == graphs
    agree = sum(a == b for x, y in zip(*outs) for a, b in zip(x, y))
    assert agree >= 0.8 * 10 * len(prompts), (agree, outs)


def _tp_worker(rank, world, pattern):
    import torch.distributed as dist
    from hybrid_model_factory_b200.parallel.tp import TPContext, shard_model
    torch.manual_seed(0)
    kw = dict(num_experts=4, num_experts_per_tok=2, moe_intermediate_size=32) if pattern == "moe" else {}
    cfg = tiny("*-GDN-M2-GKA" if pattern != "moe" else "*-GDN", **kw)
    if pattern == "moe":
        d = {k: v for k, v in cfg.to_dict().items() if k != "model_type"}
        cfg = HybridConfig("hybrid_qwen3_moe", **d)
    model = build_model(cfg).eval()
    prompts = [torch.randint(0, 128, (n,)).tolist() for n in (5, 19, 11)]
    ref = [model.generate(torch.tensor([p]), max_new_tokens=5)[0, len(p):].tolist() for p in prompts]
    tp = TPContext(dist.group.WORLD)
    shard_model(model, tp)
    eng = ServingEngine(model, block_size=4, num_blocks=64, max_num_seqs=4, max_num_batched_tokens=8, max_model_len=64,
                        tp=tp)
    out = eng.generate(prompts, SamplingParams(max_new_tokens=5))
    assert out == ref, (rank, out, ref)


@pytest.mark.parametrize("pattern", ["dense", "moe"])
def test_tensor_parallel_engine_gloo(pattern):
    from dist_utils import run_ranks
    run_ranks(_tp_worker, 2, pattern)


@pytest.mark.gpu
@pytest.mark.parametrize("M,N,K", [(1, 256, 64), (7, 4096, 512), (64, 4096, 1536), (200, 1024, 192)])
def test_gemm_allreduce_single_rank(M, N, K):
    """World size 1: the fused kernel is a skinny GEMM that reduces over its own partial (twice, to cover both
    parity buffers and the device-side epoch)."""
    from hybrid_model_factory_b200.ops.fused_comm import PeerGemmAllReduce
    from hybrid_model_factory_b200.ops import _lib
    torch.manual_seed(0)
    op = PeerGemmAllReduce(None, max_m=256, max_n=4096)
    for it in range(3):
        x = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
        w = torch.randn(N, K, device="cuda", dtype=torch.bfloat16) * 0.05
        assert op.accepts(x, w)
        y = op(x, w)
        ref = x.float() @ w.float().t()
        assert (y.float() - ref).abs().max() < 2e-2 * ref.abs().max() + 1e-2
    torch.cuda.synchronize()
    _lib.assert_status_ok()
    assert int(op.sync[0]) == 3


@pytest.mark.gpu
def test_moe_grouped_gemm_single_rank():
    """Grouped expert GEMMs with device-built tile tables against the per-expert reference (one rank: the
    send / receive buffers are local, the dispatch and combine paths still run through flags)."""
    from hybrid_model_factory_b200.ops import _lib
    from hybrid_model_factory_b200.ops import reference as R
    from hybrid_model_factory_b200.parallel.ep_fused import FusedExpertParallel
    torch.manual_seed(0)
    E, Dm, Fi, T, k = 8, 512, 256, 700, 2
    x = (torch.randn(T, Dm, device="cuda") * 0.5).bfloat16()
    wgu = (torch.randn(E, 2 * Fi, Dm, device="cuda") * 0.05).bfloat16()
    wd = (torch.randn(E, Dm, Fi, device="cuda") * 0.05).bfloat16()
    logits = torch.randn(T, E, device="cuda")
    logits[:, 3] = -1e9                                     # an expert without tokens
    w, idx = R.moe_router(logits, k)
    ep = FusedExpertParallel(None, E, Dm, Fi, max_send_rows=T * k, capacity_rows=T * k)
    for _ in range(3):
        out = ep.forward(x, w, idx, wgu, wd)
    torch.cuda.synchronize()
    _lib.assert_status_ok()
    ref = R.moe_experts(x.float(), wgu.float(), wd.float(), w, idx)
    assert int(ep.counts[1]) == T * k and int(ep.counts[2]) == 0
    err = (out.float() - ref).abs().max() / ref.abs().max()
    assert err < 3e-2, err


@pytest.mark.gpu
def test_moe_model_uses_grouped_gemm_kernels():
    from hybrid_model_factory_b200.parallel.ep_fused import attach_fused_moe
    torch.manual_seed(0)
    cfg = HybridConfig("hybrid_qwen3_moe", vocab_size=256, hidden_size=256, intermediate_size=512, num_hidden_layers=2,
                       num_attention_heads=2, num_key_value_heads=2, head_dim=128, num_experts=8, num_experts_per_tok=2,
                       moe_intermediate_size=128, hybrid_override_pattern="*-GDN")
    model = build_model(cfg).to("cuda", torch.bfloat16).eval()
    ids = torch.randint(0, 256, (2, 96), device="cuda")
    with torch.no_grad():
        ref = model(ids).logits.float()
        assert attach_fused_moe(model) == 2
        out = model(ids).logits.float()
    assert model.model.layers[0].mlp.fused_ep.calls > 0
    assert (out - ref).abs().max() < 0.05 * ref.abs().max()


def test_openai_compatible_server_routes():
    """The completion, chat, streaming and metrics routes of the API server, called in-process (no HTTP client in the
    test environment): the generated tokens equal the model's own greedy generation."""
    import asyncio
    import json
    from hybrid_model_factory_b200.data.formats import ByteTokenizer
    from hybrid_model_factory_b200.serving.api_server import create_app
    torch.manual_seed(0)
    cfg = tiny("*-GDN", vocab_size=259)
    model = build_model(cfg).eval()
    eng = ServingEngine(model, block_size=4, num_blocks=128, max_num_seqs=4, max_num_batched_tokens=32, max_model_len=128)
    tok = ByteTokenizer()
    app = create_app(eng, tok, model_name="tiny", template="qwen3")
    routes = {r.path: r.endpoint for r in app.routes if hasattr(r, "endpoint")}

    async def scenario():
        models = await routes["/v1/models"]()
        assert models["data"][0]["id"] == "tiny"
        prompt = "hello"
        resp = await routes["/v1/completions"]({"prompt": prompt, "max_tokens": 5, "ignore_eos": True})
        body = json.loads(resp.body)
        ids = tok.encode(prompt, add_special_tokens=False)
        want = model.generate(torch.tensor([ids]), max_new_tokens=5)[0, len(ids):].tolist()
        assert body["usage"] == {"prompt_tokens": len(ids), "completion_tokens": 5, "total_tokens": len(ids) + 5}
        assert body["choices"][0]["text"] == tok.decode(want)
        chat = await routes["/v1/chat/completions"]({"messages": [{"role": "system", "content": "be brief"},
                                                                  {"role": "user", "content": "hi"}],
                                                     "max_tokens": 3, "ignore_eos": True})
        cbody = json.loads(chat.body)
        assert cbody["object"] == "chat.completion" and cbody["choices"][0]["message"]["role"] == "assistant"
        stream = await routes["/v1/completions"]({"prompt": prompt, "max_tokens": 3, "stream": True, "ignore_eos": True})
        chunks = [c async for c in stream.body_iterator]
        assert chunks[-1].strip() == "data: [DONE]" and 2 <= len(chunks) <= 4      # partial characters are held back
        assert "".join(json.loads(c[6:])["choices"][0]["text"] for c in chunks[:-1]) == tok.decode(want[:3])
        m = await routes["/metrics"]()
        assert m["output_tokens"] >= 11
        # stop strings: the text ends before the first one, the request is dropped early, the reason says so
        long = json.loads((await routes["/v1/completions"]({"prompt": prompt, "max_tokens": 12, "ignore_eos": True})).body)
        text = long["choices"][0]["text"]
        assert long["choices"][0]["finish_reason"] == "length" and len(text) >= 6
        stop = text[3:5]
        cut = json.loads((await routes["/v1/completions"]({"prompt": prompt, "max_tokens": 12, "ignore_eos": True,
                                                           "stop": stop})).body)
        assert cut["choices"][0]["text"] == text[:text.find(stop)] and cut["choices"][0]["finish_reason"] == "stop"
        assert cut["usage"]["completion_tokens"] < 12
        for _ in range(50):                                        # the serving thread retires it before its next step
            if not eng.has_unfinished():
                break
            await asyncio.sleep(0.02)
        assert not eng.has_unfinished()
        assert [r.finish_reason for r in eng.requests.values()][-1] == "abort"
        # a streamed answer never shows text that turns out to be (the start of) a stop string
        stream = await routes["/v1/completions"]({"prompt": prompt, "max_tokens": 12, "stream": True, "ignore_eos": True,
                                                  "stop": [stop]})
        chunks = [json.loads(c[6:]) for c in [c async for c in stream.body_iterator][:-1]]
        assert "".join(c["choices"][0]["text"] for c in chunks) == text[:text.find(stop)]
        assert chunks[-1]["choices"][0]["finish_reason"] == "stop"
        # a client that stops reading: closing the stream drops the request inside the engine
        stream = await routes["/v1/completions"]({"prompt": prompt, "max_tokens": 40, "stream": True, "ignore_eos": True})
        it = stream.body_iterator
        await it.__anext__()
        await it.aclose()
        for _ in range(100):
            if not eng.has_unfinished():
                break
            await asyncio.sleep(0.02)
        last = list(eng.requests.values())[-1]
        assert last.finish_reason == "abort" and len(last.output) < 40
        # stop tokens end a request inside the engine; n > 1 returns that many choices
        third = tok.encode(text, add_special_tokens=False)[2]
        st = json.loads((await routes["/v1/completions"]({"prompt": prompt, "max_tokens": 12, "ignore_eos": True,
                                                          "stop_token_ids": [third]})).body)
        assert st["choices"][0]["finish_reason"] == "stop" and st["usage"]["completion_tokens"] <= 3
        many = json.loads((await routes["/v1/completions"]({"prompt": prompt, "max_tokens": 4, "n": 3,
                                                            "ignore_eos": True})).body)
        assert [c["index"] for c in many["choices"]] == [0, 1, 2] and many["usage"]["completion_tokens"] == 12
        assert len({c["text"] for c in many["choices"]}) == 1                      # greedy: identical
        # log-probabilities: the greedy token is the likeliest one, values are those of the model's own distribution
        lp = json.loads((await routes["/v1/completions"]({"prompt": prompt, "max_tokens": 4, "ignore_eos": True,
                                                          "logprobs": 3})).body)["choices"][0]["logprobs"]
        assert len(lp["tokens"]) == 4 and all(1 <= len(t) <= 3 for t in lp["top_logprobs"])    # (bytes may decode alike)
        assert all(abs(max(t.values()) - v) < 1e-6 for t, v in zip(lp["top_logprobs"], lp["token_logprobs"]))
        with torch.no_grad():
            ref_lp = torch.log_softmax(model(input_ids=torch.tensor([ids])).logits[0, -1].float(), -1).max()
        assert abs(float(ref_lp) - lp["token_logprobs"][0]) < 1e-4
        clp = json.loads((await routes["/v1/chat/completions"]({"messages": [{"role": "user", "content": "hi"}],
                                                                "max_tokens": 2, "ignore_eos": True, "logprobs": True,
                                                                "top_logprobs": 2})).body)["choices"][0]["logprobs"]
        assert len(clp["content"]) == 2 and len(clp["content"][0]["top_logprobs"]) == 2
    try:
        asyncio.run(scenario())
    finally:
        app.state.loop_runner.stop = True          # ends the engine thread


def test_chat_route_formats_tools_and_returns_structured_calls():
    """``tools`` are written into the system prompt in the template's format, earlier tool traffic becomes function /
    observation turns, and an answer holding a call block comes back as ``tool_calls``."""
    import asyncio
    import json
    from hybrid_model_factory_b200.data.formats import ByteTokenizer, get_template
    from hybrid_model_factory_b200.serving import api_server
    tpl = get_template("qwen3")
    text, calls = tpl.extract_tool_calls('Let me look.\n<tool_call>\n{"name": "weather", "arguments": {"city": "Oslo"}}\n'
                                         '</tool_call>\n<tool_call>\n{"name": "time", "arguments": {}}\n</tool_call>')
    assert text == "Let me look." and [c["name"] for c in calls] == ["weather", "time"] and calls[0]["arguments"] == {"city": "Oslo"}
    assert tpl.extract_tool_calls("<tool_call>\nnot json\n</tool_call>") == ("<tool_call>\nnot json\n</tool_call>", [])
    torch.manual_seed(0)
    model = build_model(tiny("*-GDN", vocab_size=259)).eval()
    eng = ServingEngine(model, block_size=8, num_blocks=256, max_num_seqs=2, max_num_batched_tokens=1024, max_model_len=1024)
    tok = ByteTokenizer()
    app = api_server.create_app(eng, tok, model_name="tiny", template="qwen3")
    routes = {r.path: r.endpoint for r in app.routes if hasattr(r, "endpoint")}
    seen = {}
    real_submit = app.state.loop_runner.submit

    def spy(prompt, params, loop):
        seen["prompt"] = tok.decode(prompt)
        return real_submit(prompt, params, loop)
    app.state.loop_runner.submit = spy
    answer = '<tool_call>\n{"name": "weather", "arguments": {"city": "Oslo"}}\n</tool_call>'
    real_decode = tok.decode
    tools = [{"type": "function", "function": {"name": "weather", "parameters": {"type": "object"}}}]
    msgs = [{"role": "user", "content": "weather in Bergen?"},
            {"role": "assistant", "content": None, "tool_calls": [{"id": "c1", "type": "function", "function": {
                "name": "weather", "arguments": "{\"city\": \"Bergen\"}"}}]},
            {"role": "tool", "tool_call_id": "c1", "content": "rain"},
            {"role": "user", "content": "and Oslo?"}]

    async def scenario():
        tok.decode = lambda ids: answer if len(ids) <= 4 else real_decode(ids)     # the "model" answers with a call
        try:
            resp = await routes["/v1/chat/completions"]({"messages": msgs, "tools": tools, "max_tokens": 4,
                                                         "ignore_eos": True})
        finally:
            tok.decode = real_decode
        return json.loads(resp.body)
    try:
        body = asyncio.run(scenario())
    finally:
        app.state.loop_runner.stop = True
    prompt = seen["prompt"]
    assert "# Tools" in prompt and '"name": "weather"' in prompt
    assert '<tool_call>\n{"name": "weather", "arguments": {"city": "Bergen"}}\n</tool_call>' in prompt
    assert "<tool_response>\nrain\n</tool_response>" in prompt and prompt.rstrip().endswith("<|im_start|>assistant")
    choice = body["choices"][0]
    assert choice["finish_reason"] == "tool_calls" and choice["message"]["content"] is None
    call = choice["message"]["tool_calls"][0]
    assert call["function"]["name"] == "weather" and json.loads(call["function"]["arguments"]) == {"city": "Oslo"}


def test_plugin_registry_targets_resolve_to_the_native_models():
    import importlib
    from hybrid_model_factory_b200.serving import vllm_plugin
    reg = vllm_plugin.registry()
    assert set(reg) == set(vllm_plugin.ARCHITECTURES)
    for name, target in vllm_plugin.ARCHITECTURES.items():
        mod, cls = target.split(":")
        assert getattr(importlib.import_module(mod), cls) is reg[name]
    model = reg["HybridQwen3ForCausalLM"](tiny("*-GDN"))
    assert model(torch.randint(0, 128, (1, 8))).logits.shape == (1, 8, 128)


def test_chat_cli_round_trip(tmp_path, monkeypatch, capsys):
    """`hmf chat` on a saved tiny checkpoint: two user turns, `clear`, `exit`."""
    from hybrid_model_factory_b200.serving import chat
    from hybrid_model_factory_b200.utils import checkpoint_io
    torch.manual_seed(0)
    model = build_model(tiny("*-GDN", vocab_size=259))
    checkpoint_io.save_pretrained(model, str(tmp_path / "ckpt"))
    lines = iter(["hello", "clear", "again", "exit"])
    monkeypatch.setattr("builtins.input", lambda _prompt="": next(lines))
    assert chat.main([str(tmp_path / "ckpt"), "--max-new-tokens", "4", "--template", "qwen3"]) == 0
    out = capsys.readouterr().out
    assert out.count("Assistant:") == 2


def _tp_server_worker(rank, world):
    import asyncio
    import json
    import torch.distributed as dist
    from hybrid_model_factory_b200.data.formats import ByteTokenizer
    from hybrid_model_factory_b200.parallel.tp import TPContext, shard_model
    from hybrid_model_factory_b200.serving import api_server as S
    torch.manual_seed(0)
    cfg = tiny("*-GDN-M2", vocab_size=260)
    model = build_model(cfg).eval()
    tok = ByteTokenizer()
    prompts = ["hello there", "tensor parallel"]
    want = []
    for p in prompts:
        ids = tok.encode(p, add_special_tokens=False)
        want.append(model.generate(torch.tensor([ids]), max_new_tokens=6)[0, len(ids):].tolist())
    tp = TPContext(dist.group.WORLD)
    shard_model(model, tp)
    control = S.ControlChannel()
    eng = ServingEngine(model, block_size=4, num_blocks=128, max_num_seqs=4, max_num_batched_tokens=32, max_model_len=128,
                        tp=tp)
    if rank != 0:
        assert S.follow(eng, control) >= 6          # stepped along with rank 0 until it was told to stop
        return
    app = S.create_app(eng, tok, model_name="tiny", control=control)
    routes = {r.path: r.endpoint for r in app.routes if hasattr(r, "endpoint")}

    async def scenario():
        resps = await asyncio.gather(*[routes["/v1/completions"]({"prompt": p, "max_tokens": 6, "ignore_eos": True})
                                       for p in prompts])
        return [json.loads(r.body)["choices"][0]["text"] for r in resps]
    try:
        texts = asyncio.run(scenario())
    finally:
        app.state.loop_runner.stop = True
        app.state.loop_runner.wake.set()
        app.state.loop_runner.thread.join(timeout=10)
    assert texts == [tok.decode(w) for w in want], (texts, want)


def test_tensor_parallel_api_server_gloo():
    """Rank 0 serves the routes, rank 1 follows the broadcast request stream; outputs equal the unsharded model's."""
    from dist_utils import run_ranks
    run_ranks(_tp_server_worker, 2)


def test_api_server_reports_an_engine_failure_instead_of_hanging():
    import asyncio
    import json
    from hybrid_model_factory_b200.data.formats import ByteTokenizer
    from hybrid_model_factory_b200.serving.api_server import create_app
    model = build_model(tiny("*-GDN", vocab_size=259)).eval()
    eng = ServingEngine(model, block_size=4, num_blocks=64, max_num_seqs=2, max_num_batched_tokens=16, max_model_len=64)

    def boom():
        raise RuntimeError("engine exploded")
    eng.step = boom
    app = create_app(eng, ByteTokenizer(), model_name="tiny")
    routes = {r.path: r.endpoint for r in app.routes if hasattr(r, "endpoint")}

    async def scenario():
        r1 = await asyncio.wait_for(routes["/v1/completions"]({"prompt": "hi", "max_tokens": 2}), timeout=20)
        r2 = await asyncio.wait_for(routes["/v1/completions"]({"prompt": "again", "max_tokens": 2}), timeout=20)
        return r1, r2
    r1, r2 = asyncio.run(scenario())
    assert r1.status_code == 500 and "engine exploded" in json.loads(r1.body)["error"]
    assert r2.status_code == 500


def test_state_shapes_match_the_engine_allocations():
    """The published per-request state shapes agree with what `ServingState` allocates for each mixer type, and shrink
    with the tensor-parallel size."""
    from hybrid_model_factory_b200.serving import state_shapes as SS
    from hybrid_model_factory_b200.serving.cache import ServingState
    model = build_model(tiny("*-GDN-M2-GKA")).eval()
    st = ServingState(model, num_blocks=8, block_size=4, num_slots=2, num_snapshots=0, device=torch.device("cpu"),
                      dtype=torch.float32)
    cfg = model.config
    H, Hkv, D = cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim
    by_layer = {i: type(l.seq_mixer).__name__ for i, l in enumerate(model.model.layers)}
    for i, entry in st.ssm.items():
        name = by_layer[i]
        rec = next(v for k, v in entry.items() if k in ("state", "recurrent", "h_kv"))
        assert tuple(rec.shape[1:]) in (SS.gdn_state_shapes(H, H, H, D)["recurrent"][0],
                                        SS.mamba2_state_shapes(H * D, Hkv * D, D)["ssm"][0]), (name, rec.shape)
    kv = SS.attention_kv_shape(Hkv, D, 4)
    k_cache = st.kv[0][0]
    assert tuple(k_cache.shape[-2:]) == kv["k"][0][1:]
    full = SS.bytes_per_request(SS.gka_state_shapes(32, 8, 32, 128))
    half = SS.bytes_per_request(SS.gka_state_shapes(32, 8, 32, 128, tp=2))
    assert full == 2 * half and SS.gka_state_shapes(32, 8, 32, 128, use_v_conv=False)["conv"][0][1] == 40 * 128
    with pytest.raises(AssertionError):
        SS.gdn_state_shapes(32, 8, 32, 128, tp=16)


@pytest.mark.parametrize("device", ["cpu", pytest.param("cuda", marks=pytest.mark.gpu)])
def test_sampler_filters(device):
    """Temperature / top-k / top-p / min-p / repetition penalty: the sampled token always lies in the kept set, greedy
    rows return the arg-max, and the empirical distribution follows the renormalised probabilities (the PyTorch
    procedure on the CPU, the sampling kernel on the GPU)."""
    from hybrid_model_factory_b200.serving.engine import SamplingParams, sample_tokens
    devs = [device]
    g = torch.Generator().manual_seed(0)
    V = 1000
    base = torch.randn(V, generator=g) * 3
    for dev in devs:
        logits = base.repeat(64, 1).to(dev)
        top5 = set(torch.topk(base, 5).indices.tolist())
        toks = sample_tokens(logits, [SamplingParams(temperature=1.0, top_k=5)] * 64, generator=g)
        assert set(toks) <= top5 and len(set(toks)) > 1
        assert sample_tokens(logits[:3], [SamplingParams(temperature=0.0)] * 3) == [int(base.argmax())] * 3
        # nucleus: the smallest prefix of the sorted probabilities that reaches top_p
        pr = torch.softmax(base, 0)
        srt, order = torch.sort(pr, descending=True)
        n_keep = int((torch.cumsum(srt, 0) < 0.6).sum()) + 1
        toks = sample_tokens(logits, [SamplingParams(temperature=1.0, top_p=0.6)] * 64, generator=g)
        assert set(toks) <= set(order[:n_keep + 1].tolist())
        toks = sample_tokens(logits, [SamplingParams(temperature=1.0, min_p=0.5)] * 64, generator=g)
        assert all(pr[t] >= 0.5 * pr.max() - 1e-6 for t in toks)
        # repetition penalty pushes the arg-max away from a token already produced
        best = int(base.argmax())
        boosted = base.clone()
        boosted[best] = boosted.abs().max() + 0.1
        second = int(torch.topk(boosted, 2).indices[1])
        out = sample_tokens(boosted[None].to(dev), [SamplingParams(temperature=0.0, repetition_penalty=50.0)], [[best, best]])
        assert out == [second]
    # distribution check on the widest device available
    dev = devs[-1]
    small = torch.tensor([[2.0, 1.0, 0.0, -1.0]]).repeat(4000, 1).to(dev)
    toks = torch.tensor(sample_tokens(small, [SamplingParams(temperature=1.0)] * 4000, generator=g))
    freq = torch.bincount(toks, minlength=4).float() / 4000
    assert (freq - torch.softmax(small[0].float().cpu(), 0)).abs().max() < 0.03


def test_api_server_scores_texts_with_a_reward_head():
    import asyncio
    import json
    from hybrid_model_factory_b200.data.formats import ByteTokenizer
    from hybrid_model_factory_b200.serving.api_server import create_app
    from hybrid_model_factory_b200.train.preference import attach_value_head
    torch.manual_seed(0)
    model = build_model(tiny("*-GDN", vocab_size=259)).eval()
    eng = ServingEngine(model, block_size=4, num_blocks=64, max_num_seqs=2, max_num_batched_tokens=16, max_model_len=64)
    app = create_app(eng, ByteTokenizer(), model_name="tiny")
    routes = {r.path: r.endpoint for r in app.routes if hasattr(r, "endpoint")}
    try:
        r = asyncio.run(routes["/v1/score/evaluation"]({"messages": ["a"]}))
        assert r.status_code == 400                                     # no value head yet
        attach_value_head(model)
        out = asyncio.run(routes["/v1/score/evaluation"]({"messages": ["good answer", "bad"]}))
        assert len(out["scores"]) == 2 and out["scores"][0] != out["scores"][1]
        # same as scoring the tokens directly
        from hybrid_model_factory_b200.train.preference import reward_scores
        ids = torch.tensor([ByteTokenizer().encode("bad", add_special_tokens=False)])
        assert abs(float(reward_scores(model, ids)[0]) - out["scores"][1]) < 1e-5
    finally:
        app.state.loop_runner.stop = True
        app.state.loop_runner.wake.set()
        app.state.loop_runner.thread.join(timeout=5)


@pytest.mark.parametrize("pattern", ["*-GDN", "M2-GKA", "SWA-*"])
def test_packed_prefill_of_several_requests_matches_one_by_one(pattern):
    """Several requests' prefill pieces share one forward (one row with sample boundaries, one cache per sample); the
    generated tokens equal those of request-by-request prefill, also when pieces continue a chunked prompt."""
    torch.manual_seed(0)
    model = build_model(tiny(pattern, vocab_size=259)).eval()
    g = torch.Generator().manual_seed(3)
    prompts = [torch.randint(0, 259, (n,), generator=g).tolist() for n in (9, 23, 5, 14)]
    outs = []
    for packed in (False, True):
        eng = ServingEngine(model, block_size=4, num_blocks=128, max_num_seqs=4, max_num_batched_tokens=24,
                            max_model_len=64)
        eng.packed_prefill = packed
        outs.append(eng.generate(prompts, SamplingParams(max_new_tokens=5)))
        assert (eng.stats["packed_prefills"] > 0) == packed
    assert outs[0] == outs[1]


def test_engine_raises_on_a_recorded_device_wait_timeout():
    """A tensor-parallel engine reads the kernels' status block; a recorded timeout must end the run loudly."""
    from hybrid_model_factory_b200.ops import _lib
    model = build_model(tiny("*-GDN", vocab_size=259)).eval()
    eng = ServingEngine(model, block_size=4, num_blocks=64, max_num_seqs=2, max_num_batched_tokens=16, max_model_len=64)
    eng.check_kernel_status(lambda: (0, 0, 0, 0))
    with pytest.raises(_lib.KernelError, match="wait ran out"):
        eng.check_kernel_status(lambda: (3, 17, 0x40, 2))


@pytest.mark.parametrize("pattern", ["*-GDN", "M2-GKA-*", "*-*"])
def test_speculative_decoding_is_exact(pattern):
    """Drafts from the request's own n-grams, verified in one forward; rejected drafts roll the recurrent state back.
    The tokens equal plain greedy decoding whatever is accepted."""
    torch.manual_seed(0)
    model = build_model(tiny(pattern, vocab_size=24)).eval()         # a small vocabulary makes repeats (and drafts) common
    g = torch.Generator().manual_seed(5)
    base = torch.randint(0, 24, (6,), generator=g).tolist()
    prompts = [base * 3, torch.randint(0, 24, (17,), generator=g).tolist(), (base[:3] * 5)[:13]]
    outs, stats = [], []
    for k in (0, 4):
        eng = ServingEngine(model, block_size=8, num_blocks=64, max_num_seqs=4, max_num_batched_tokens=64,
                            max_model_len=128)
        outs.append(eng.generate(prompts, SamplingParams(max_new_tokens=24, speculative_tokens=k)))
        stats.append(dict(eng.stats))
    assert outs[0] == outs[1]
    assert stats[0]["spec_steps"] == 0 and stats[1]["spec_steps"] > 0 and stats[1]["spec_drafted"] > 0
    assert all(len(o) == 24 for o in outs[1])
    assert stats[1]["steps"] <= stats[0]["steps"]


@pytest.mark.gpu
def test_speculative_decoding_on_gpu_kernels():
    """bf16 kernels: the verify forward (prefill kernels) and the decode step (decode kernels) round differently, so the
    two runs may part at a near-tie; they must agree on almost all tokens and drafts must get accepted."""
    torch.manual_seed(0)
    cfg = tiny("*-GDN-M2-*", hidden_size=512, intermediate_size=1024, num_attention_heads=4, num_key_value_heads=2,
               head_dim=128, vocab_size=64)
    model = build_model(cfg).to("cuda", torch.bfloat16).eval()
    g = torch.Generator().manual_seed(5)
    base = torch.randint(0, 64, (8,), generator=g).tolist()
    prompts = [base * 6, torch.randint(0, 64, (70,), generator=g).tolist(), (base[:4] * 20)[:75]]
    outs, stats = [], []
    for k in (0, 4):
        eng = ServingEngine(model, block_size=64, num_blocks=32, max_num_seqs=4, max_num_batched_tokens=256,
                            max_model_len=512)
        outs.append(eng.generate(prompts, SamplingParams(max_new_tokens=32, speculative_tokens=k)))
        stats.append(dict(eng.stats))
    from hybrid_model_factory_b200.ops import _lib
    _lib.assert_status_ok()
    agree = sum(a == b for x, y in zip(*outs) for a, b in zip(x, y))
    assert stats[1]["spec_steps"] > 0 and all(len(o) == 32 for o in outs[1])
    assert all(x[0] == y[0] for x, y in zip(*outs)) and agree >= 0.7 * 96, (agree, outs)


def test_speculative_decoding_with_a_draft_model():
    """A draft model proposes tokens where the n-gram index has none.  With the target's own weights as the draft every
    proposal is accepted and the steps shrink; with an unrelated draft most are rejected; the tokens are those of plain
    greedy decoding either way."""
    import copy
    torch.manual_seed(0)
    model = build_model(tiny("*-GDN-M2", vocab_size=64)).eval()
    twin = copy.deepcopy(model)
    torch.manual_seed(1)
    other = build_model(tiny("GDN-*", vocab_size=64, num_hidden_layers=2)).eval()
    g = torch.Generator().manual_seed(5)
    prompts = [torch.randint(0, 64, (n,), generator=g).tolist() for n in (9, 17, 12)]
    runs = {}
    for name, draft, k in (("plain", None, 0), ("twin", twin, 3), ("other", other, 3)):
        eng = ServingEngine(model, block_size=8, num_blocks=64, max_num_seqs=4, max_num_batched_tokens=64,
                            max_model_len=128, draft_model=draft)
        eng.spec_ngram = (64, 63)                                   # no n-gram of that length exists: drafts come from the model
        runs[name] = (eng.generate(prompts, SamplingParams(max_new_tokens=20, speculative_tokens=k)), dict(eng.stats))
    assert runs["twin"][0] == runs["plain"][0] and runs["other"][0] == runs["plain"][0]
    st = runs["twin"][1]
    assert st["spec_model_drafts"] > 0 and st["spec_accepted"] == st["spec_drafted"] > 0
    assert st["steps"] < runs["plain"][1]["steps"]
    assert runs["other"][1]["spec_accepted"] < runs["other"][1]["spec_drafted"]
