"""Serving benchmark (the ``vllm bench serve`` workload of the reference, offline): N concurrent requests,
random prompts with lengths uniform in a range, fixed number of greedy output tokens; reports output
tokens/s and time-to-first-token percentiles.

    hmf bench-serve --pattern "*-M2" --num-requests 64 --prompt-min 4096 --prompt-max 16384 --output-len 512
"""
from __future__ import annotations

import argparse
import json
import random
import time

import torch

from ..models.configuration import qwen3_8b_config
from ..models.modeling_hybrid import build_model
from ..utils import checkpoint_io
from .engine import SamplingParams, ServingEngine


def run(model, num_requests=64, prompt_min=4096, prompt_max=16384, output_len=512, seed=0, max_num_batched_tokens=16384,
        max_num_seqs=64, block_size=64, tp=None) -> dict:
    rng = random.Random(seed)
    vocab = model.config.vocab_size
    prompts = [[rng.randrange(vocab) for _ in range(rng.randint(prompt_min, prompt_max))] for _ in range(num_requests)]
    engine = ServingEngine(model, block_size=block_size, max_num_seqs=max_num_seqs,
                           max_num_batched_tokens=max_num_batched_tokens, max_model_len=prompt_max + output_len + 64,
                           tp=tp)
    params = SamplingParams(max_new_tokens=output_len, temperature=0.0)
    # untimed warm-up: graph capture for every decode bucket and one short request through prefill + decode
    engine.warmup(prompt_max + output_len)
    engine.generate([prompts[0][:prompt_min]], SamplingParams(max_new_tokens=4))
    engine.requests.clear()
    for k in engine.stats:
        engine.stats[k] = type(engine.stats[k])()
    if torch.cuda.is_available():
        torch.cuda.synchronize()
    t0 = time.perf_counter()
    for p in prompts:
        engine.add_request(p, params)
    while engine.has_unfinished():
        engine.step()
    if torch.cuda.is_available():
        torch.cuda.synchronize()
    dt = time.perf_counter() - t0
    m = engine.request_metrics()
    ttft = sorted((r.first_token_time - r.arrival) * 1e3 for r in engine.requests.values())
    first_done = max(r.first_token_time for r in engine.requests.values()) - t0
    decode_tokens = m["output_tokens"] - num_requests
    return {"num_requests": num_requests, "prompt_tokens": sum(map(len, prompts)), "output_tokens": m["output_tokens"],
            "wall_s": dt, "output_tok_per_s": m["output_tokens"] / dt,
            "decode_tok_per_s_after_prefill": decode_tokens / max(dt - first_done, 1e-9),
            "p50_ttft_ms": ttft[len(ttft) // 2], "mean_ttft_ms": sum(ttft) / len(ttft), "p99_ttft_ms": ttft[-1],
            "engine_steps": m["steps"], "decode_ms_per_step": 1e3 * m["decode_s"] / max(m["decode_steps"], 1),
            "decode_gpu_ms_per_step": 1e3 * m["decode_gpu_s"] / max(m["graph_replays"], 1),
            "prefill_tok_per_s": m["prefill_tokens"] / max(m["prefill_s"], 1e-9), "graphs": len(engine._graphs),
            "max_num_batched_tokens": max_num_batched_tokens}


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="hmf bench-serve")
    ap.add_argument("model", nargs="?", default=None, help="checkpoint directory (default: random-init Qwen3-8B hybrid)")
    ap.add_argument("--pattern", default="*-M2")
    ap.add_argument("--layers", type=int, default=36)
    ap.add_argument("--num-requests", type=int, default=64)
    ap.add_argument("--prompt-min", type=int, default=4096)
    ap.add_argument("--prompt-max", type=int, default=16384)
    ap.add_argument("--output-len", type=int, default=512)
    ap.add_argument("--max-num-batched-tokens", type=int, default=16384)
    args = ap.parse_args(argv)
    import os
    import torch.distributed as dist
    world, rank = int(os.environ.get("WORLD_SIZE", "1")), int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    dev = torch.device("cuda", local) if torch.cuda.is_available() else torch.device("cpu")
    tp = None
    if world > 1:       # tensor parallel over all ranks (launch with torchrun)
        from ..parallel.tp import TPContext, shard_model
        torch.cuda.set_device(dev)
        dist.init_process_group("nccl", device_id=dev)
        tp = TPContext(dist.group.WORLD)
        if os.environ.get("HMF_TP_FUSED", "1") == "1":
            tp.enable_fused_gemm(max_m=256, max_n=8192)
    if args.model:
        model = checkpoint_io.from_pretrained(args.model, device=dev, init="meta")
    else:
        cfg = qwen3_8b_config(args.pattern, num_hidden_layers=args.layers)
        torch.set_default_dtype(torch.bfloat16)
        with torch.device(dev):
            model = build_model(cfg)
        torch.set_default_dtype(torch.float32)
        model = model.to(torch.bfloat16)
    if tp is not None:
        shard_model(model, tp)
        torch.cuda.empty_cache()
    res = run(model, args.num_requests, args.prompt_min, args.prompt_max, args.output_len,
              max_num_batched_tokens=args.max_num_batched_tokens, tp=tp)
    res["tp"] = world
    if tp is not None:
        res["fused_gemm_allreduce_calls"] = tp.fused_gemm.calls if tp.fused_gemm is not None else 0
        dist.barrier()
    if rank == 0:
        print(json.dumps(res))
    if tp is not None:
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
