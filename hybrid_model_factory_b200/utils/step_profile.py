"""Kernel-level breakdown of one training step (forward, backward, optimizer) of a hybrid model on one GPU.

    python -m hybrid_model_factory_b200.utils.step_profile --seq 65536 --layers 36 --pattern "*-GDN"

Runs one untimed warm-up step and one step under ``torch.profiler`` and prints the CUDA time per kernel, grouped
into classes (attention, GEMM, GDN, elementwise / norms, optimizer, copies).  The shares are what the table is for;
step times are taken with CUDA events by ``bench.py``, never under the profiler.
"""
from __future__ import annotations

import argparse
from collections import defaultdict

import torch

CLASSES = (("attention backward", ("attn_bwd", "delta_kernel")), ("attention forward", ("attn_fwd",)),
           ("GDN kernels", ("gdn_", "gla_segment")), ("GKA kernels", ("gka_",)),
           ("GEMM (cuBLAS / own)", ("nvjet", "gemm", "cutlass", "sgemm", "xmma", "cublas")),
           ("optimizer / grad norm", ("adamw", "sumsq")), ("cross entropy", ("ce_", "linear_ce", "softmax")),
           ("norms / rope / swiglu / conv", ("rms_norm", "gated_norm", "rope", "swiglu", "conv1d", "heads_norm")),
           ("copies / casts / elementwise (PyTorch)", ("elementwise", "copy", "Memcpy", "Memset", "cat", "fill", "reduce")))


def classify(name: str) -> str:
    for label, keys in CLASSES:
        if any(k in name for k in keys):
            return label
    return "other"


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="step_profile")
    ap.add_argument("--seq", type=int, default=65536)
    ap.add_argument("--layers", type=int, default=36)
    ap.add_argument("--pattern", default="*-GDN")
    ap.add_argument("--top", type=int, default=18)
    args = ap.parse_args(argv)
    from ..models.configuration import qwen3_8b_config
    from ..models.modeling_hybrid import build_model
    from ..train.trainer import Trainer, TrainingArguments
    dev = torch.device("cuda", 0)
    cfg = qwen3_8b_config(args.pattern, num_hidden_layers=args.layers, max_position_embeddings=args.seq)
    torch.set_default_dtype(torch.bfloat16)
    with torch.device(dev):
        model = build_model(cfg)
    torch.set_default_dtype(torch.float32)
    model = model.to(torch.bfloat16)
    tr = Trainer(model, TrainingArguments(output_dir="", max_steps=10 ** 6, logging_steps=0, lr_scheduler_type="constant"),
                 device=dev)
    ids = torch.randint(0, cfg.vocab_size, (1, args.seq))
    batch = {"input_ids": ids.pin_memory(), "labels": ids.pin_memory()}
    tr.train_step(batch)
    torch.cuda.synchronize()
    from torch.profiler import ProfilerActivity, profile
    with profile(activities=[ProfilerActivity.CUDA]) as prof:
        tr.train_step(batch)
        torch.cuda.synchronize()
    rows = [(e.key, e.device_time_total / 1e3, e.count) for e in prof.key_averages() if e.device_time_total > 0]
    total = sum(r[1] for r in rows)
    groups = defaultdict(float)
    for name, ms, _ in rows:
        groups[classify(name)] += ms
    print(f"one training step, {args.layers} layers '{args.pattern}', {args.seq} tokens: {total:.0f} ms of CUDA kernel time")
    for label, ms in sorted(groups.items(), key=lambda kv: -kv[1]):
        print(f"  {ms:9.1f} ms {100 * ms / total:5.1f}%  {label}")
    print("top kernels:")
    for name, ms, n in sorted(rows, key=lambda r: -r[1])[:args.top]:
        print(f"  {ms:9.1f} ms {100 * ms / total:5.1f}% x{n:<5d} {name[:100]}")
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
