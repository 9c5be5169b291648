"""Training statistics: FLOPs per token, MFU, learning-rate suggestion, perplexity, length CDF
(reference: ``training/scripts/stat_utils/*.py``)."""
from __future__ import annotations

import math
from typing import Dict, Iterable, Sequence

import torch


def flops_per_token(cfg, seq_len: int, backward: bool = True) -> float:
    """Matmul FLOPs per token of a hybrid decoder: dense projections + sequence mixing (attention is quadratic,
    linear mixers are ``O(d_state)`` per token) + ``lm_head``.  Backward counts 2x forward."""
    Dm, L = cfg.hidden_size, cfg.num_hidden_layers
    Hq, Hkv = cfg.num_attention_heads, cfg.num_key_value_heads
    D = getattr(cfg, "head_dim", None) or Dm // Hq
    Fi = cfg.intermediate_size
    pattern = (cfg.hybrid_override_pattern or "-".join(["*"] * L)).split("-")
    total = 0.0
    for sym in pattern:
        proj = 2 * Dm * (Hq * D + 2 * Hkv * D) + 2 * Hq * D * Dm
        if sym.startswith("*") or sym.startswith("SWA"):
            ctx = seq_len / 2 if sym.startswith("*") else min(seq_len, (getattr(cfg, "swa_config", None) or {}).get("window_size", 2048))
            mix = 4 * Hq * D * ctx
        else:
            proj += 2 * Dm * Hq * D                      # output gate projection
            mix = 6 * Hq * D * D                         # state update + read (+ intra-chunk work of similar size)
        if getattr(cfg, "num_experts", None):
            mlp = 6 * Dm * cfg.moe_intermediate_size * cfg.num_experts_per_tok
        else:
            mlp = 6 * Dm * Fi
        total += proj + mix + mlp
    total += 2 * Dm * cfg.vocab_size
    return total * (3.0 if backward else 1.0)


def mfu(tokens_per_second: float, cfg, seq_len: int, peak_flops: float, n_gpus: int = 1) -> float:
    return tokens_per_second * flops_per_token(cfg, seq_len) / (peak_flops * n_gpus)


def suggest_lr(batch_tokens: int, base_lr: float = 3e-4, base_tokens: int = 4_000_000, rule: str = "sqrt") -> float:
    ratio = batch_tokens / base_tokens
    return base_lr * (math.sqrt(ratio) if rule == "sqrt" else ratio)


@torch.no_grad()
def perplexity(model, batches: Iterable[Dict[str, torch.Tensor]]) -> float:
    nll, n = 0.0, 0
    for b in batches:
        out = model(b["input_ids"], labels=b["labels"])
        valid = int((b["labels"][:, 1:] != -100).sum())
        nll += float(out.loss) * valid
        n += valid
    return math.exp(nll / max(n, 1))


def length_cdf(lengths: Sequence[int], points: Sequence[int] = (512, 1024, 2048, 4096, 8192, 16384, 32768, 65536, 131072)):
    n = max(len(lengths), 1)
    return {p: sum(1 for x in lengths if x <= p) / n for p in points}
