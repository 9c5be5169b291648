"""Layer-selection helpers: which attention layers to replace first, and per-layer SWA variants of a checkpoint.

``rank_layers`` reads a CSV of per-layer scores (``layer,score`` with a header; lower score = less harmful to
replace) and returns a hybrid pattern that keeps the ``keep`` most important attention layers.
``create_swa_variants`` makes one directory per layer whose config turns exactly that layer into sliding-window
attention; weights are shared by symbolic links.  Reference: ``vllm-inference/selection/layer_selection.py:22-78``,
``create_swa_variants.py``.
"""
from __future__ import annotations

import csv
import json
import os
from typing import List, Tuple


def read_scores(csv_path: str) -> List[Tuple[int, float]]:
    rows = []
    with open(csv_path) as f:
        for rec in csv.DictReader(f):
            keys = {k.lower(): v for k, v in rec.items()}
            rows.append((int(keys.get("layer", keys.get("layer_idx"))), float(keys.get("score", keys.get("delta")))))
    return rows


def rank_layers(csv_path: str, num_layers: int, keep: int, symbol: str = "GDN") -> str:
    """Keeps attention in the ``keep`` layers with the highest score, ``symbol`` elsewhere."""
    scores = dict(read_scores(csv_path))
    order = sorted(range(num_layers), key=lambda i: scores.get(i, 0.0), reverse=True)
    attn = set(order[:keep])
    return "-".join("*" if i in attn else symbol for i in range(num_layers))


def create_swa_variants(ckpt: str, out_root: str, window: int = 2048) -> List[str]:
    with open(os.path.join(ckpt, "config.json")) as f:
        cfg = json.load(f)
    pattern = cfg["hybrid_override_pattern"].split("-")
    out = []
    for i, sym in enumerate(pattern):
        if sym != "*":
            continue
        d = os.path.join(out_root, f"swa_layer_{i}")
        os.makedirs(d, exist_ok=True)
        for name in os.listdir(ckpt):
            src, dst = os.path.join(ckpt, name), os.path.join(d, name)
            if name != "config.json" and not os.path.lexists(dst):
                os.symlink(os.path.abspath(src), dst)
        variant = dict(cfg)
        variant["hybrid_override_pattern"] = "-".join("SWA" if j == i else s for j, s in enumerate(pattern))
        variant["swa_config"] = {**(cfg.get("swa_config") or {}), "window_size": window}
        with open(os.path.join(d, "config.json"), "w") as f:
            json.dump(variant, f, indent=2)
        out.append(d)
    return out
