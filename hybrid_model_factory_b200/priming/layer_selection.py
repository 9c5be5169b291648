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
    if cfg.get("hybrid_override_pattern"):
        pattern = cfg["hybrid_override_pattern"].split("-")
    else:                                   # a plain Transformer checkpoint: attention everywhere
        pattern = ["*"] * int(cfg["num_hidden_layers"])
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


def read_task_scores(csv_path: str, task_filter: str = None):
    """CSV of benchmark scores per single-layer variant: a ``layer_num`` column, one column per task; the row with
    ``layer_num = -1`` is the unmodified model.  Returns ``(scores: layer -> {task: score}, baseline or None, tasks)``;
    ``task_filter`` keeps the task columns whose name contains it."""
    with open(csv_path) as f:
        rows = list(csv.DictReader(f))
    if not rows or "layer_num" not in rows[0]:
        raise ValueError(f"{csv_path}: expected a 'layer_num' column followed by one column per task")
    tasks = [k for k in rows[0] if k != "layer_num" and (task_filter is None or task_filter in k)]
    if not tasks:
        raise ValueError(f"{csv_path}: no task column matches '{task_filter}'")
    scores, baseline = {}, None
    for rec in rows:
        vals = {t: float(rec[t]) for t in tasks}
        if int(rec["layer_num"]) == -1:
            baseline = vals
        else:
            scores[int(rec["layer_num"])] = vals
    return scores, baseline, tasks


def select_layers(csv_path: str, M: int, task_filter: str = None, exclude_layer_0: bool = False):
    """The ``M`` layers whose replacement keeps most of the model's score (mean over tasks, highest first).  Returns
    ``(selected layer indices, full ranking [(layer, mean score)], baseline mean or None)``."""
    scores, baseline, tasks = read_task_scores(csv_path, task_filter)
    ranked = sorted(((l, sum(v.values()) / len(tasks)) for l, v in scores.items()
                     if not (exclude_layer_0 and l == 0)), key=lambda x: x[1], reverse=True)
    base = None if baseline is None else sum(baseline.values()) / len(tasks)
    return sorted(l for l, _ in ranked[:M]), ranked, base


def main(argv=None) -> int:
    """``hmf select-layers``: rank (``rank``) or make the per-layer variants (``variants``)."""
    import argparse
    ap = argparse.ArgumentParser(prog="hmf select-layers")
    sub = ap.add_subparsers(dest="what", required=True)
    r = sub.add_parser("rank", help="choose the layers to replace from a CSV of per-variant benchmark scores")
    r.add_argument("csv")
    r.add_argument("--M", type=int, default=14, help="number of layers to replace")
    r.add_argument("--task-filter", default=None)
    r.add_argument("--exclude-layer-0", action="store_true")
    r.add_argument("--num-layers", type=int, default=None, help="print a hybrid_override_pattern of this length")
    r.add_argument("--symbol", default="GDN")
    v = sub.add_parser("variants", help="one directory per layer with that layer turned into sliding-window attention")
    v.add_argument("src")
    v.add_argument("dst")
    v.add_argument("--window-size", type=int, default=2048)
    a = ap.parse_args(argv)
    if a.what == "variants":
        for d in create_swa_variants(a.src, a.dst, a.window_size):
            print(d)
        return 0
    selected, ranked, base = select_layers(a.csv, a.M, a.task_filter, a.exclude_layer_0)
    if base is not None:
        print(f"baseline mean: {base:.4f}")
    for i, (layer, score) in enumerate(ranked):
        drop = "" if base is None else f" | drop: {score - base:+.4f}"
        print(f"  {i + 1:2d}. layer {layer:2d}  score: {score:.4f}{drop}")
    print(f"selected (M={a.M}): {selected}")
    if a.num_layers:
        print("-".join(a.symbol if i in set(selected) else "*" for i in range(a.num_layers)))
    return 0
