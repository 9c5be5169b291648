"""Loss curves from ``trainer_log.jsonl`` (``plot_loss: true``; reference: ``extras/ploting.py``).

Writes ``training_loss.png`` (and ``training_eval_loss.png`` when evaluation losses were logged) with matplotlib
when it is importable, else the same curves as a dependency-free ``.svg``.  The smoothed curve is the exponential
moving average the reference draws, with its weight chosen from the curve length by the same sigmoid rule.
"""
from __future__ import annotations

import json
import math
import os
from typing import List, Optional, Sequence, Tuple


def smooth(scalars: Sequence[float]) -> List[float]:
    """EMA smoothing; the weight grows with the number of points (``1.8 * (sigmoid(n / 1000 * e) - 0.5)``)."""
    if not scalars:
        return []
    weight = 1.8 * (1 / (1 + math.exp(-1e-3 * len(scalars))) - 0.5)
    last, out = scalars[0], []
    for v in scalars:
        last = last * weight + (1 - weight) * v
        out.append(last)
    return out


def read_log(output_dir: str, key: str) -> Tuple[List[int], List[float]]:
    path = os.path.join(output_dir, "trainer_log.jsonl")
    steps, vals = [], []
    if os.path.exists(path):
        with open(path) as f:
            for line in f:
                line = line.strip()
                if not line:
                    continue
                rec = json.loads(line)
                if key in rec and isinstance(rec[key], (int, float)) and math.isfinite(rec[key]):
                    steps.append(int(rec.get("current_steps", len(steps) + 1)))
                    vals.append(float(rec[key]))
    return steps, vals


def _svg(steps, vals, smoothed, title: str) -> str:
    W, H, L, B = 640, 400, 60, 40
    lo, hi = min(vals + smoothed), max(vals + smoothed)
    span = (hi - lo) or 1.0
    x0, x1 = steps[0], steps[-1] if steps[-1] != steps[0] else steps[0] + 1

    def pts(ys):
        return " ".join(f"{L + (s - x0) / (x1 - x0) * (W - L - 20):.1f},{H - B - (y - lo) / span * (H - B - 30):.1f}"
                        for s, y in zip(steps, ys))
    return (f'<svg xmlns="http://www.w3.org/2000/svg" width="{W}" height="{H}" font-family="sans-serif" font-size="12">'
            f'<rect width="{W}" height="{H}" fill="white"/><text x="{W / 2}" y="18" text-anchor="middle">{title}</text>'
            f'<line x1="{L}" y1="{H - B}" x2="{W - 20}" y2="{H - B}" stroke="black"/>'
            f'<line x1="{L}" y1="30" x2="{L}" y2="{H - B}" stroke="black"/>'
            f'<text x="{L - 5}" y="{H - B}" text-anchor="end">{lo:.3g}</text><text x="{L - 5}" y="40" text-anchor="end">{hi:.3g}</text>'
            f'<text x="{L}" y="{H - B + 16}">{x0}</text><text x="{W - 20}" y="{H - B + 16}" text-anchor="end">{x1}</text>'
            f'<polyline fill="none" stroke="#1f77b4" stroke-opacity="0.4" points="{pts(vals)}"/>'
            f'<polyline fill="none" stroke="#1f77b4" stroke-width="2" points="{pts(smoothed)}"/>'
            f'<text x="{W / 2}" y="{H - 8}" text-anchor="middle">step</text></svg>')


def plot_loss(output_dir: str, keys: Sequence[str] = ("loss", "eval_loss")) -> List[str]:
    """One figure per key that was logged; returns the written paths."""
    written = []
    for key in keys:
        steps, vals = read_log(output_dir, key)
        if not steps:
            continue
        sm = smooth(vals)
        name = "training_" + key.replace("/", "_")
        title = f"training {key} of {os.path.basename(os.path.normpath(output_dir))}"
        try:
            import matplotlib
            matplotlib.use("Agg")
            import matplotlib.pyplot as plt
            plt.figure()
            plt.plot(steps, vals, color="#1f77b4", alpha=0.4, label="original")
            plt.plot(steps, sm, color="#1f77b4", label="smoothed")
            plt.title(title)
            plt.xlabel("step")
            plt.ylabel(key)
            plt.legend()
            path = os.path.join(output_dir, name + ".png")
            plt.savefig(path, format="png", dpi=100)
            plt.close()
        except ImportError:
            path = os.path.join(output_dir, name + ".svg")
            with open(path, "w") as f:
                f.write(_svg(steps, vals, sm, title))
        written.append(path)
    return written
