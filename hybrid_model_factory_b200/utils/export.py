"""``hmf export CKPT OUT [--dtype bf16|fp16|fp32] [--max-shard-size 5GB]``: re-shard / cast a checkpoint."""
from __future__ import annotations

import argparse
import json
import os
import shutil

import torch

from . import checkpoint_io

DTYPES = {"bf16": torch.bfloat16, "bfloat16": torch.bfloat16, "fp16": torch.float16, "float16": torch.float16,
          "fp32": torch.float32, "float32": torch.float32}


def export(src: str, dst: str, dtype: str = None, max_shard_size="5GB") -> str:
    os.makedirs(dst, exist_ok=True)
    state = checkpoint_io.load_state_dict(src)
    if dtype:
        dt = DTYPES[dtype]
        state = {k: (v.to(dt) if v.is_floating_point() else v) for k, v in state.items()}
    checkpoint_io.save_state_dict(state, dst, max_shard_size)
    for name in os.listdir(src):
        if name.endswith((".json", ".txt", ".model", ".jinja")) and not name.endswith("index.json"):
            shutil.copy(os.path.join(src, name), os.path.join(dst, name))
    if dtype and os.path.exists(os.path.join(dst, "config.json")):
        with open(os.path.join(dst, "config.json")) as f:
            cfg = json.load(f)
        cfg["torch_dtype"] = str(DTYPES[dtype]).replace("torch.", "")
        with open(os.path.join(dst, "config.json"), "w") as f:
            json.dump(cfg, f, indent=2)
    return dst


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="hmf export")
    ap.add_argument("src")
    ap.add_argument("dst")
    ap.add_argument("--dtype", default=None, choices=sorted(DTYPES))
    ap.add_argument("--max-shard-size", default="5GB")
    a = ap.parse_args(argv)
    print(export(a.src, a.dst, a.dtype, a.max_shard_size))
    return 0
