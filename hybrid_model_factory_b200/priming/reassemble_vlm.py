"""Puts a distilled hybrid text backbone back into its vision-language wrapper.

Stage 1/2 train the text decoder alone (``model.*`` / ``lm_head.*`` names).  ``reassemble_vlm`` copies the
vision tower (and everything else that is not text) from the original VL checkpoint, the decoder from the
hybrid text checkpoint (renamed to ``model.language_model.*``), and writes a checkpoint whose config has
``model_type = hybrid_qwen2_5_vl`` with the hybrid text config nested as ``text_config``.
Reference: ``reassemble_vlm.py:36-127``.
"""
from __future__ import annotations

import json
import os
import shutil
from typing import Dict

import torch

from ..utils import checkpoint_io

TEXT_PREFIXES = ("model.language_model.", "language_model.model.", "model.layers.", "model.embed_tokens.",
                 "model.norm.", "lm_head.")


def is_text_key(name: str) -> bool:
    return name.startswith(TEXT_PREFIXES)


def to_vl_name(name: str) -> str:
    if name.startswith("lm_head."):
        return name
    if name.startswith("model."):
        return "model.language_model." + name[len("model."):]
    return name


def reassemble_state(text_state: Dict[str, torch.Tensor], vl_state: Dict[str, torch.Tensor]) -> Dict[str, torch.Tensor]:
    out = {k: v for k, v in vl_state.items() if not is_text_key(k)}
    out.update({to_vl_name(k): v for k, v in text_state.items()})
    return out


def reassemble_vlm(text_ckpt: str, vl_ckpt: str, out_dir: str, max_shard_size="5GB") -> str:
    os.makedirs(out_dir, exist_ok=True)
    state = reassemble_state(checkpoint_io.load_state_dict(text_ckpt), checkpoint_io.load_state_dict(vl_ckpt))
    checkpoint_io.save_state_dict(state, out_dir, max_shard_size)
    with open(os.path.join(text_ckpt, "config.json")) as f:
        text_cfg = json.load(f)
    with open(os.path.join(vl_ckpt, "config.json")) as f:
        vl_cfg = json.load(f)
    vl_cfg["model_type"] = "hybrid_qwen2_5_vl"
    vl_cfg["architectures"] = ["HybridQwen2_5_VLForConditionalGeneration"]
    vl_cfg["text_config"] = text_cfg
    with open(os.path.join(out_dir, "config.json"), "w") as f:
        json.dump(vl_cfg, f, indent=2)
    for name in os.listdir(vl_ckpt):        # tokenizer / processor files travel with the wrapper
        if name.endswith((".json", ".txt", ".model", ".jinja")) and name != "config.json" \
                and not name.endswith("index.json"):
            shutil.copy(os.path.join(vl_ckpt, name), os.path.join(out_dir, name))
    return out_dir
