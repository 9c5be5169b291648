"""``prime-unfuse``: turn a stage-1 (fused, two-stream) checkpoint into the plain hybrid model used for
stage 2 and serving.  Pattern symbols are rewritten ``X* -> X``, ``*DA -> *``, ``A>B -> B``; a new
model is built for the rewritten pattern and every tensor whose name exists in both models is
copied (teacher-only weights are dropped); missing keys are reported.
Reference: ``priming/fused_to_standard.py:142-324``."""
from __future__ import annotations

import os
from typing import List, Tuple

import torch

from ..models.configuration import HybridConfig
from ..models.modeling_hybrid import build_model
from ..models.patterns import pattern_to_layer_types, unfuse_pattern
from ..utils import checkpoint_io
from ..utils.logging import get_logger

logger = get_logger(__name__)


def unfuse_config(cfg: HybridConfig) -> HybridConfig:
    d = cfg.to_dict()
    d["hybrid_override_pattern"] = unfuse_pattern(cfg.hybrid_override_pattern)
    d["layer_types"] = pattern_to_layer_types(d["hybrid_override_pattern"])
    return HybridConfig.from_dict(d)


def unfuse_model(fused_model) -> Tuple[torch.nn.Module, List[str]]:
    new_cfg = unfuse_config(fused_model.config)
    model = build_model(new_cfg)
    src = fused_model.state_dict()
    own = dict(model.state_dict(keep_vars=True))
    missing = []
    with torch.no_grad():
        for k, p in own.items():
            if k in src and tuple(src[k].shape) == tuple(p.shape):
                p.data.copy_(src[k].to(p.dtype))
            else:
                missing.append(k)
    if missing:
        logger.warning("unfuse: %d tensors of the standard model were not found in the fused checkpoint: %s",
                       len(missing), missing[:8])
    return model, missing


def unfuse_checkpoint(path: str, output_dir: str = None, dtype=torch.bfloat16) -> str:
    fused = checkpoint_io.from_pretrained(path, dtype=torch.float32)
    model, _ = unfuse_model(fused)
    out = output_dir or (path.rstrip("/") + "_unfused")
    checkpoint_io.save_pretrained(model.to(dtype), out)
    for fn in os.listdir(path):
        if fn.startswith("tokenizer") or fn in ("vocab.json", "merges.txt", "special_tokens_map.json",
                                                "generation_config.json", "chat_template.jinja"):
            import shutil
            shutil.copy(os.path.join(path, fn), os.path.join(out, fn))
    return out
