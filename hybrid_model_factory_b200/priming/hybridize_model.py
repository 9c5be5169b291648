"""Stage 0 ("prime-init"): turn a pretrained Transformer checkpoint into a hybrid model without
training.  Input is a YAML file with ``base_model_name_or_path``, ``hybrid_override_pattern``,
``output_dir``, optional ``dtype`` / ``copy_auxiliary_files`` and one block of knobs per layer
family (``gdn:``, ``gka:``, ``mamba2:``, ``bmojo:``, ``swa:``).  Entirely host side.

Steps: read the base ``config.json`` -> hybrid config (pattern, per-family ``*_config`` dicts derived
from the base dimensions) -> instantiate the hybrid model -> copy every tensor whose name and
shape exist in the base checkpoint -> initialise each replaced mixer from the attention weights
of its layer -> save safetensors shards of at most 5 GB plus ``config.json``.
Reference: ``priming/hybridize_model.py:78-332``, ``priming/utils.py:75-288``,
``layers/hybrid_dataclasses.py:7-170``.
"""
from __future__ import annotations

import json
import os
import shutil
from dataclasses import dataclass, field
from typing import Dict, Optional

import torch
import yaml

from ..layers.gdn import construct_gdn_config
from ..layers.gka import construct_gka_config
from ..layers.mamba2 import construct_mamba2_config
from ..models.configuration import BASE_TO_HYBRID, HybridConfig
from ..models.modeling_hybrid import FusedDecoderLayer, build_model
from ..models.patterns import LAYER_SYMBOLS, parse_override_pattern, unfuse_symbol
from ..utils import checkpoint_io
from ..utils.logging import get_logger
from .hybrid_layer_init import extract_attention_weights, init_mixer

logger = get_logger(__name__)

_DTYPES = {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16, "float16": torch.float16, "fp16": torch.float16,
           "float32": torch.float32, "fp32": torch.float32}
_AUX_FILES = ("tokenizer.json", "tokenizer_config.json", "vocab.json", "merges.txt", "special_tokens_map.json",
              "generation_config.json", "added_tokens.json", "tokenizer.model", "chat_template.jinja",
              "preprocessor_config.json")


@dataclass
class HybridizationConfig:
    base_model_name_or_path: str
    hybrid_override_pattern: str
    output_dir: str
    dtype: str = "bfloat16"
    copy_auxiliary_files: bool = False
    swa: Optional[dict] = None
    bmojo: Optional[dict] = None
    mamba2: Optional[dict] = None
    gka: Optional[dict] = None
    gdn: Optional[dict] = None
    l2a: Optional[dict] = None           # sliding_window, sigmoid_threshold, temperature, leak_prob, router_zero_init
    extra: dict = field(default_factory=dict)


def load_config(path_or_dict) -> HybridizationConfig:
    if isinstance(path_or_dict, dict):
        raw = dict(path_or_dict)
    else:
        with open(path_or_dict) as f:
            raw = yaml.safe_load(f)
    known = {k: raw.pop(k) for k in list(raw) if k in HybridizationConfig.__dataclass_fields__ and k != "extra"}
    if isinstance(known.get("dtype"), torch.dtype):
        known["dtype"] = str(known["dtype"]).replace("torch.", "")
    return HybridizationConfig(**known, extra=raw)


def verify_hybrid_config(cfg: HybridizationConfig, num_layers: int) -> None:
    pat = parse_override_pattern(cfg.hybrid_override_pattern)  # raises on unknown symbols
    if len(pat) != num_layers:
        raise ValueError(f"hybrid_override_pattern has {len(pat)} symbols but the base model has {num_layers} layers")
    for i, s in pat.items():
        assert s in LAYER_SYMBOLS, (i, s)


def add_hybrid_configs(base: HybridConfig, cfg: HybridizationConfig) -> Dict[str, dict]:
    """Per-family config dicts stored in ``config.json`` (derived dims + user knobs)."""
    symbols = {unfuse_symbol(s) for s in cfg.hybrid_override_pattern.split("-")} | \
              ({"GDN"} if "GDN>GKA" in cfg.hybrid_override_pattern else set())
    out: Dict[str, dict] = {}
    bmojo_inner = (cfg.bmojo or {}).get("ssm_mixer", "mamba2").lower() if "BMF" in symbols else None
    if "GDN" in symbols or bmojo_inner in ("gdn", "gated_deltanet"):
        out["gdn_config"] = construct_gdn_config(base, cfg.gdn).to_dict()
    if "GKA" in symbols or bmojo_inner in ("gka", "gated_kalmanet"):
        out["gka_config"] = construct_gka_config(base, cfg.gka).to_dict()
    if "M2" in symbols or bmojo_inner == "mamba2":
        out["mamba2_config"] = construct_mamba2_config(base, cfg.mamba2).to_dict()
    if "BMF" in symbols:
        b = dict(cfg.bmojo or {})
        out["bmojo_config"] = {"window_size": int(b.get("window_size", 2048)),
                               "tie_attn_weights": bool(b.get("tie_attn_weights", True)),
                               "ssm_mixer": str(b.get("ssm_mixer", "mamba2"))}
    if "SWA" in symbols:
        if not cfg.swa or "window_size" not in cfg.swa:
            raise ValueError("pattern uses SWA layers but the config has no `swa.window_size`")
        out["swa_config"] = {"window_size": int(cfg.swa["window_size"])}
    if "L2A" in symbols:
        l2a = dict(cfg.l2a or {})
        if "sliding_window" not in l2a:
            raise ValueError("pattern uses L2A layers but the config has no `l2a.sliding_window`")
        out["l2a_config"] = {"sliding_window": int(l2a["sliding_window"]),
                             "sigmoid_threshold": float(l2a.get("sigmoid_threshold", 0.5)),
                             "temperature": float(l2a.get("temperature", 0.1)),
                             "leak_prob": float(l2a.get("leak_prob", 0.1))}
    return out


def hybridize_state(base_cfg: HybridConfig, base_state: Dict[str, torch.Tensor], cfg: HybridizationConfig):
    """Builds the hybrid model and fills it from ``base_state``.  Returns ``(model, report)``."""
    verify_hybrid_config(cfg, base_cfg.num_hidden_layers)
    d = base_cfg.to_dict()
    d.pop("model_type", None)
    d.update(add_hybrid_configs(base_cfg, cfg))
    d["hybrid_override_pattern"] = cfg.hybrid_override_pattern
    d["layer_types"] = None
    d["torch_dtype"] = cfg.dtype
    d.pop("quantization_config", None)
    hybrid_cfg = HybridConfig(base_cfg.model_type, **d)
    model = build_model(hybrid_cfg)
    own = dict(model.state_dict(keep_vars=True))
    copied, skipped = [], []
    with torch.no_grad():
        for k, t in base_state.items():
            if k in own and tuple(own[k].shape) == tuple(t.shape):
                own[k].data.copy_(t.to(own[k].dtype))
                copied.append(k)
            else:
                skipped.append(k)
        if hybrid_cfg.tie_word_embeddings and "lm_head.weight" not in base_state:
            model.lm_head.weight = model.model.embed_tokens.weight
        pat = parse_override_pattern(cfg.hybrid_override_pattern)
        for i, layer in enumerate(model.model.layers):
            sym = pat[i]
            if sym == "*":
                continue
            attn = extract_attention_weights(base_state, i)
            if isinstance(layer, FusedDecoderLayer):
                if sym == "*DA":
                    continue  # same attention weights on both streams: already copied by name
                if sym == "GDN>GKA":
                    init_mixer("GKA", attn, layer.seq_mixer, i)
                    continue
                init_mixer(unfuse_symbol(sym), attn, layer.seq_mixer, i)
            elif sym == "L2A":
                # both streams start as the attention they replace, the second norm as the layer's input norm, and
                # the router at zero (or random): the model then departs from the Transformer only by the window
                init_mixer("L2A", attn, layer.seq_mixer, i)
                norm = base_state.get(f"model.layers.{i}.input_layernorm.weight")
                if norm is not None:
                    layer.seq_mixer.global_norm.weight.data.copy_(norm.to(layer.seq_mixer.global_norm.weight.dtype))
                if (cfg.l2a or {}).get("router_zero_init", True):
                    layer.seq_mixer.router.weight.data.zero_()
            else:
                init_mixer(sym, attn, layer.seq_mixer, i)
    model = model.to(_DTYPES[cfg.dtype])
    report = {"copied": len(copied), "skipped": skipped}
    logger.info("stage 0: copied %d shared tensors, %d base tensors had no counterpart", len(copied), len(skipped))
    return model, report


def hybridize_model(cfg: HybridizationConfig):
    """Full stage-0 run from a checkpoint directory to ``cfg.output_dir``."""
    base_dir = cfg.base_model_name_or_path
    with open(os.path.join(base_dir, "config.json")) as f:
        raw = json.load(f)
    mt = raw.get("model_type", "qwen3")
    if mt not in BASE_TO_HYBRID and not mt.startswith("hybrid") and not mt.endswith("_hmf"):
        raise ValueError(f"unsupported base model_type '{mt}'; supported: {sorted(BASE_TO_HYBRID)}")
    raw.setdefault("use_qk_norm", mt in ("qwen3", "qwen3_moe", "qwen3_next", "qwen3_5_moe"))
    raw.pop("hybrid_override_pattern", None)
    base_cfg = HybridConfig.from_dict(raw)
    base_state = checkpoint_io.load_state_dict(base_dir)
    model, report = hybridize_state(base_cfg, base_state, cfg)
    checkpoint_io.save_pretrained(model, cfg.output_dir, max_shard_size="5GB")
    if cfg.copy_auxiliary_files:
        for fn in _AUX_FILES:
            src = os.path.join(base_dir, fn)
            if os.path.exists(src):
                shutil.copy(src, os.path.join(cfg.output_dir, fn))
    return model, report


def main(config_path: str):
    cfg = load_config(config_path)
    return hybridize_model(cfg)
