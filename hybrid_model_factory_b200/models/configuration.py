"""Model configuration: HF ``config.json`` compatible, no dependency on ``transformers``.

One ``HybridConfig`` class serves every family; ``model_type`` selects the family defaults
(attention flavour, norm flavour, MoE) and the extra keys written by stage-0 priming
(``hybrid_override_pattern``, ``layer_types``, ``gdn_config``, ``gka_config``, ``mamba2_config``,
``bmojo_config``, ``swa_config``) are carried verbatim.
Reference: ``models/model_register.py:74-221``, ``priming/utils.py:139-221``,
``models/hybrid_qwen3/configuration_hybrid_qwen3.py``.
"""
from __future__ import annotations

import copy
import json
import os
from typing import Any, Dict, List, Optional

from .patterns import expand_pattern_for_layers, parse_override_pattern, pattern_to_layer_types

# family defaults keyed by model_type
FAMILY_DEFAULTS: Dict[str, Dict[str, Any]] = {
    "hybrid_qwen3": dict(use_qk_norm=True, attention_bias=False, rope_theta=1e6, rms_norm_eps=1e-6,
                         architectures=["HybridQwen3ForCausalLM"]),
    "hybrid_qwen2": dict(use_qk_norm=False, qkv_bias=True, rope_theta=1e6, rms_norm_eps=1e-6,
                         architectures=["HybridQwen2ForCausalLM"]),
    "hybrid_llama": dict(use_qk_norm=False, attention_bias=False, rope_theta=5e5, rms_norm_eps=1e-5,
                         architectures=["HybridLlamaForCausalLM"]),
    "hybrid_ministral3": dict(use_qk_norm=False, attention_bias=False, rope_theta=1e6, rms_norm_eps=1e-5,
                              architectures=["HybridMinistral3ForCausalLM"]),
    "hybrid_qwen3_moe": dict(use_qk_norm=True, attention_bias=False, rope_theta=1e6, rms_norm_eps=1e-6,
                             num_experts=128, num_experts_per_tok=8, moe_intermediate_size=768,
                             norm_topk_prob=True, decoder_sparse_step=1, mlp_only_layers=[],
                             router_aux_loss_coef=0.001, architectures=["HybridQwen3MoeForCausalLM"]),
    "qwen3_next_hmf": dict(use_qk_norm=True, attention_bias=False, rope_theta=1e7, rms_norm_eps=1e-6,
                           gated_attention=True, zero_centered_norm=True, partial_rotary_factor=0.25,
                           num_experts=512, num_experts_per_tok=10, moe_intermediate_size=512,
                           shared_expert_intermediate_size=512, norm_topk_prob=True, decoder_sparse_step=1,
                           mlp_only_layers=[], router_aux_loss_coef=0.001, full_attention_interval=4,
                           linear_num_key_heads=16, linear_num_value_heads=32, linear_key_head_dim=128,
                           linear_value_head_dim=128, linear_conv_kernel_dim=4,
                           architectures=["Qwen3NextHMFForCausalLM"]),
}
FAMILY_DEFAULTS["qwen3_5_moe_hmf_text"] = dict(FAMILY_DEFAULTS["qwen3_next_hmf"],
                                               architectures=["Qwen3_5MoeHMFForCausalLM"])
FAMILY_DEFAULTS["qwen3_5_moe_hmf"] = dict(FAMILY_DEFAULTS["qwen3_next_hmf"],
                                          architectures=["Qwen3_5MoeHMFForConditionalGeneration"])
FAMILY_DEFAULTS["hybrid_qwen2_5_vl"] = dict(FAMILY_DEFAULTS["hybrid_qwen2"],
                                            architectures=["HybridQwen2_5_VLForConditionalGeneration"])

# base (non-hybrid) HF model types and the hybrid family they are primed into
BASE_TO_HYBRID = {
    "qwen3": "hybrid_qwen3", "qwen2": "hybrid_qwen2", "llama": "hybrid_llama", "ministral3": "hybrid_ministral3",
    "mistral": "hybrid_ministral3", "qwen3_moe": "hybrid_qwen3_moe", "qwen3_next": "qwen3_next_hmf",
    "qwen3_5_moe": "qwen3_5_moe_hmf", "qwen3_5_moe_text": "qwen3_5_moe_hmf_text", "qwen2_5_vl": "hybrid_qwen2_5_vl",
}

_COMMON_DEFAULTS = dict(
    vocab_size=151936, hidden_size=4096, intermediate_size=12288, num_hidden_layers=36, num_attention_heads=32,
    num_key_value_heads=8, head_dim=None, hidden_act="silu", max_position_embeddings=40960, initializer_range=0.02,
    rms_norm_eps=1e-6, use_cache=True, tie_word_embeddings=False, rope_theta=1e6, rope_scaling=None,
    attention_bias=False, qkv_bias=False, use_qk_norm=False, sliding_window=None, attention_dropout=0.0,
    gated_attention=False, zero_centered_norm=False, partial_rotary_factor=1.0, mlp_bias=False,
    hybrid_override_pattern=None, layer_types=None, gdn_config=None, gka_config=None, mamba2_config=None,
    bmojo_config=None, swa_config=None, gka_overrides=None, torch_dtype="bfloat16", bos_token_id=None,
    eos_token_id=None, pad_token_id=None, num_experts=0, num_experts_per_tok=0, moe_intermediate_size=0,
    shared_expert_intermediate_size=0, norm_topk_prob=True, decoder_sparse_step=1, mlp_only_layers=None,
    router_aux_loss_coef=0.0, output_router_logits=False,
)


class HybridConfig:
    """Attribute bag with HF-compatible (de)serialisation."""

    def __init__(self, model_type: str = "hybrid_qwen3", **kwargs):
        if model_type in BASE_TO_HYBRID:
            model_type = BASE_TO_HYBRID[model_type]
        if model_type not in FAMILY_DEFAULTS:
            raise ValueError(f"unknown model_type '{model_type}'; known: {sorted(FAMILY_DEFAULTS)}")
        self.model_type = model_type
        values = dict(_COMMON_DEFAULTS)
        values.update(copy.deepcopy(FAMILY_DEFAULTS[model_type]))
        if "text_config" in kwargs and isinstance(kwargs["text_config"], dict):
            # composite (VL) configs keep the language-model fields in text_config
            values.update(kwargs["text_config"])
        values.update(kwargs)
        if "num_local_experts" in kwargs and "num_experts" not in kwargs:      # newer serialisations name it so
            values["num_experts"] = kwargs["num_local_experts"]
        for k, v in values.items():
            setattr(self, k, v)
        self._sync_rope(prefer_parameters="rope_theta" not in kwargs and "rope_scaling" not in kwargs)
        if self.head_dim is None:
            self.head_dim = self.hidden_size // self.num_attention_heads
        if self.num_key_value_heads is None:
            self.num_key_value_heads = self.num_attention_heads
        if self.hybrid_override_pattern is None:
            self.hybrid_override_pattern = "-".join(["*"] * self.num_hidden_layers)
        pat = parse_override_pattern(self.hybrid_override_pattern)
        if len(pat) != self.num_hidden_layers:
            raise ValueError(f"hybrid_override_pattern has {len(pat)} entries but num_hidden_layers="
                             f"{self.num_hidden_layers}")
        if getattr(self, "native_window_layers", None) is None:
            self.native_window_layers = self._native_window_layers(pat)
        plain = isinstance(self.layer_types, (list, tuple)) and \
            set(self.layer_types) <= {"full_attention", "sliding_attention"}
        if self.layer_types is None or (plain and "hybrid_override_pattern" not in kwargs):
            # (a plain Transformer's list: its sliding layers are now in native_window_layers, the symbols are all `*`)
            self.layer_types = pattern_to_layer_types(self.hybrid_override_pattern)
        if self.mlp_only_layers is None:
            self.mlp_only_layers = []

    def _native_window_layers(self, pat) -> List[int]:
        """Attention layers (symbol ``*``) that the base architecture runs with its own ``sliding_window``: where the
        checkpoint's ``layer_types`` say ``sliding_attention``; for older configs without that list, every layer of
        a Mistral-family model, and the layers from ``max_window_layers`` on of a Qwen model with
        ``use_sliding_window``."""
        if not getattr(self, "sliding_window", None):
            return []
        n = self.num_hidden_layers
        types = self.layer_types
        if isinstance(types, (list, tuple)) and len(types) == n and set(types) <= {"full_attention", "sliding_attention"}:
            chosen = [i for i, t in enumerate(types) if t == "sliding_attention"]
        elif "ministral" in self.model_type:
            chosen = list(range(n))
        elif getattr(self, "use_sliding_window", False):
            chosen = list(range(int(getattr(self, "max_window_layers", 0) or 0), n))
        else:
            chosen = []
        return [i for i in chosen if pat[i] == "*"]

    def _sync_rope(self, prefer_parameters: bool) -> None:
        """Newer checkpoints describe the rotary embedding in one ``rope_parameters`` dict (``rope_theta``,
        ``rope_type`` and the scaling fields, optionally ``partial_rotary_factor``), older ones in ``rope_theta`` +
        ``rope_scaling``.  The model reads the older pair; this keeps the two views equal, taking the dict as the
        source when ``prefer_parameters`` (a config file that holds it) and the pair otherwise (explicit overrides)."""
        rp = getattr(self, "rope_parameters", None)
        if isinstance(rp, dict) and rp and prefer_parameters:
            if rp.get("rope_theta") is not None:
                self.rope_theta = float(rp["rope_theta"])
            kind = rp.get("rope_type", rp.get("type", "default"))
            rest = {k: v for k, v in rp.items() if k not in ("rope_theta", "partial_rotary_factor")}
            self.rope_scaling = rest if kind not in (None, "default") else None
            if rp.get("partial_rotary_factor") is not None and hasattr(self, "partial_rotary_factor"):
                self.partial_rotary_factor = float(rp["partial_rotary_factor"])
        if isinstance(rp, dict) and rp:
            new = dict(self.rope_scaling or {"rope_type": "default"})
            new["rope_theta"] = self.rope_theta
            if rp.get("partial_rotary_factor") is not None:
                new["partial_rotary_factor"] = getattr(self, "partial_rotary_factor", rp["partial_rotary_factor"])
            self.rope_parameters = new

    # -- helpers ----------------------------------------------------------------------
    @property
    def pattern(self) -> List[str]:
        p = parse_override_pattern(self.hybrid_override_pattern)
        return [p[i] for i in range(len(p))]

    @property
    def is_moe(self) -> bool:
        return bool(self.num_experts and self.num_experts > 0)

    def layer_is_moe(self, layer_idx: int) -> bool:
        if not self.is_moe or layer_idx in (self.mlp_only_layers or []):
            return False
        step = max(int(self.decoder_sparse_step or 1), 1)
        return (layer_idx + 1) % step == 0

    def to_dict(self) -> Dict[str, Any]:
        out = {k: copy.deepcopy(v) for k, v in self.__dict__.items() if not k.startswith("_")}
        for k in ("gdn_config", "gka_config", "mamba2_config", "bmojo_config", "swa_config"):
            if out.get(k) is not None and hasattr(out[k], "to_dict"):
                out[k] = out[k].to_dict()
        return out

    @classmethod
    def from_dict(cls, d: Dict[str, Any]) -> "HybridConfig":
        d = dict(d)
        mt = d.pop("model_type", "hybrid_qwen3")
        return cls(model_type=mt, **d)

    def to_json_string(self) -> str:
        return json.dumps(self.to_dict(), indent=2, sort_keys=True, default=str) + "\n"

    def save_pretrained(self, path: str) -> None:
        os.makedirs(path, exist_ok=True)
        with open(os.path.join(path, "config.json"), "w") as f:
            f.write(self.to_json_string())

    @classmethod
    def from_pretrained(cls, path: str, **overrides) -> "HybridConfig":
        fn = os.path.join(path, "config.json") if os.path.isdir(path) else path
        with open(fn) as f:
            d = json.load(f)
        d.update(overrides)
        return cls.from_dict(d)

    def apply_overrides(self, overrides: Dict[str, Any]) -> None:
        """Dotted-key overrides, e.g. ``{"gka_config.num_iter": 10, "rope_theta": 5e6}``
        (reference: ``model/loader.py:132-170``)."""
        for key, value in (overrides or {}).items():
            parts = key.split(".")
            target = self
            for p in parts[:-1]:
                nxt = target[p] if isinstance(target, dict) else getattr(target, p)
                if nxt is None:
                    nxt = {}
                    if isinstance(target, dict):
                        target[p] = nxt
                    else:
                        setattr(target, p, nxt)
                target = nxt
            if isinstance(target, dict):
                target[parts[-1]] = value
            else:
                setattr(target, parts[-1], value)
        keys = list(overrides or {})
        if any(k.startswith("rope_parameters") for k in keys):
            self._sync_rope(prefer_parameters=True)
        elif any(k.split(".")[0] in ("rope_theta", "rope_scaling") for k in keys):
            self._sync_rope(prefer_parameters=False)

    def __repr__(self):
        return f"HybridConfig({self.model_type}, layers={self.num_hidden_layers}, hidden={self.hidden_size}, " \
               f"pattern={self.hybrid_override_pattern})"


def qwen3_8b_config(pattern: Optional[str] = None, **kw) -> HybridConfig:
    """Qwen3-8B backbone dimensions (36 layers, hidden 4096, SwiGLU 12288, 32/8 heads, head_dim 128)."""
    base = dict(vocab_size=151936, hidden_size=4096, intermediate_size=12288, num_hidden_layers=36,
                num_attention_heads=32, num_key_value_heads=8, head_dim=128, rope_theta=1e6,
                max_position_embeddings=131072)
    base.update(kw)
    n = base["num_hidden_layers"]
    if pattern is None:
        pattern = "-".join(["*"] * n)
    else:
        pattern = expand_pattern_for_layers(pattern, n)
    return HybridConfig("hybrid_qwen3", hybrid_override_pattern=pattern, **base)
