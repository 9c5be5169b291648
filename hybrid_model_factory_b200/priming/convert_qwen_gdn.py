"""Converters from released Qwen models that already contain Gated DeltaNet layers (Qwen3-Next, Qwen3.5-MoE) to
this framework's layout (``hmf convert-qwen-gdn``).

Source layouts of a ``linear_attn`` block:

* Qwen3-Next: fused and *interleaved per key head*: ``in_proj_qkvz [Hk * (2 dk + 2 r dv), hidden]`` with per-head
  blocks ``[q (dk) | k (dk) | v (r dv) | z (r dv)]`` (``r = Hv / Hk`` value heads per key head) and
  ``in_proj_ba [Hk * 2 r, hidden]`` with blocks ``[b (r) | a (r)]``;
* Qwen3.5-MoE: plain ``in_proj_qkv [q | k | v]``, ``in_proj_z``, ``in_proj_b``, ``in_proj_a``;
* both: one depthwise convolution over the ``[q | k | v]`` channels, ``A_log``, ``dt_bias``, ``norm``, ``out_proj``.

The hybrid layers keep separate ``q/k/v/g/b/gk`` projections and one convolution per stream under the decoder
layer's mixer attribute (``gdn.``, ``gka.``, ``self_attn.``: ``models/patterns.py::MIXER_ATTR``).  Per target symbol:

* ``linear_attention -> GDN``: exact (every tensor has a destination);
* ``linear_attention -> GKA``: q/k/v/g/o, the three convolutions, ``b_proj <- b``, ``a_proj <- a``, ``A_log``,
  ``dt_bias``, ``o_norm`` are copied; ``alpha_proj`` and the gate biases keep their fresh initialisation;
* ``linear_attention -> GDN>GKA`` (fused stage-1 layer): both of the above (GDN teacher, GKA student);
* ``full_attention -> *``: copied as is (gated attention keeps the ``[q | gate]`` rows of ``q_proj``);
* ``full_attention -> GDN | GKA | M2``: the stage-0 rules of ``priming/hybrid_layer_init.py`` applied to the attention
  weights, with the query rows taken out of the per-head ``[q | gate]`` blocks.

Multi-token-prediction heads (``mtp.*``) have no counterpart and are dropped; vision tensors are kept under their
own names for the VL wrapper or dropped for a text-only target.  The result is loaded into a freshly built target
model with a check that every parameter was either converted or is on the list of parameters that are meant to keep
their initial values, so a naming mismatch cannot pass silently.

Reference: ``priming/convert_qwen_gdn_models.py:57-1009``, ``convert_qwen3_next.py:31-248``,
``convert_qwen3_5_moe.py:33-204``.
"""
from __future__ import annotations

import json
import os
import re
from typing import Dict, List, Optional, Tuple

import torch

from ..models.patterns import MIXER_ATTR, parse_override_pattern, unfuse_symbol

# parameters of a target mixer that have no source and keep the values the target model was built with
FRESH_OK = {
    ("linear", "GKA"): ("alpha_proj.", "b_proj.bias"),
    ("full", "GDN"): ("q_conv1d.", "k_conv1d.", "v_conv1d.", "b_proj.", "gk_proj.", "A_log", "dt_bias", "o_norm."),
    ("full", "GKA"): ("q_conv1d.", "k_conv1d.", "v_conv1d.", "b_proj.", "a_proj.", "alpha_proj.", "A_log", "dt_bias",
                      "o_norm."),
    ("full", "M2"): ("conv1d.", "A_log", "dt_bias", "D", "norm.", "in_proj."),
}


def deinterleave_qkvz(w: torch.Tensor, Hk: int, Hv: int, dk: int, dv: int) -> Tuple[torch.Tensor, ...]:
    """``w [Hk * (2 dk + 2 r dv), in]`` -> ``(q [Hk dk, in], k [Hk dk, in], v [Hv dv, in], z [Hv dv, in])``."""
    r = Hv // Hk
    blk = w.view(Hk, 2 * dk + 2 * r * dv, -1)
    q, k, v, z = torch.split(blk, [dk, dk, r * dv, r * dv], dim=1)
    return (q.reshape(Hk * dk, -1), k.reshape(Hk * dk, -1), v.reshape(Hv * dv, -1), z.reshape(Hv * dv, -1))


def deinterleave_ba(w: torch.Tensor, Hk: int, Hv: int) -> Tuple[torch.Tensor, torch.Tensor]:
    r = Hv // Hk
    blk = w.view(Hk, 2 * r, -1)
    b, a = torch.split(blk, [r, r], dim=1)
    return b.reshape(Hv, -1), a.reshape(Hv, -1)


def interleave_qkvz(q, k, v, z, Hk: int, Hv: int, dk: int, dv: int) -> torch.Tensor:
    """Inverse of :func:`deinterleave_qkvz` (export back to the Qwen3-Next layout, and the round-trip test)."""
    r = Hv // Hk
    parts = [q.view(Hk, dk, -1), k.view(Hk, dk, -1), v.view(Hk, r * dv, -1), z.view(Hk, r * dv, -1)]
    return torch.cat(parts, dim=1).reshape(Hk * (2 * dk + 2 * r * dv), -1)


def interleave_ba(b, a, Hk: int, Hv: int) -> torch.Tensor:
    r = Hv // Hk
    return torch.cat([b.view(Hk, r, -1), a.view(Hk, r, -1)], dim=1).reshape(2 * Hv, -1)


def extract_linear_attn(prefix: str, src: Dict[str, torch.Tensor], Hk: int, Hv: int, dk: int, dv: int) -> Dict[str, torch.Tensor]:
    """De-interleaved tensors of one ``linear_attn`` block, whichever of the two source layouts it uses."""
    if prefix + "in_proj_qkvz.weight" in src:
        q, k, v, z = deinterleave_qkvz(src[prefix + "in_proj_qkvz.weight"], Hk, Hv, dk, dv)
        b, a = deinterleave_ba(src[prefix + "in_proj_ba.weight"], Hk, Hv)
    elif prefix + "in_proj_qkv.weight" in src:
        q, k, v = torch.split(src[prefix + "in_proj_qkv.weight"], [Hk * dk, Hk * dk, Hv * dv], dim=0)
        z, b, a = (src[prefix + n + ".weight"] for n in ("in_proj_z", "in_proj_b", "in_proj_a"))
    else:
        raise KeyError(f"{prefix}: neither in_proj_qkvz nor in_proj_qkv found")
    cq, ck, cv = torch.split(src[prefix + "conv1d.weight"], [Hk * dk, Hk * dk, Hv * dv], dim=0)
    return dict(q=q, k=k, v=v, z=z, b=b, a=a, cq=cq, ck=ck, cv=cv, A_log=src[prefix + "A_log"],
                dt_bias=src[prefix + "dt_bias"], norm=src[prefix + "norm.weight"], out=src[prefix + "out_proj.weight"])


def linear_attn_to_mixer(w: Dict[str, torch.Tensor], prefix_out: str, target: str) -> Dict[str, torch.Tensor]:
    """Tensors of one hybrid mixer (``target`` = ``GDN`` or ``GKA``) from an extracted ``linear_attn`` block."""
    out = {prefix_out + "q_proj.weight": w["q"], prefix_out + "k_proj.weight": w["k"], prefix_out + "v_proj.weight": w["v"],
           prefix_out + "g_proj.weight": w["z"], prefix_out + "q_conv1d.weight": w["cq"],
           prefix_out + "k_conv1d.weight": w["ck"], prefix_out + "v_conv1d.weight": w["cv"],
           prefix_out + "o_proj.weight": w["out"], prefix_out + "o_norm.weight": w["norm"],
           prefix_out + "A_log": w["A_log"], prefix_out + "dt_bias": w["dt_bias"], prefix_out + "b_proj.weight": w["b"]}
    if target == "GDN":
        out[prefix_out + "gk_proj.weight"] = w["a"]
    elif target == "GKA":
        out[prefix_out + "a_proj.weight"] = w["a"]
    else:
        raise ValueError(f"a linear_attention layer converts to GDN or GKA, not {target!r}")
    return {k: v.clone() for k, v in out.items()}


_LAYER = re.compile(r"^(model\.(?:language_model\.)?layers\.(\d+)\.)(.*)$")
_VISION = ("model.visual.", "visual.", "model.vision_tower.", "vision_tower.")


def default_pattern(layer_types) -> str:
    """``["linear_attention", "full_attention", ...]`` -> ``"GDN-GDN-GDN-*-..."``."""
    return "-".join("*" if t == "full_attention" else "GDN" for t in layer_types)


def pattern_from_layer_types(layer_types, targets: Dict[int, str] = None) -> str:
    targets = targets or {}
    sym = {"gdn": "GDN", "gka": "GKA"}
    return "-".join("*" if t == "full_attention" and i not in targets else sym.get(targets.get(i, "gdn"), "GDN")
                    for i, t in enumerate(layer_types))


def convert_state_dict(src: Dict[str, torch.Tensor], config, pattern: Optional[str] = None, keep_vision: bool = False,
                       attention_targets: Optional[dict] = None) -> Tuple[Dict[str, torch.Tensor], dict]:
    """Whole checkpoint.  ``config`` supplies ``layer_types``, ``linear_num_key_heads``, ``linear_num_value_heads``,
    ``linear_key_head_dim``, ``linear_value_head_dim``, ``num_attention_heads``, ``head_dim``.  ``pattern`` is the
    target ``hybrid_override_pattern`` (default: GDN where the source is linear attention, ``*`` elsewhere).
    ``attention_targets[layer]`` is the freshly built target mixer module of a ``full_attention`` layer that becomes
    an SSM (the stage-0 rules write into modules).  Returns ``(tensors, report)``; ``report`` lists dropped keys
    and, per layer, which conversion ran."""
    Hk, Hv = config.linear_num_key_heads, config.linear_num_value_heads
    dk, dv = config.linear_key_head_dim, config.linear_value_head_dim
    layer_types = list(config.layer_types)
    symbols = parse_override_pattern(pattern or default_pattern(layer_types))
    if len(symbols) != len(layer_types):
        raise ValueError(f"pattern has {len(symbols)} symbols, the source model {len(layer_types)} layers")
    out: Dict[str, torch.Tensor] = {}
    report = {"dropped": [], "layers": {}, "fresh": []}
    done = set()
    for name, t in src.items():
        if name.startswith("mtp.") or ".mtp." in name:
            report["dropped"].append(name)
            continue
        if name.startswith(_VISION):
            if keep_vision:
                out[name] = t
            else:
                report["dropped"].append(name)
            continue
        m = _LAYER.match(name)
        if not m:
            out[name.replace("model.language_model.", "model.")] = t
            continue
        layer = int(m.group(2))
        base_in, rest = m.group(1), m.group(3)
        base_out = f"model.layers.{layer}."
        sym = symbols[layer]
        source = "linear" if layer_types[layer] != "full_attention" else "full"
        if rest.startswith("linear_attn."):
            if source != "linear":
                raise ValueError(f"layer {layer}: linear_attn tensors in a layer typed {layer_types[layer]}")
            if layer in done:
                continue
            done.add(layer)
            w = extract_linear_attn(base_in + "linear_attn.", src, Hk, Hv, dk, dv)
            targets = ["GDN", "GKA"] if sym == "GDN>GKA" else [unfuse_symbol(sym)]
            for tg in targets:
                out.update(linear_attn_to_mixer(w, base_out + MIXER_ATTR[tg] + ".", tg))
                if (source, tg) in FRESH_OK:
                    report["fresh"] += [base_out + MIXER_ATTR[tg] + "." + p for p in FRESH_OK[(source, tg)]]
            report["layers"][layer] = f"linear_attention -> {sym}"
        elif rest.startswith("self_attn."):
            tg = unfuse_symbol(sym)
            if tg == "*":
                out[base_out + rest] = t
                report["layers"][layer] = "full_attention -> *"
                if sym != "*":           # fused X* layer: student X initialised from this attention as well
                    raise ValueError(f"layer {layer}: pattern symbol {sym!r} is not a valid target for attention")
                continue
            if layer in done:
                continue
            done.add(layer)
            if attention_targets is None or layer not in attention_targets:
                raise ValueError(f"layer {layer}: full_attention -> {tg} needs the target mixer module "
                                 f"(attention_targets[{layer}]) for the stage-0 initialisation rules")
            out.update(_attention_to_ssm(src, base_in + "self_attn.", base_out + MIXER_ATTR[tg] + ".", tg,
                                         attention_targets[layer], layer, config))
            report["fresh"] += [base_out + MIXER_ATTR[tg] + "." + p for p in FRESH_OK[(source, tg)]]
            report["layers"][layer] = f"full_attention -> {tg}"
        else:
            out[base_out + rest] = t
    return out, report


def _attention_to_ssm(src, prefix_in: str, prefix_out: str, target: str, mixer, layer: int, config) -> Dict[str, torch.Tensor]:
    """Stage-0 rules on a (gated) attention layer: the query rows are the first ``head_dim`` rows of every per-head
    ``[q | gate]`` block of ``q_proj`` (reference: ``convert_qwen_gdn_models.py:411-487``)."""
    from .hybrid_layer_init import AttentionWeights, init_mixer
    H = config.num_attention_heads
    D = getattr(config, "head_dim", None) or config.hidden_size // H
    qw = src[prefix_in + "q_proj.weight"].float()
    if qw.shape[0] == 2 * H * D:
        qw = qw.view(H, 2 * D, -1)[:, :D].reshape(H * D, -1)
    attn = AttentionWeights(qw, src[prefix_in + "k_proj.weight"].float(), src[prefix_in + "v_proj.weight"].float(),
                            src[prefix_in + "o_proj.weight"].float())
    init_mixer(target, attn, mixer, layer)
    return {prefix_out + k: v.detach().clone() for k, v in mixer.state_dict().items()}


def target_config_dict(src_cfg: dict, pattern: str, text_only: bool = True) -> dict:
    """``config.json`` of the converted model: the source's text configuration under this framework's model type,
    with the target pattern."""
    cfg = dict(src_cfg.get("text_config", src_cfg)) if text_only else dict(src_cfg)
    src_type = str(src_cfg.get("model_type", ""))
    cfg["model_type"] = "qwen3_5_moe_hmf_text" if "qwen3_5" in src_type else "qwen3_next_hmf"
    cfg["hybrid_override_pattern"] = pattern
    cfg.pop("architectures", None)
    cfg.pop("quantization_config", None)
    return cfg


def convert_checkpoint(src_dir: str, out_dir: str, pattern: Optional[str] = None, keep_vision: bool = False,
                       dtype: Optional[torch.dtype] = None, max_shard_size="5GB") -> dict:
    """Reads a Qwen3-Next / Qwen3.5-MoE checkpoint directory, converts it, checks that the result fills the target
    model, and writes ``out_dir`` (safetensors shards + ``config.json``).  Returns the conversion report."""
    from types import SimpleNamespace

    from ..models.configuration import HybridConfig
    from ..models.modeling_hybrid import build_model
    from ..utils import checkpoint_io
    with open(os.path.join(src_dir, "config.json")) as f:
        src_cfg = json.load(f)
    text = src_cfg.get("text_config", src_cfg)
    ns = SimpleNamespace(**text)
    pattern = pattern or default_pattern(ns.layer_types)
    cfg = HybridConfig.from_dict(target_config_dict(src_cfg, pattern))
    model = build_model(cfg)
    if dtype is not None:
        model = model.to(dtype)
    src = dict(checkpoint_io.iter_tensors(src_dir))
    symbols = parse_override_pattern(pattern)
    attention_targets = {i: model.model.layers[i].seq_mixer for i, t in enumerate(ns.layer_types)
                         if t == "full_attention" and unfuse_symbol(symbols[i]) != "*"}
    tensors, report = convert_state_dict(src, ns, pattern, keep_vision, attention_targets)
    report["missing"], report["unexpected"] = load_converted(model, tensors, report["fresh"])
    checkpoint_io.save_pretrained(model, out_dir, max_shard_size=max_shard_size)
    with open(os.path.join(out_dir, "conversion_report.json"), "w") as f:
        json.dump({k: (v if not isinstance(v, dict) else {str(a): b for a, b in v.items()}) for k, v in report.items()},
                  f, indent=1)
    return report


def load_converted(model: torch.nn.Module, tensors: Dict[str, torch.Tensor], fresh_ok: List[str]) -> Tuple[list, list]:
    """Strict load of converted tensors: a model parameter without a tensor must be on the fresh-initialisation list,
    and every tensor must have a parameter.  Raises ``KeyError`` otherwise."""
    from ..utils import checkpoint_io
    state = checkpoint_io.from_hf_names(tensors)
    own = dict(model.state_dict(keep_vars=True))
    missing = [k for k in own if k not in state]
    if getattr(model.config, "tie_word_embeddings", False) and "lm_head.weight" in missing:
        missing.remove("lm_head.weight")
    bad = [k for k in missing if not any(k.startswith(p) for p in fresh_ok)]
    unexpected = [k for k in state if k not in own]
    if bad or unexpected:
        raise KeyError(f"conversion does not fill the target model: parameters without a source {bad[:8]}, "
                       f"tensors without a parameter {unexpected[:8]}")
    with torch.no_grad():
        for k, t in state.items():
            if own[k].shape != t.shape:
                raise ValueError(f"shape mismatch for {k}: converted {tuple(t.shape)} vs model {tuple(own[k].shape)}")
            own[k].data.copy_(t.to(own[k].dtype))
    return missing, unexpected


def main(argv=None) -> int:
    import argparse
    ap = argparse.ArgumentParser(prog="hmf convert-qwen-gdn", description=__doc__.split("\n\n")[0])
    ap.add_argument("source", help="directory of the Qwen3-Next / Qwen3.5-MoE checkpoint (config.json + safetensors)")
    ap.add_argument("output")
    ap.add_argument("--pattern", default=None, help="target hybrid_override_pattern (default: GDN / * as in the source)")
    ap.add_argument("--keep-vision", action="store_true")
    ap.add_argument("--dtype", default="bfloat16")
    a = ap.parse_args(argv)
    rep = convert_checkpoint(a.source, a.output, a.pattern, a.keep_vision, getattr(torch, a.dtype))
    print(json.dumps({"layers": {str(k): v for k, v in rep["layers"].items()}, "dropped": len(rep["dropped"]),
                      "fresh": len(rep["missing"])}))
    return 0
