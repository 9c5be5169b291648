"""Converters from released Qwen models that already contain Gated DeltaNet layers (Qwen3-Next, Qwen3.5) to this
framework's layout.

Those checkpoints store the linear-attention projections fused and *interleaved per key head*:
``in_proj_qkvz [Hk * (2 dk + 2 r dv), hidden]`` with per-head blocks ``[q (dk) | k (dk) | v (r dv) | z (r dv)]``
(``r = Hv / Hk`` value heads per key head) and ``in_proj_ba [Hk * 2 r, hidden]`` with blocks ``[b (r) | a (r)]``;
the depthwise convolution runs over ``[q | k | v]`` channels.  The hybrid layer keeps separate ``q/k/v/g/b/gk``
projections and one convolution per stream, so the converter de-interleaves rows and splits the convolution.
Targets: GDN -> GDN (exact), GDN -> GKA (shared projections copied, the rest freshly initialised), and the
attention layers stay attention (gated attention and zero-centred norms are config switches of the same layer).
Reference: ``convert_qwen_gdn_models.py:57-1009``, ``convert_qwen3_next.py:31-248``, ``convert_qwen3_5_moe.py:33-204``.
"""
from __future__ import annotations

import re
from typing import Dict, Tuple

import torch


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
    """Inverse of :func:`deinterleave_qkvz` (used by the round-trip test and by export)."""
    r = Hv // Hk
    parts = [q.view(Hk, dk, -1), k.view(Hk, dk, -1), v.view(Hk, r * dv, -1), z.view(Hk, r * dv, -1)]
    return torch.cat(parts, dim=1).reshape(Hk * (2 * dk + 2 * r * dv), -1)


def convert_linear_attn(prefix_in: str, prefix_out: str, src: Dict[str, torch.Tensor], Hk: int, Hv: int, dk: int,
                        dv: int, target: str = "gdn") -> Dict[str, torch.Tensor]:
    """One ``linear_attn`` block -> one hybrid mixer (``gdn`` or ``gka``)."""
    out: Dict[str, torch.Tensor] = {}
    q, k, v, z = deinterleave_qkvz(src[prefix_in + "in_proj_qkvz.weight"], Hk, Hv, dk, dv)
    b, a = deinterleave_ba(src[prefix_in + "in_proj_ba.weight"], Hk, Hv)
    conv = src[prefix_in + "conv1d.weight"]                       # [2 Hk dk + Hv dv, 1, K]
    cq, ck, cv = torch.split(conv, [Hk * dk, Hk * dk, Hv * dv], dim=0)
    out.update({prefix_out + "q_proj.weight": q, prefix_out + "k_proj.weight": k, prefix_out + "v_proj.weight": v,
                prefix_out + "g_proj.weight": z, prefix_out + "q_conv1d.weight": cq, prefix_out + "k_conv1d.weight": ck,
                prefix_out + "o_proj.weight": src[prefix_in + "out_proj.weight"],
                prefix_out + "o_norm.weight": src[prefix_in + "norm.weight"]})
    if target == "gdn":
        out.update({prefix_out + "v_conv1d.weight": cv, prefix_out + "b_proj.weight": b,
                    prefix_out + "gk_proj.weight": a, prefix_out + "A_log": src[prefix_in + "A_log"],
                    prefix_out + "dt_bias": src[prefix_in + "dt_bias"]})
    elif target == "gka":
        # shared: q/k/v/g/o, q/k convolutions, decay parameters; GKA-only parameters keep their fresh init
        out.update({prefix_out + "v_conv1d.weight": cv, prefix_out + "a_proj.weight": a,
                    prefix_out + "A_log": src[prefix_in + "A_log"], prefix_out + "dt_bias": src[prefix_in + "dt_bias"]})
    else:
        raise ValueError(f"unknown target mixer {target!r}")
    return out


_LAYER = re.compile(r"^(model\.layers\.(\d+)\.)(.*)$")


def convert_state_dict(src: Dict[str, torch.Tensor], config, targets: Dict[int, str] = None) -> Dict[str, torch.Tensor]:
    """Whole checkpoint.  ``config`` supplies ``linear_num_key_heads``, ``linear_num_value_heads``,
    ``linear_key_head_dim``, ``linear_value_head_dim``; ``targets[layer] in {"gdn", "gka"}`` (default gdn)."""
    Hk, Hv = config.linear_num_key_heads, config.linear_num_value_heads
    dk, dv = config.linear_key_head_dim, config.linear_value_head_dim
    targets = targets or {}
    out: Dict[str, torch.Tensor] = {}
    done = set()
    for name, t in src.items():
        m = _LAYER.match(name)
        if m and m.group(3).startswith("linear_attn."):
            layer = int(m.group(2))
            if layer not in done:
                done.add(layer)
                out.update(convert_linear_attn(m.group(1) + "linear_attn.", m.group(1) + "seq_mixer.", src, Hk, Hv,
                                               dk, dv, targets.get(layer, "gdn")))
            continue
        if m and m.group(3).startswith("self_attn."):
            out[m.group(1) + "seq_mixer." + m.group(3)[len("self_attn."):]] = t
            continue
        out[name] = t
    return out


def pattern_from_layer_types(layer_types, targets: Dict[int, str] = None) -> str:
    """``["linear_attention", "full_attention", ...]`` -> ``"GDN-GDN-GDN-*-..."``."""
    targets = targets or {}
    sym = {"gdn": "GDN", "gka": "GKA"}
    return "-".join("*" if t == "full_attention" else sym[targets.get(i, "gdn")] for i, t in enumerate(layer_types))
