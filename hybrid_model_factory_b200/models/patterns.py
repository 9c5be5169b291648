"""``hybrid_override_pattern`` grammar: a dash-separated list with one symbol per decoder layer.

    *      softmax attention          M2     Mamba2            GDN   Gated DeltaNet
    GKA    Gated KalmaNet             BMF    B'MOJO-F          SWA   sliding-window attention
    M2* GDN* GKA* BMF* SWA*   fused stage-1 layers (student mixer + frozen attention teacher)
    *DA    dual-path attention (same weights on student and teacher streams)
    GDN>GKA  fused SSM->SSM layer (GDN teacher, GKA student)
    L2A    sliding-window attention + routed global attention (research example)

Reference: ``models/utils.py:6-154`` and ``priming/fused_to_standard.py:142-164``.
"""
from __future__ import annotations

from typing import Dict, List

LAYER_SYMBOLS = ["*", "M2", "BMF", "GDN", "GKA", "SWA", "M2*", "BMF*", "GDN*", "GKA*", "SWA*", "GDN>GKA", "*DA", "L2A"]

FUSED_SYMBOLS = {"M2*": "M2", "BMF*": "BMF", "GDN*": "GDN", "GKA*": "GKA", "SWA*": "SWA", "GDN>GKA": "GKA", "*DA": "*"}

# attribute name of the sequence mixer inside a decoder layer, per (unfused) symbol
MIXER_ATTR = {"*": "self_attn", "M2": "mamba", "BMF": "bmojo_f", "GDN": "gdn", "GKA": "gka", "SWA": "swa", "L2A": "l2a"}

LAYER_TYPE_NAMES = {"*": "full_attention", "SWA": "sliding_attention", "M2": "mamba2", "GDN": "linear_attention",
                    "GKA": "gated_kalmanet", "BMF": "bmojo_f", "L2A": "l2a_attention"}


def parse_override_pattern(pattern: str) -> Dict[int, str]:
    """``"*-GDN-*"`` -> ``{0: "*", 1: "GDN", 2: "*"}``; unknown symbols raise."""
    parts = pattern.split("-")
    for i, s in enumerate(parts):
        if s not in LAYER_SYMBOLS:
            raise ValueError(f"unknown layer symbol '{s}' at position {i}; valid symbols: {LAYER_SYMBOLS}")
    return {i: s for i, s in enumerate(parts)}


def is_fused(symbol: str) -> bool:
    return symbol in FUSED_SYMBOLS


def unfuse_symbol(symbol: str) -> str:
    """``X* -> X``, ``*DA -> *``, ``A>B -> B``; plain symbols are returned unchanged."""
    return FUSED_SYMBOLS.get(symbol, symbol)


def unfuse_pattern(pattern: str) -> str:
    p = parse_override_pattern(pattern)
    return "-".join(unfuse_symbol(p[i]) for i in range(len(p)))


def pattern_to_layer_types(pattern: str) -> List[str]:
    p = parse_override_pattern(pattern)
    return [LAYER_TYPE_NAMES[unfuse_symbol(p[i])] for i in range(len(p))]


def expand_pattern_for_layers(pattern: str, num_layers: int) -> str:
    """Repeats a short pattern (e.g. ``"*-GDN"``) until it covers ``num_layers`` layers."""
    parts = pattern.split("-")
    if len(parts) == num_layers:
        return pattern
    if num_layers % len(parts) != 0:
        raise ValueError(f"pattern of {len(parts)} symbols does not tile {num_layers} layers")
    return "-".join(parts * (num_layers // len(parts)))


def count_symbols(pattern: str) -> Dict[str, int]:
    out: Dict[str, int] = {}
    for s in pattern.split("-"):
        out[s] = out.get(s, 0) + 1
    return out
