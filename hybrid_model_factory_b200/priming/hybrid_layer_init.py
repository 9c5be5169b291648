"""Stage-0 weight surgery: initialise hybrid mixers from the attention weights they replace.

Rules (reference: ``priming/hybrid_layer_init.py:354-705``):
  * ``q/k/v/o_proj`` are copied (GDN, GKA; B'MOJO attention and SWA copy all four as well);
  * the output gate ``g_proj`` (GDN / GKA) and Mamba2's ``z`` block are set to
    ``0.5 * (W_o^T + repeat_interleave(W_v, Hq / Hkv, dim=0))``;
  * Mamba2 ``in_proj`` rows are laid out ``[z, x(=v), B(=k), C(=q), dt]``; ``out_proj = W_o``;
    ``B_norm <- k_norm``, ``C_norm <- q_norm``;
  * everything else (convolutions, gates' small projections, ``A_log``, ``dt_bias``) keeps its
    random initialisation.
Every rule logs the weight sums before / after as a sanity signal.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, Optional

import torch

from ..utils.logging import get_logger

logger = get_logger(__name__)


@dataclass
class AttentionWeights:
    q_weight: torch.Tensor
    k_weight: torch.Tensor
    v_weight: torch.Tensor
    o_weight: torch.Tensor
    q_bias: Optional[torch.Tensor] = None
    k_bias: Optional[torch.Tensor] = None
    v_bias: Optional[torch.Tensor] = None
    o_bias: Optional[torch.Tensor] = None
    q_norm: Optional[torch.Tensor] = None
    k_norm: Optional[torch.Tensor] = None


def extract_attention_weights(state: Dict[str, torch.Tensor], layer_idx: int, prefix: str = "model.layers") -> AttentionWeights:
    base = f"{prefix}.{layer_idx}.self_attn"

    def get(name):
        t = state.get(f"{base}.{name}")
        return None if t is None else t.float()

    w = AttentionWeights(get("q_proj.weight"), get("k_proj.weight"), get("v_proj.weight"), get("o_proj.weight"),
                         get("q_proj.bias"), get("k_proj.bias"), get("v_proj.bias"), get("o_proj.bias"),
                         get("q_norm.weight"), get("k_norm.weight"))
    if w.q_weight is None or w.o_weight is None:
        raise KeyError(f"attention weights of layer {layer_idx} not found under '{base}'")
    return w


def _copy(dst: torch.nn.Parameter, src: Optional[torch.Tensor], what: str, layer_idx: int) -> None:
    if src is None or dst is None:
        return
    if tuple(dst.shape) != tuple(src.shape):
        raise ValueError(f"layer {layer_idx}: cannot copy {what}: shape {tuple(src.shape)} into {tuple(dst.shape)}")
    before = dst.data.float().sum().item()
    dst.data.copy_(src.to(dst.dtype))
    logger.debug("layer %d %s: sum %.6f -> %.6f", layer_idx, what, before, dst.data.float().sum().item())


def gate_from_output_and_value(attn: AttentionWeights, rows: int) -> torch.Tensor:
    """``0.5 * (W_o^T + repeat_interleave(W_v, rows / W_v.rows, dim=0))``."""
    groups = rows // attn.v_weight.shape[0]
    return 0.5 * (attn.o_weight.t() + attn.v_weight.repeat_interleave(groups, dim=0))


def _copy_qkvo(attn: AttentionWeights, layer, layer_idx: int, names=("q_proj", "k_proj", "v_proj", "o_proj")) -> None:
    for n, wname, bname in zip(names, ("q_weight", "k_weight", "v_weight", "o_weight"),
                               ("q_bias", "k_bias", "v_bias", "o_bias")):
        proj = getattr(layer, n)
        _copy(proj.weight, getattr(attn, wname), n, layer_idx)
        if getattr(proj, "bias", None) is not None:
            _copy(proj.bias, getattr(attn, bname), n + ".bias", layer_idx)


def gated_deltanet_proj_init(attn: AttentionWeights, layer, layer_idx: int) -> None:
    _copy_qkvo(attn, layer, layer_idx)
    if getattr(layer, "use_gate", False):
        _copy(layer.g_proj.weight, gate_from_output_and_value(attn, layer.g_proj.weight.shape[0]), "g_proj", layer_idx)
    logger.info("layer %d: Gated DeltaNet initialised from attention", layer_idx)


def gka_proj_init(attn: AttentionWeights, layer, layer_idx: int) -> None:
    _copy_qkvo(attn, layer, layer_idx)
    if getattr(layer, "use_gate", False):
        _copy(layer.g_proj.weight, gate_from_output_and_value(attn, layer.g_proj.weight.shape[0]), "g_proj", layer_idx)
    logger.info("layer %d: Gated KalmaNet initialised from attention", layer_idx)


def mamba2_init(attn: AttentionWeights, layer, layer_idx: int) -> None:
    d_inner, d_xb = layer.d_inner, layer.d_xb
    _copy(layer.out_proj.weight, attn.o_weight, "out_proj", layer_idx)
    w = layer.in_proj.weight.data
    before = w.float().sum().item()
    w[d_inner:d_inner + d_xb].copy_(attn.v_weight.to(w.dtype))
    w[d_inner + d_xb:d_inner + 2 * d_xb].copy_(attn.k_weight.to(w.dtype))
    w[d_inner + 2 * d_xb:2 * d_inner + 2 * d_xb].copy_(attn.q_weight.to(w.dtype))
    w[:d_inner].copy_(gate_from_output_and_value(attn, d_inner).to(w.dtype))
    logger.info("layer %d: Mamba2 in_proj sum %.6f -> %.6f", layer_idx, before, w.float().sum().item())
    if attn.k_norm is not None and layer.B_norm is not None:
        _copy(layer.B_norm.weight, attn.k_norm, "B_norm", layer_idx)
        _copy(layer.C_norm.weight, attn.q_norm, "C_norm", layer_idx)


def attention_like_init(attn: AttentionWeights, layer, layer_idx: int) -> None:
    """SWA and B'MOJO attention: same projections (and q/k norms) as the source attention; untied
    fading-stream projections start as copies too."""
    _copy_qkvo(attn, layer, layer_idx)
    if getattr(layer, "q_norm", None) is not None and attn.q_norm is not None:
        _copy(layer.q_norm.weight, attn.q_norm, "q_norm", layer_idx)
        _copy(layer.k_norm.weight, attn.k_norm, "k_norm", layer_idx)
    if hasattr(layer, "q_proj_"):
        _copy_qkvo(attn, layer, layer_idx, names=("q_proj_", "k_proj_", "v_proj_", "o_proj"))
        if getattr(layer, "q_norm_", None) is not None and attn.q_norm is not None:
            _copy(layer.q_norm_.weight, attn.q_norm, "q_norm_", layer_idx)
            _copy(layer.k_norm_.weight, attn.k_norm, "k_norm_", layer_idx)


def init_mixer(symbol: str, attn: AttentionWeights, mixer, layer_idx: int) -> None:
    """Dispatch on the (unfused) layer symbol."""
    if symbol == "GDN":
        gated_deltanet_proj_init(attn, mixer, layer_idx)
    elif symbol == "GKA":
        gka_proj_init(attn, mixer, layer_idx)
    elif symbol == "M2":
        mamba2_init(attn, mixer, layer_idx)
    elif symbol == "SWA":
        attention_like_init(attn, mixer, layer_idx)
    elif symbol == "BMF":
        attention_like_init(attn, mixer.bmojo_attn, layer_idx)
        inner = mixer.ssm_mixer_type
        sub = {"mamba2": "M2", "gdn": "GDN", "gated_deltanet": "GDN", "gka": "GKA", "gated_kalmanet": "GKA"}[inner]
        init_mixer(sub, attn, mixer.ssm_mixer, layer_idx)
    elif symbol == "*":
        attention_like_init(attn, mixer, layer_idx)
    elif symbol == "L2A":
        attention_like_init(attn, mixer.local, layer_idx)
        attention_like_init(attn, mixer.global_attn, layer_idx)
    else:
        raise ValueError(f"no stage-0 initialisation rule for layer symbol '{symbol}'")
