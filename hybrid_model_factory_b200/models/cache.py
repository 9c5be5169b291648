"""Inference cache for hybrid models (HF-style ``past_key_values`` object).

Per layer it holds whichever state that layer type needs:
  * attention: concatenated K/V ``[B, T, Hkv, D]`` (optionally truncated to a window);
  * SSM mixers: ``{"recurrent_state": ..., "conv_state": ...}`` where the recurrent state is
    ``[B,H,Dk,Dv]`` (GDN), ``(h_kk, h_kv)`` (GKA) or ``[B,H,P,N]`` (Mamba2) in fp32 and the conv
    state keeps the last ``K-1`` pre-convolution inputs; Mamba2 also accumulates the log of its
    cumulative decay (``log_aprod``) for state composition;
  * B'MOJO: the last ``2w-1`` keys/values of both streams with their positions.
A global ``seqlen_offset`` counts tokens already consumed.
Reference: ``models/cache.py:18-414``.
"""
from __future__ import annotations

import copy as _copy
from typing import Dict, Optional, Tuple

import torch


class HybridCache:
    def __init__(self, cache_aprods: bool = True):
        self.attention: Dict[int, Tuple[torch.Tensor, torch.Tensor]] = {}
        self.ssm: Dict[int, dict] = {}
        self.bmojo: Dict[int, dict] = {}
        self.seqlen_offset = 0
        self.cache_aprods = cache_aprods
        self.cache_transitions = False      # Gated DeltaNet layers also store the chunk's transition matrix

    # -- attention ------------------------------------------------------------------
    def update_attention(self, layer_idx: int, k: torch.Tensor, v: torch.Tensor, window: Optional[int] = None):
        if layer_idx in self.attention:
            pk, pv = self.attention[layer_idx]
            k, v = torch.cat([pk, k], dim=1), torch.cat([pv, v], dim=1)
        if window is not None and k.shape[1] > window:
            keep_k, keep_v = k[:, -window:], v[:, -window:]
        else:
            keep_k, keep_v = k, v
        self.attention[layer_idx] = (keep_k, keep_v)
        return k, v

    # -- SSM ----------------------------------------------------------------------------
    def get_ssm(self, layer_idx: int) -> Optional[dict]:
        return self.ssm.get(layer_idx)

    def update_ssm(self, layer_idx: int, recurrent_state=None, conv_state=None, offset: int = 0, log_aprod=None,
                   transition=None):
        entry = self.ssm.setdefault(layer_idx, {"recurrent_state": None, "conv_state": None, "log_aprod": None})
        if transition is not None:     # S_out = transition @ S_in + ...; later segments multiply from the left
            entry["transition"] = transition if entry.get("transition") is None else transition @ entry["transition"]
        if recurrent_state is not None:
            entry["recurrent_state"] = recurrent_state
        if conv_state is not None:
            entry["conv_state"] = conv_state
        if log_aprod is not None and self.cache_aprods:
            entry["log_aprod"] = log_aprod if entry["log_aprod"] is None else entry["log_aprod"] + log_aprod

    # -- B'MOJO -------------------------------------------------------------------------
    def update_bmojo(self, layer_idx: int, k_s, v_s, k_c, v_c, positions, keep: int):
        e = self.bmojo.get(layer_idx)
        if e is not None:
            k_s, v_s = torch.cat([e["k_s"], k_s], 1), torch.cat([e["v_s"], v_s], 1)
            k_c, v_c = torch.cat([e["k_c"], k_c], 1), torch.cat([e["v_c"], v_c], 1)
            k_pos = torch.cat([e["pos"], positions], 1)
        else:
            k_pos = positions
        self.bmojo[layer_idx] = {"k_s": k_s[:, -keep:], "v_s": v_s[:, -keep:], "k_c": k_c[:, -keep:],
                                 "v_c": v_c[:, -keep:], "pos": k_pos[:, -keep:]}
        return k_s, v_s, k_c, v_c, k_pos

    # -- housekeeping ---------------------------------------------------------------------
    def get_seq_length(self, layer_idx: int = 0) -> int:
        return self.seqlen_offset

    def update_offset(self, n: int) -> None:
        self.seqlen_offset += n

    def copy(self, share_attention: bool = False) -> "HybridCache":
        new = HybridCache(self.cache_aprods)
        clone = lambda t: t.clone() if isinstance(t, torch.Tensor) else (  # noqa: E731
            tuple(clone(x) for x in t) if isinstance(t, tuple) else _copy.copy(t))
        if share_attention:
            new.attention = dict(self.attention)
        else:
            new.attention = {i: (k.clone(), v.clone()) for i, (k, v) in self.attention.items()}
        new.ssm = {i: {n: clone(s) for n, s in e.items()} for i, e in self.ssm.items()}
        new.bmojo = {i: {n: clone(s) for n, s in e.items()} for i, e in self.bmojo.items()}
        new.seqlen_offset = self.seqlen_offset
        new.cache_transitions = self.cache_transitions
        return new

    def snapshot(self) -> "HybridCache":
        """A cache that stays at this position while the original moves on.  Attention keys / values are replaced, not
        written in place, when tokens are appended, so they are shared; the (small) recurrent entries are cloned."""
        return self.copy(share_attention=True)

    def clear(self) -> None:
        self.attention.clear()
        self.ssm.clear()
        self.bmojo.clear()
        self.seqlen_offset = 0

    def state_bytes(self) -> int:
        def nbytes(t):
            if isinstance(t, torch.Tensor):
                return t.numel() * t.element_size()
            if isinstance(t, (tuple, list)):
                return sum(nbytes(x) for x in t)
            if isinstance(t, dict):
                return sum(nbytes(x) for x in t.values())
            return 0
        return nbytes(self.attention) + nbytes(self.ssm) + nbytes(self.bmojo)
