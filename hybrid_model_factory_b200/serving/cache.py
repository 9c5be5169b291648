"""Device-side serving state: paged K/V for attention layers and fixed-size slots for recurrent layers.

* attention / SWA layers: ``k_cache, v_cache [num_blocks, block_size, Hkv, D]`` (bf16), addressed through
  per-request block tables from the native block manager;
* GDN / GKA / Mamba2 layers: recurrent state ``[num_slots + num_snapshots, ...]`` in **fp32** (the
  reference serves with ``--mamba-ssm-cache-dtype float32``; GKA's ``h_kk`` must be fp32,
  ``primed_gka_layer.py:423-430``) and the convolution window ``[slots, K-1, C]`` over the concatenated
  conv channels.

``SlotCache`` adapts one scheduled request to the ``past_key_values`` protocol of the layers
(``models/cache.py``), so chunked prefill reuses the training-path kernels with the slot's state as the
initial state; the batched decode path indexes the same tensors directly with slot ids.
"""
from __future__ import annotations

from typing import Dict, List, Optional, Tuple

import torch

from ..layers.attention import Attention
from ..layers.bmojo import BMojoLayer
from ..layers.gdn import GatedDeltaNet
from ..layers.gka import GatedKalmaNet
from ..layers.mamba2 import Mamba2


class ServingState:
    def __init__(self, model, num_blocks: int, block_size: int, num_slots: int, num_snapshots: int = 0,
                 device=None, dtype=torch.bfloat16):
        self.block_size, self.num_blocks, self.num_slots = block_size, num_blocks, num_slots
        self.device = device or next(model.parameters()).device
        self.kv: Dict[int, Tuple[torch.Tensor, torch.Tensor]] = {}
        self.ssm: Dict[int, dict] = {}
        # B'MOJO-F layers keep a bounded per-request state (SSM state + the last 2w-1 keys / values of both
        # streams); it lives in one small ``HybridCache`` per request instead of the paged pools
        self.bmojo_layers = set()
        self.side: Dict[int, object] = {}
        total_slots = num_slots + num_snapshots
        for i, layer in enumerate(model.model.layers):
            mixer = layer.seq_mixer
            if isinstance(mixer, Attention):
                shape = (num_blocks, block_size, mixer.num_kv_heads, mixer.head_dim)
                self.kv[i] = (torch.zeros(shape, device=self.device, dtype=dtype),
                              torch.zeros(shape, device=self.device, dtype=dtype))
            elif isinstance(mixer, GatedDeltaNet):
                H, D = mixer.expanded_num_heads, mixer.head_dim
                C = mixer.query_dim + mixer.key_dim + mixer.value_dim
                self.ssm[i] = {"kind": "gdn", "state": torch.zeros(total_slots, H, D, D, device=self.device),
                               "conv": torch.zeros(total_slots, mixer.conv_size - 1, C, device=self.device, dtype=dtype),
                               "split": [mixer.query_dim, mixer.key_dim, mixer.value_dim]}
            elif isinstance(mixer, GatedKalmaNet):
                H, D = mixer.expanded_num_heads, mixer.head_dim
                split = [mixer.query_dim, mixer.key_dim] + ([mixer.value_dim] if mixer.use_v_conv else [])
                self.ssm[i] = {"kind": "gka", "state": torch.zeros(total_slots, H, D, D, device=self.device),
                               "state_kk": torch.zeros(total_slots, H, D, D, device=self.device),
                               "conv": torch.zeros(total_slots, mixer.conv_size - 1, sum(split), device=self.device,
                                                   dtype=dtype), "split": split}
            elif isinstance(mixer, Mamba2):
                self.ssm[i] = {"kind": "mamba2",
                               "state": torch.zeros(total_slots, mixer.nheads, mixer.headdim, mixer.d_state,
                                                    device=self.device),
                               "conv": torch.zeros(total_slots, mixer.d_conv - 1, mixer.conv_dim, device=self.device,
                                                   dtype=dtype), "split": None}
            elif isinstance(mixer, BMojoLayer):
                self.bmojo_layers.add(i)
            else:
                raise NotImplementedError(f"layer {i} ({type(mixer).__name__}) is not supported by the paged engine")

    def bytes(self) -> int:
        n = sum(k.numel() * k.element_size() * 2 for k, _ in self.kv.values())
        for e in self.ssm.values():
            n += sum(t.numel() * t.element_size() for t in e.values() if isinstance(t, torch.Tensor))
        return n

    def side_cache(self, req_id: int):
        from ..models.cache import HybridCache
        c = self.side.get(req_id)
        if c is None:
            c = self.side[req_id] = HybridCache()
        return c

    def copy_slot(self, src: int, dst: int) -> None:
        """Snapshot / restore of the recurrent state (align-mode prefix caching)."""
        for e in self.ssm.values():
            for key in ("state", "state_kk", "conv"):
                if key in e:
                    e[key][dst].copy_(e[key][src])

    def clear_slot(self, slot: int) -> None:
        for e in self.ssm.values():
            for key in ("state", "state_kk", "conv"):
                if key in e:
                    e[key][slot].zero_()


class SlotCache:
    """``past_key_values`` adapter for one request during (chunked) prefill."""

    def __init__(self, state: ServingState, slot: int, block_table: List[int], start_pos: int, side=None):
        self.s, self.slot, self.start = state, slot, start_pos
        self.side = side          # per-request HybridCache for B'MOJO-F layers
        self.block_table = torch.tensor(block_table, dtype=torch.long, device=state.device)
        self.seqlen_offset = start_pos
        self.cache_aprods = False

    # -- attention ---------------------------------------------------------------------
    def update_attention(self, layer_idx: int, k: torch.Tensor, v: torch.Tensor, window: Optional[int] = None):
        kc, vc = self.s.kv[layer_idx]
        bs = self.s.block_size
        n = k.shape[1]
        pos = torch.arange(self.start, self.start + n, device=k.device)
        flat = self.block_table[pos // bs] * bs + pos % bs
        kc.view(-1, *kc.shape[2:])[flat] = k[0]
        vc.view(-1, *vc.shape[2:])[flat] = v[0]
        if self.start == 0:
            return k, v
        lo = 0 if window is None else max(0, self.start - window + 1)
        prev = torch.arange(lo, self.start, device=k.device)
        pf = self.block_table[prev // bs] * bs + prev % bs
        k_all = torch.cat([kc.view(-1, *kc.shape[2:])[pf][None], k], dim=1)
        v_all = torch.cat([vc.view(-1, *vc.shape[2:])[pf][None], v], dim=1)
        return k_all, v_all

    # -- recurrent layers ----------------------------------------------------------------
    def update_bmojo(self, layer_idx, *args, **kw):
        return self.side.update_bmojo(layer_idx, *args, **kw)

    def get_ssm(self, layer_idx: int) -> Optional[dict]:
        if layer_idx in self.s.bmojo_layers:
            return self.side.get_ssm(layer_idx)
        if self.start == 0:
            return None
        e = self.s.ssm[layer_idx]
        conv = e["conv"][self.slot][None]
        if e["split"] is not None:
            parts = list(torch.split(conv, e["split"], dim=-1))
            while len(parts) < 3:
                parts.append(None)
            conv_state = tuple(p.contiguous() if p is not None else None for p in parts)
        else:
            conv_state = conv
        if e["kind"] == "gka":
            rec = (e["state_kk"][self.slot][None], e["state"][self.slot][None])
        else:
            rec = e["state"][self.slot][None]
        return {"recurrent_state": rec, "conv_state": conv_state, "log_aprod": None}

    def update_ssm(self, layer_idx: int, recurrent_state=None, conv_state=None, offset: int = 0, log_aprod=None, **kw):
        if layer_idx in self.s.bmojo_layers:
            return self.side.update_ssm(layer_idx, recurrent_state=recurrent_state, conv_state=conv_state, offset=offset)
        e = self.s.ssm[layer_idx]
        if recurrent_state is not None:
            if e["kind"] == "gka":
                h_kk, h_kv = recurrent_state
                if h_kk is not None:
                    e["state_kk"][self.slot].copy_(h_kk[0])
                e["state"][self.slot].copy_(h_kv[0])
            else:
                e["state"][self.slot].copy_(recurrent_state[0])
        if conv_state is not None:
            if isinstance(conv_state, (tuple, list)):
                parts = [c for c in conv_state if c is not None]
                e["conv"][self.slot].copy_(torch.cat(parts, dim=-1)[0])
            else:
                e["conv"][self.slot].copy_(conv_state[0])

    def update_offset(self, n: int) -> None:
        self.seqlen_offset += n

    def get_seq_length(self, layer_idx: int = 0) -> int:
        return self.seqlen_offset
