"""Collators for packed sequences (``neat_packing``): samples packed into one row must not attend to one another.

* ``prepare_4d_attention_mask``: from a mask that numbers the packed samples (``1 1 1 2 2 3 3 3 0 0``) to the additive
  block-diagonal causal mask ``[B, 1, T, T]`` (0 where attention is allowed, the dtype's minimum elsewhere) that eager
  attention implementations take (reference: ``data/collator.py:257-295``, ``model_utils/packing.py``).
* ``segment_boundaries``: the same information as ``cu_seqlens`` (``[0, e_1, e_2, ..., T]`` per row), which is what
  this framework's model consumes: every sequence mixer (attention kernels, GDN / GKA / Mamba2 scans) then runs once per
  packed sample on its slice (``HybridModel.forward(..., cu_seqlens=...)``), so no ``T x T`` mask is ever built on
  the GPU path and recurrent state never leaks across samples.
* ``PackedSequenceCollator``: pads a list of tokenised rows, passes ``position_ids`` through (they restart at every
  packed sample) and emits ``cu_seqlens`` (and the 4-D mask on request).
"""
from __future__ import annotations

from typing import Dict, List, Optional, Sequence

import torch

IGNORE_INDEX = -100


def prepare_4d_attention_mask(attention_mask_with_indices: torch.Tensor, dtype: torch.dtype = torch.float32) -> torch.Tensor:
    """``[B, T]`` sample numbers (0 = padding) -> additive mask ``[B, 1, T, T]``."""
    B, T = attention_mask_with_indices.shape
    idx = attention_mask_with_indices
    same = (idx[:, None, :, None] == idx[:, None, None, :]) & (idx[:, None, None, :] != 0)
    causal = torch.tril(torch.ones(T, T, dtype=torch.bool, device=idx.device))
    allowed = same & causal
    return torch.where(allowed, torch.zeros((), dtype=dtype, device=idx.device),
                       torch.full((), torch.finfo(dtype).min, dtype=dtype, device=idx.device))


def segment_boundaries(attention_mask_with_indices: torch.Tensor) -> List[List[int]]:
    """Per row: ``[0, end of sample 1, end of sample 2, ..., T]`` (the padding tail is its own last segment)."""
    out = []
    for row in attention_mask_with_indices.tolist():
        cuts = [0]
        for t in range(1, len(row)):
            if row[t] != row[t - 1]:
                cuts.append(t)
        cuts.append(len(row))
        out.append(cuts)
    return out


def indices_from_position_ids(position_ids: Sequence[int], valid: int) -> List[int]:
    """Sample numbers of a packed row whose position ids restart at 0 for every sample (``valid`` real tokens)."""
    idx, cur = [], 0
    for t, p in enumerate(position_ids):
        if t >= valid:
            idx.append(0)
            continue
        if p == 0:
            cur += 1
        idx.append(cur)
    return idx


class PackedSequenceCollator:
    def __init__(self, pad_id: int = 0, block_diag_attn: bool = True, with_4d_mask: bool = False,
                 mask_dtype: torch.dtype = torch.float32, pad_to_multiple_of: Optional[int] = 8):
        self.pad_id, self.block_diag_attn, self.with_4d_mask = pad_id, block_diag_attn, with_4d_mask
        self.mask_dtype, self.multiple = mask_dtype, pad_to_multiple_of

    def __call__(self, rows: Sequence[Dict[str, List[int]]]) -> Dict[str, torch.Tensor]:
        L = max(len(r["input_ids"]) for r in rows)
        if self.multiple:
            L = (L + self.multiple - 1) // self.multiple * self.multiple
        ids, labels, pos, seg = [], [], [], []
        for r in rows:
            n = len(r["input_ids"])
            valid = n
            while valid > 0 and r["labels"][valid - 1] == IGNORE_INDEX and r["input_ids"][valid - 1] == self.pad_id:
                valid -= 1                                     # rows that were padded at packing time
            p = list(r.get("position_ids") or range(n))
            ids.append(list(r["input_ids"]) + [self.pad_id] * (L - n))
            labels.append(list(r["labels"]) + [IGNORE_INDEX] * (L - n))
            pos.append(p + list(range(L - n)))
            seg.append((indices_from_position_ids(p, valid) if self.block_diag_attn else [1] * valid + [0] * (n - valid))
                       + [0] * (L - n))
        batch = {"input_ids": torch.tensor(ids), "labels": torch.tensor(labels), "position_ids": torch.tensor(pos)}
        seg_t = torch.tensor(seg)
        batch["attention_mask"] = seg_t
        batch["cu_seqlens"] = segment_boundaries(seg_t)
        if self.with_4d_mask:
            batch["attention_mask_4d"] = prepare_4d_attention_mask(seg_t, self.mask_dtype)
        return batch
