"""Mixture-of-depths: a decoder layer sees only the tokens its router picks; the others pass through on the residual
stream untouched.  Every ``every``-th layer gets a one-output router.  In training the router keeps the ``capacity``
fraction of each row with the highest scores (in sequence order, with their own rotary positions) and the layer's
update is scaled by the sigmoid of the score, so the router receives gradient; a binary cross-entropy term teaches the
same score to predict "would have been in the top-k", which is the causal rule used when decoding with a cache (a
token is processed when its sigmoid exceeds one half, whatever comes after it).

The reference obtains this from an external package (``model/model_utils/mod.py:30-44`` calls ``apply_mod_to_hf`` for a
list of supported architectures, ``hparams/model_args.py`` flag ``mixture_of_depths: convert | load``); here it is a
wrapper around this package's own ``DecoderLayer`` and therefore covers every mixer type.  Router weights are saved as
``model.layers.<i>.mod_router.weight``; :func:`apply_mixture_of_depths` has to run before such a checkpoint is loaded
(the ``load`` mode)."""
from __future__ import annotations

import math
import types
from typing import List, Optional

import torch
import torch.nn as nn
import torch.nn.functional as F


def _gather_tokens(t: Optional[torch.Tensor], idx: torch.Tensor) -> Optional[torch.Tensor]:
    """Rows ``idx`` ([B, k]) of a ``[B or 1, T, ...]`` tensor along the time axis."""
    if t is None:
        return None
    if t.dim() == 2:                                                  # position ids [B, T]
        return t.expand(idx.shape[0], -1).gather(1, idx)
    full = t.expand(idx.shape[0], *t.shape[1:])
    return full.gather(1, idx.reshape(*idx.shape, *([1] * (t.dim() - 2))).expand(-1, -1, *t.shape[2:]))


def _mod_forward(self, hidden_states, position_embeddings=None, position_ids=None, past_key_values=None,
                 use_cache=False, **kwargs):
    if kwargs.get("cu_seqlens") is not None or kwargs.get("sample_caches") is not None:
        raise NotImplementedError("mixture-of-depths layers take padded batches, not packed rows")
    B, T, _ = hidden_states.shape
    scores = F.linear(hidden_states, self.mod_router.weight).squeeze(-1).float()     # [B, T]
    causal = past_key_values is not None or not self.training
    if causal:
        keep = scores > 0                                                             # sigmoid > 1/2
        k = int(keep.sum(1).max())
        if k == 0:
            return hidden_states, None
        # rows pick different counts: every row takes its k best and the surplus gets weight zero
        order = torch.where(keep, scores, scores.new_full((), -float("inf"))).topk(k, dim=1).indices.sort(1).values
        live = keep.gather(1, order)
    else:
        k = max(1, min(T, math.ceil(self.mod_capacity * T)))
        order = scores.topk(k, dim=1).indices.sort(1).values
        live = None
        target = torch.zeros_like(scores).scatter_(1, order, 1.0)
        self.mod_aux_loss = F.binary_cross_entropy_with_logits(scores, target)
    picked = _gather_tokens(hidden_states, order)
    pe = None if position_embeddings is None else tuple(_gather_tokens(t, order) for t in position_embeddings)
    pid = _gather_tokens(position_ids, order)
    out, router_logits = self._mod_inner(picked, position_embeddings=pe, position_ids=pid,
                                         past_key_values=past_key_values, use_cache=use_cache, **kwargs)
    gate = torch.sigmoid(scores.gather(1, order))
    if live is not None:
        gate = gate * live
    delta = (out - picked) * gate.unsqueeze(-1).to(out.dtype)
    return hidden_states.scatter_add(1, order.unsqueeze(-1).expand_as(delta), delta), router_logits


def apply_mixture_of_depths(model: nn.Module, capacity: float = 0.125, every: int = 2, first: int = 1) -> List[int]:
    """Gives every ``every``-th decoder layer from ``first`` on a router and the routed forward.  Returns the indices."""
    if not 0.0 < capacity <= 1.0:
        raise ValueError(f"capacity {capacity} is not in (0, 1]")
    layers = model.model.layers if hasattr(model, "model") else model.layers
    hidden = model.config.hidden_size
    done = []
    for i in range(first, len(layers), every):
        layer = layers[i]
        if hasattr(layer, "mod_router"):
            continue
        if not hasattr(layer, "seq_mixer") or hasattr(layer, "teacher_mixer"):
            raise ValueError(f"layer {i} ({type(layer).__name__}) cannot be routed")
        ref = next(layer.parameters())
        layer.mod_router = nn.Linear(hidden, 1, bias=False, device=ref.device, dtype=ref.dtype)
        nn.init.normal_(layer.mod_router.weight, std=0.02)
        layer.mod_capacity = float(capacity)
        layer.mod_aux_loss = None
        layer._mod_inner = layer.forward
        layer.forward = types.MethodType(_mod_forward, layer)
        done.append(i)
    model.config.mixture_of_depths = {"capacity": capacity, "every": every, "first": first}
    return done


def mod_aux_loss(model: nn.Module) -> Optional[torch.Tensor]:
    """Mean of the routers' top-k prediction losses of the last training forward (``None`` without routed layers)."""
    terms = [m.mod_aux_loss for m in model.modules()
             if getattr(m, "mod_aux_loss", None) is not None and m.mod_aux_loss.requires_grad]
    return torch.stack(terms).mean() if terms else None
