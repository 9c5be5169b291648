"""State composition over independently processed context chunks (PICASO, arXiv 2502.17605).

A long context is cut into ``N`` chunks that are prefilled independently (each after an optional shared
prefix); their caches are merged into one cache from which the query is answered:

* KV side: ``full`` (ordinary prefill of the whole context), ``concat`` (K/V of all chunks side by side, the
  prefix kept once), ``sw`` (prefix + last chunk only);
* SSM side: ``kv_only`` (recurrent states zeroed), ``soup`` (mean of the chunk states), ``fuse`` (permutation
  average of sequential composition: chunk ``i`` gets weight ``1/N * sum_k e_k(A_{-i}) / C(N-1, k)`` with
  ``e_k`` the elementary symmetric polynomial of the other chunks' cumulative transitions; scalar and
  log-space for Mamba2, matrix-valued for Gated DeltaNet, plain sum for Gated KalmaNet whose states are
  information matrices).

``compose_type`` is ``"<kv>_<ssm>"`` (nine combinations), as in the reference
(``models/cache_compose.py:30-44``, coefficient math ``:912-1035``).
"""
from __future__ import annotations

import math
from typing import List, Optional, Sequence

import torch

from ..layers.gdn import GatedDeltaNet
from ..layers.gka import GatedKalmaNet
from ..layers.mamba2 import Mamba2
from .cache import HybridCache

KV_MODES, SSM_MODES = ("full", "concat", "sw"), ("kv_only", "soup", "fuse")


# -- coefficients --------------------------------------------------------------------------------
def picaso_coefficients(A: torch.Tensor) -> torch.Tensor:
    """``A [N, ...]`` scalar (elementwise) transitions of the chunks.  Returns ``c [N, ...]`` such that
    ``sum_i c_i s_i`` is the average over all chunk orders of the sequentially composed state."""
    N = A.shape[0]
    out = []
    for i in range(N):
        others = torch.cat([A[:i], A[i + 1:]], dim=0)
        # e[k] = elementary symmetric polynomial of degree k of `others`
        e = [torch.ones_like(A[0])] + [torch.zeros_like(A[0]) for _ in range(N - 1)]
        for a in others:
            for k in range(N - 1, 0, -1):
                e[k] = e[k] + a * e[k - 1]
        out.append(sum(e[k] / math.comb(N - 1, k) for k in range(N)) / N)
    return torch.stack(out, dim=0)


def picaso_log_coefficients(log_A: torch.Tensor) -> torch.Tensor:
    """Same in log space (``log_A`` = log of the cumulative decays); returns ``log c``."""
    N = log_A.shape[0]
    log_A = log_A.float()
    out = []
    neg_inf = torch.full_like(log_A[0], float("-inf"))
    for i in range(N):
        others = torch.cat([log_A[:i], log_A[i + 1:]], dim=0)
        e = [torch.zeros_like(log_A[0])] + [neg_inf.clone() for _ in range(N - 1)]
        for a in others:
            for k in range(N - 1, 0, -1):
                e[k] = torch.logaddexp(e[k], a + e[k - 1])
        terms = torch.stack([e[k] - math.log(math.comb(N - 1, k)) for k in range(N)], dim=0)
        out.append(torch.logsumexp(terms, dim=0) - math.log(N))
    return torch.stack(out, dim=0)


def picaso_matrix_coefficients(Phi: torch.Tensor) -> torch.Tensor:
    """Matrix-valued transitions ``Phi [N, ..., D, D]`` (products taken in chunk order)."""
    N = Phi.shape[0]
    eye = torch.eye(Phi.shape[-1], dtype=Phi.dtype, device=Phi.device).expand_as(Phi[0])
    out = []
    for i in range(N):
        others = torch.cat([Phi[:i], Phi[i + 1:]], dim=0)
        e = [eye.clone()] + [torch.zeros_like(Phi[0]) for _ in range(N - 1)]
        for a in others:
            for k in range(N - 1, 0, -1):
                e[k] = e[k] + a @ e[k - 1]
        out.append(sum(e[k] / math.comb(N - 1, k) for k in range(N)) / N)
    return torch.stack(out, dim=0)


# -- merging caches --------------------------------------------------------------------------------
def _mean_conv(states):
    first = states[0]
    if first is None:
        return None
    if isinstance(first, (tuple, list)):
        return tuple(None if first[j] is None else torch.stack([s[j] for s in states]).mean(0) for j in range(len(first)))
    return torch.stack(states).mean(0)


def combine_ssm(mixer, entries: Sequence[dict], mode: str) -> dict:
    """Merges the per-chunk SSM cache entries of one layer."""
    rec = [e["recurrent_state"] for e in entries]
    conv = _mean_conv([e["conv_state"] for e in entries])
    if isinstance(mixer, GatedKalmaNet):
        stack = lambda j: None if rec[0][j] is None else torch.stack([r[j] for r in rec])  # noqa: E731
        hkk, hkv = stack(0), stack(1)
        if mode == "kv_only":
            new = (None if hkk is None else torch.zeros_like(hkk[0]), torch.zeros_like(hkv[0]))
        elif mode == "soup":
            new = (None if hkk is None else hkk.mean(0), hkv.mean(0))
        else:   # information matrices / vectors add up
            new = (None if hkk is None else hkk.sum(0), hkv.sum(0))
        return {"recurrent_state": new, "conv_state": conv, "log_aprod": None}
    S = torch.stack(rec)                                   # [N, B, H, ., .]
    if mode == "kv_only":
        new = torch.zeros_like(S[0])
    elif mode == "soup" or len(entries) == 1:
        new = S.mean(0)
    elif isinstance(mixer, Mamba2):
        la = [e.get("log_aprod") for e in entries]
        if any(a is None for a in la):
            raise ValueError("fuse composition of Mamba2 needs the cumulative log decays (cache_aprods=True)")
        c = torch.exp(picaso_log_coefficients(torch.stack(la)))          # [N, B, H]
        new = (c[..., None, None] * S).sum(0)
    elif isinstance(mixer, GatedDeltaNet):
        tr = [e.get("transition") for e in entries]
        if any(t is None for t in tr):
            raise ValueError("fuse composition of Gated DeltaNet needs the chunk transition matrices "
                             "(cache_transitions=True)")
        c = picaso_matrix_coefficients(torch.stack(tr).float())          # [N, B, H, Dk, Dk]
        new = (c @ S.float()).sum(0)
    else:
        raise NotImplementedError(type(mixer).__name__)
    return {"recurrent_state": new, "conv_state": conv, "log_aprod": None}


@torch.no_grad()
def compose_cache(model, chunks: List[torch.Tensor], compose_type: str = "concat_fuse",
                  prefix: Optional[torch.Tensor] = None, sequential_positions: bool = True) -> HybridCache:
    """Prefills ``chunks`` (each ``[1, T_i]`` token ids) independently after ``prefix`` and merges the caches."""
    kv_mode, _, ssm_mode = compose_type.partition("_")
    assert kv_mode in KV_MODES and ssm_mode in SSM_MODES, f"unknown compose_type {compose_type}"
    layers = model.model.layers
    P = 0 if prefix is None else prefix.shape[1]
    caches, start = [], P
    for ch in chunks:
        cache = HybridCache(cache_aprods=True)
        cache.cache_transitions = ssm_mode == "fuse"
        ids = ch if prefix is None else torch.cat([prefix, ch], dim=1)
        first = start if sequential_positions else P
        pos = torch.arange(first, first + ch.shape[1], device=ch.device)
        if prefix is not None:
            pos = torch.cat([torch.arange(P, device=ch.device), pos])
        model.model(ids, position_ids=pos[None], past_key_values=cache, use_cache=True)
        caches.append(cache)
        start += ch.shape[1]
    total = P + sum(c.shape[1] for c in chunks)
    if kv_mode == "full":      # ordinary prefill for the K/V side, composed states for the SSM side
        full = HybridCache(cache_aprods=False)
        ids = torch.cat(([prefix] if prefix is not None else []) + list(chunks), dim=1)
        model.model(ids, past_key_values=full, use_cache=True)
        out = full
    else:
        out = HybridCache(cache_aprods=False)
    for i, layer in enumerate(layers):
        mixer = layer.seq_mixer
        if i in caches[0].ssm:
            out.ssm[i] = combine_ssm(mixer, [c.ssm[i] for c in caches], ssm_mode)
        elif i in caches[0].attention and kv_mode != "full":
            ks, vs = zip(*[c.attention[i] for c in caches])
            if kv_mode == "sw":
                out.attention[i] = (ks[-1], vs[-1])
            else:   # the prefix once, then every chunk's own keys / values
                k = torch.cat([ks[0][:, :P]] + [kk[:, P:] for kk in ks], dim=1)
                v = torch.cat([vs[0][:, :P]] + [vv[:, P:] for vv in vs], dim=1)
                out.attention[i] = (k, v)
    out.seqlen_offset = total
    return out


@torch.no_grad()
def generate_composed(model, context: torch.Tensor, query: torch.Tensor, num_chunks: int = 4,
                      compose_type: str = "concat_fuse", prefix: Optional[torch.Tensor] = None,
                      max_new_tokens: int = 32, eos_token_id: Optional[int] = None) -> torch.Tensor:
    """Greedy generation from a composed cache: ``context [1, T]`` is cut into ``num_chunks`` pieces."""
    chunks = [c for c in torch.tensor_split(context, num_chunks, dim=1) if c.shape[1]]
    cache = compose_cache(model, chunks, compose_type, prefix)
    pos0 = cache.seqlen_offset
    ids = query
    out = []
    for _ in range(max_new_tokens):
        pos = torch.arange(pos0, pos0 + ids.shape[1], device=ids.device)[None]
        h, _ = model.model(ids, position_ids=pos, past_key_values=cache, use_cache=True)
        nxt = model.lm_head(h[:, -1:]).argmax(-1)
        out.append(nxt)
        pos0 += ids.shape[1]
        ids = nxt
        if eos_token_id is not None and int(nxt) == eos_token_id:
            break
    return torch.cat(out, dim=1)


def wrap_for_composition(model, tokenizer=None):
    """Adds ``model.generate_composed`` / ``model.compose_cache`` (API of the reference's
    ``wrap_for_composition``)."""
    import types
    model.has_cache_compose = True
    model.compose_cache = types.MethodType(compose_cache, model)
    model.generate_composed = types.MethodType(generate_composed, model)
    if tokenizer is not None:
        model.config.newline_token_id = tokenizer.encode("\n", add_special_tokens=False)[0]
    return model
