"""Token-reweighted supervised losses, evaluated chunk by chunk on the hidden states so that the ``[T, vocab]`` logits
of a long sample never exist at once.

* ``dft``  (dynamic fine-tuning): every token's cross entropy is scaled by the (detached) probability the model
  gives its target, which damps the gradient of tokens the model finds implausible.
* ``eaft`` (entropy-aware fine-tuning): scaled by ``(H_20 / 3) ** alpha`` with ``H_20`` the entropy of the
  re-normalised 20 largest probabilities (detached): confident positions count less.

Reference: ``train/trainer_utils.py:696-801`` (``dft_loss_func``, ``eaft_loss_func``).  Under sequence parallelism the
sums are reduced over the group like the ordinary loss (``parallel/sp.py::reduce_loss``)."""
from __future__ import annotations

from typing import Callable

import torch
import torch.nn.functional as F

from ..parallel.sp import reduce_loss

IGNORE_INDEX = -100


def token_weights(logits: torch.Tensor, ce: torch.Tensor, kind: str, alpha: float = 1.0) -> torch.Tensor:
    """Detached per-token weights for ``logits [n, V]`` (fp32) and their cross entropies ``ce [n]``."""
    with torch.no_grad():
        if kind == "dft":
            return torch.exp(-ce)
        if kind == "eaft":
            top = torch.topk(logits, k=min(20, logits.shape[-1]), dim=-1).values
            logp = top - torch.logsumexp(top, dim=-1, keepdim=True)
            entropy = -(logp.exp() * logp).sum(-1)
            return torch.pow(entropy / 3.0, alpha)
    raise ValueError(f"unknown loss '{kind}'")


def weighted_ce_sum(hidden: torch.Tensor, weight: torch.Tensor, labels: torch.Tensor, kind: str, alpha: float = 1.0,
                    chunk: int = 4096):
    """``(sum of weighted token losses, number of valid tokens)`` for ``hidden [n, D]`` and ``labels [n]``."""
    total = hidden.new_zeros((), dtype=torch.float32)
    count = torch.zeros((), device=hidden.device, dtype=torch.float32)
    for s in range(0, hidden.shape[0], chunk):
        y = labels[s:s + chunk]
        valid = y != IGNORE_INDEX
        if not bool(valid.any()):
            continue
        h = hidden[s:s + chunk][valid]

        def piece(h_, y_):
            logits = F.linear(h_, weight).float()
            ce = F.cross_entropy(logits, y_, reduction="none")
            return (ce * token_weights(logits, ce.detach(), kind, alpha)).sum()
        # the chunk's logits are rebuilt in the backward pass instead of being kept
        if torch.is_grad_enabled() and (h.requires_grad or weight.requires_grad):
            total = total + torch.utils.checkpoint.checkpoint(piece, h, y[valid], use_reentrant=False)
        else:
            total = total + piece(h, y[valid])
        count = count + valid.sum()
    return total, count


def make_weighted_sft_loss(kind: str, alpha: float = 1.0, chunk: int = 4096) -> Callable:
    """``loss_fn(model, batch)`` for ``train.trainer.Trainer``."""
    def loss_fn(model, batch):
        h, _ = model.model(batch["input_ids"], position_ids=batch.get("position_ids"))
        labels = batch["labels"]
        sp = getattr(model, "sequence_parallel_group", None)
        if batch.get("labels_shifted") or (sp is not None and sp.size > 1):
            hs, ys = h, labels
        else:
            hs, ys = h[:, :-1], labels[:, 1:]
        s, n = weighted_ce_sum(hs.reshape(-1, hs.shape[-1]), model.lm_head.weight, ys.reshape(-1), kind, alpha, chunk)
        return reduce_loss(s, n, sp)[0]
    return loss_fn
