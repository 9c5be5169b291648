"""Preference-style objectives on top of the shared training loop: DPO (sigmoid / IPO / hinge /
SimPO / ORPO variants), KTO and pairwise reward modelling.  Batches carry ``chosen_*`` and
``rejected_*`` tensors (KTO: ``input_ids``, ``labels``, ``kto_tags``).

The sigmoid / IPO / hinge DPO losses and KTO measure the policy against a frozen *reference policy*
(reference: ``train/dpo/trainer.py`` ``compute_reference_log_probs``, ``train/trainer_utils.py``
``create_ref_model``).  ``ReferencePolicy`` supplies its log-probabilities, in this order of preference:
values already in the batch (``ref_chosen_logps`` ...), a frozen model (``ft_args.ref_model`` or a copy of the
starting weights), or - for LoRA training - the policy itself with its adapters switched off.  A loss that needs
a reference and has none raises instead of silently training without the KL anchor.

The reward model scores a sequence with a scalar value head on the hidden state of its last real token
(reference: ``train/rm/trainer.py``).
"""
from __future__ import annotations

import contextlib
import copy
from typing import Optional

import torch
import torch.nn as nn
import torch.nn.functional as F

NEEDS_REFERENCE = ("sigmoid", "ipo", "hinge")


def sequence_logps(model, input_ids, labels, position_ids=None):
    """Sum of label log-probabilities per sequence and the number of supervised tokens."""
    out = model(input_ids, position_ids=position_ids, return_logits=True)
    logits = out.logits[:, :-1].float()
    tgt = labels[:, 1:]
    mask = tgt != -100
    logp = torch.gather(F.log_softmax(logits, dim=-1), 2, tgt.clamp(min=0).unsqueeze(-1)).squeeze(-1)
    return (logp * mask).sum(-1), mask.sum(-1)


@contextlib.contextmanager
def adapters_disabled(model: nn.Module):
    """Runs the enclosed forward passes on the base weights of a LoRA-wrapped model."""
    from .adapters import LoRALinear
    mods = [m for m in model.modules() if isinstance(m, LoRALinear)]
    for m in mods:
        m.enabled = False
    try:
        yield
    finally:
        for m in mods:
            m.enabled = True


class ReferencePolicy:
    """Log-probabilities of the frozen reference policy for a batch (see the module docstring)."""

    def __init__(self, model: Optional[nn.Module] = None, use_adapter_base: bool = False):
        self.model, self.use_adapter_base = model, use_adapter_base
        if model is not None:
            model.eval()
            for p in model.parameters():
                p.requires_grad_(False)

    @classmethod
    def build(cls, policy: nn.Module, ft_args, device=None) -> "ReferencePolicy":
        from .adapters import LoRALinear
        path = getattr(ft_args, "ref_model", None)
        if path:
            from ..utils import checkpoint_io
            ref = checkpoint_io.from_pretrained(path, device=device or next(policy.parameters()).device)
            return cls(ref.to(next(policy.parameters()).dtype))
        if any(isinstance(m, LoRALinear) for m in policy.modules()):
            return cls(None, use_adapter_base=True)
        return cls(copy.deepcopy(policy))

    @property
    def available(self) -> bool:
        return self.model is not None or self.use_adapter_base

    @torch.no_grad()
    def logps(self, policy: nn.Module, input_ids, labels):
        if self.model is not None:
            return sequence_logps(self.model, input_ids, labels)[0]
        if self.use_adapter_base:
            was = policy.training
            policy.eval()
            with adapters_disabled(policy):
                out = sequence_logps(policy, input_ids, labels)[0]
            policy.train(was)
            return out
        raise ValueError("this preference loss needs a reference policy: pass `ref_model`, train with LoRA, or put "
                         "ref_chosen_logps / ref_rejected_logps (KTO: ref_logps) into the batch")


def dpo_loss(pc, pr, rc, rr, beta=0.1, kind="sigmoid", nc=None, nr=None, gamma=0.5):
    if kind == "simpo":
        logits = beta * (pc / nc.clamp(min=1) - pr / nr.clamp(min=1)) - gamma
        return -F.logsigmoid(logits).mean()
    if kind == "orpo":
        lc, lr = pc / nc.clamp(min=1), pr / nr.clamp(min=1)
        odds = (lc - lr) - (torch.log1p(-torch.exp(lc)) - torch.log1p(-torch.exp(lr)))
        return (-lc - beta * F.logsigmoid(odds)).mean()
    if rc is None or rr is None:
        raise ValueError(f"pref_loss={kind} needs reference log-probabilities")
    logits = (pc - pr) - (rc - rr)
    if kind == "ipo":
        return ((logits - 1 / (2 * beta)) ** 2).mean()
    if kind == "hinge":
        return torch.relu(1 - beta * logits).mean()
    return -F.logsigmoid(beta * logits).mean()


def attach_value_head(model: nn.Module) -> nn.Linear:
    """Adds the scalar value head ``v_head`` (zero-initialised, saved with the checkpoint) if the model has none."""
    if not hasattr(model, "v_head"):
        p = next(model.parameters())
        head = nn.Linear(model.config.hidden_size, 1, bias=False, device=p.device, dtype=p.dtype)
        nn.init.normal_(head.weight, std=1.0 / (model.config.hidden_size + 1) ** 0.5)
        model.v_head = head
    return model.v_head


def last_token_index(input_ids: torch.Tensor, labels: Optional[torch.Tensor] = None, pad_id: int = 0) -> torch.Tensor:
    """Index of the last real token of each right-padded row: the last supervised label when labels are given,
    else the last token that is not the pad id."""
    real = (labels != -100) if labels is not None else (input_ids != pad_id)
    pos = torch.arange(input_ids.shape[1], device=input_ids.device)[None]
    return (real.long() * pos).amax(-1)


def reward_scores(model: nn.Module, input_ids, labels=None, pad_id: int = 0) -> torch.Tensor:
    h = model.model(input_ids)[0]
    last = last_token_index(input_ids, labels, pad_id)
    h_last = h[torch.arange(h.shape[0], device=h.device), last]
    return model.v_head(h_last).squeeze(-1).float()


def make_preference_loss(stage: str, ft_args, reference: Optional[ReferencePolicy] = None, pad_id: int = 0):
    beta, kind = ft_args.pref_beta, ft_args.pref_loss
    reference = reference or ReferencePolicy()

    def dpo(model, batch):
        pc, nc = sequence_logps(model, batch["chosen_input_ids"], batch["chosen_labels"])
        pr, nr = sequence_logps(model, batch["rejected_input_ids"], batch["rejected_labels"])
        rc, rr = batch.get("ref_chosen_logps"), batch.get("ref_rejected_logps")
        if kind in NEEDS_REFERENCE and (rc is None or rr is None):
            rc = reference.logps(model, batch["chosen_input_ids"], batch["chosen_labels"])
            rr = reference.logps(model, batch["rejected_input_ids"], batch["rejected_labels"])
        return dpo_loss(pc, pr, rc, rr, beta, kind, nc, nr)

    def kto(model, batch):
        lp, _ = sequence_logps(model, batch["input_ids"], batch["labels"])
        ref = batch.get("ref_logps")
        if ref is None:
            ref = reference.logps(model, batch["input_ids"], batch["labels"])
        tags = batch["kto_tags"].bool()
        r = lp - ref
        kl = r.detach().mean().clamp(min=0)
        des = 1 - torch.sigmoid(beta * (r - kl))
        und = 1 - torch.sigmoid(beta * (kl - r))
        return torch.where(tags, des, und).mean()

    def rm(model, batch):
        attach_value_head(model)
        sc = reward_scores(model, batch["chosen_input_ids"], batch.get("chosen_labels"), pad_id)
        sr = reward_scores(model, batch["rejected_input_ids"], batch.get("rejected_labels"), pad_id)
        return -F.logsigmoid(sc - sr).mean()

    return {"dpo": dpo, "kto": kto, "rm": rm}[stage]
