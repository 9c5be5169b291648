"""Preference-style objectives on top of the shared training loop: DPO (sigmoid / IPO / hinge /
SimPO / ORPO variants), KTO and pairwise reward modelling.  Batches carry ``chosen_*`` and
``rejected_*`` tensors (KTO: ``input_ids``, ``labels``, ``kto_tags``).  These stages are inherited
functionality of the reference project (``train/dpo``, ``train/kto``, ``train/rm``; "available but
untested" there) and are kept functionally, not tuned for speed.
"""
from __future__ import annotations

import torch
import torch.nn.functional as F


def sequence_logps(model, input_ids, labels, position_ids=None):
    """Sum of label log-probabilities per sequence and the number of supervised tokens."""
    out = model(input_ids, position_ids=position_ids, return_logits=True)
    logits = out.logits[:, :-1].float()
    tgt = labels[:, 1:]
    mask = tgt != -100
    logp = torch.gather(F.log_softmax(logits, dim=-1), 2, tgt.clamp(min=0).unsqueeze(-1)).squeeze(-1)
    return (logp * mask).sum(-1), mask.sum(-1)


def dpo_loss(pc, pr, rc, rr, beta=0.1, kind="sigmoid", nc=None, nr=None, gamma=0.5):
    if kind == "simpo":
        logits = beta * (pc / nc.clamp(min=1) - pr / nr.clamp(min=1)) - gamma
        return -F.logsigmoid(logits).mean()
    if kind == "orpo":
        lc, lr = pc / nc.clamp(min=1), pr / nr.clamp(min=1)
        odds = (lc - lr) - (torch.log1p(-torch.exp(lc)) - torch.log1p(-torch.exp(lr)))
        return (-lc - beta * F.logsigmoid(odds)).mean()
    logits = (pc - pr) - (rc - rr)
    if kind == "ipo":
        return ((logits - 1 / (2 * beta)) ** 2).mean()
    if kind == "hinge":
        return torch.relu(1 - beta * logits).mean()
    return -F.logsigmoid(beta * logits).mean()


def make_preference_loss(stage: str, ft_args):
    beta, kind = ft_args.pref_beta, ft_args.pref_loss

    def dpo(model, batch):
        pc, nc = sequence_logps(model, batch["chosen_input_ids"], batch["chosen_labels"])
        pr, nr = sequence_logps(model, batch["rejected_input_ids"], batch["rejected_labels"])
        rc = batch.get("ref_chosen_logps", pc.detach())
        rr = batch.get("ref_rejected_logps", pr.detach())
        return dpo_loss(pc, pr, rc, rr, beta, kind, nc, nr)

    def kto(model, batch):
        lp, _ = sequence_logps(model, batch["input_ids"], batch["labels"])
        ref = batch.get("ref_logps", lp.detach())
        tags = batch["kto_tags"].bool()
        r = lp - ref
        kl = r.detach().mean().clamp(min=0)
        des = 1 - torch.sigmoid(beta * (r - kl))
        und = 1 - torch.sigmoid(beta * (kl - r))
        return torch.where(tags, des, und).mean()

    def rm(model, batch):
        # reward = projection of the last hidden state on the LM head's EOS row (no separate value head)
        def score(ids):
            h = model.model(ids)[0][:, -1].float()
            return h @ model.lm_head.weight[0].float()
        return -F.logsigmoid(score(batch["chosen_input_ids"]) - score(batch["rejected_input_ids"])).mean()

    return {"dpo": dpo, "kto": kto, "rm": rm}[stage]
