"""L2A training objective: language-model loss + ``lambda(step) * sparsity regulariser`` with a linear / cosine /
constant ramp of ``lambda`` after warm-up.  Reference: ``examples/research/L2A/train/l2a/trainer.py:171-294``."""
from __future__ import annotations

import math

from ..layers.l2a import l2a_regulariser, router_sparsity, set_l2a_step


def lambda_schedule(step: int, lambda_reg: float, warmup_steps: int, total_steps: int, kind: str = "linear") -> float:
    if step < warmup_steps:
        return 0.0
    progress = min(1.0, (step - warmup_steps) / (total_steps - warmup_steps + 1e-9))
    if kind == "linear":
        return progress * lambda_reg
    if kind == "cosine":
        return 0.5 * (1 - math.cos(math.pi * progress)) * lambda_reg
    return lambda_reg


class L2ALoss:
    """``loss_fn`` for ``train.trainer.Trainer``."""

    def __init__(self, trainer_args, lambda_reg: float = 1e-2, scheduler: str = "linear"):
        self.args, self.lambda_reg, self.scheduler = trainer_args, lambda_reg, scheduler
        self.step = 0
        self.last_sparsity = {}

    def __call__(self, model, batch):
        set_l2a_step(model, self.step)
        out = model(input_ids=batch["input_ids"], labels=batch["labels"], position_ids=batch.get("position_ids"),
                    labels_shifted=bool(batch.get("labels_shifted", False)))
        lam = lambda_schedule(self.step, self.lambda_reg, self.args.warmup_steps, self.args.max_steps, self.scheduler)
        self.step += 1
        self.last_sparsity = router_sparsity(model)
        return out.loss + lam * l2a_regulariser(model).to(out.loss.dtype)
