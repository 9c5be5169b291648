"""Parameter-efficient fine-tuning: LoRA adapters and layer freezing (``finetuning_type: lora | freeze``).

``apply_lora`` replaces the targeted ``nn.Linear`` modules by ``LoRALinear`` (frozen base weight, trainable low-rank
update ``B A`` scaled by ``alpha / rank``, ``B`` zero-initialised); ``merge_lora`` folds the update back so the
checkpoint has the ordinary layout.  ``freeze_all_but_last`` keeps only the last ``n`` decoder layers trainable.
Reference: the LLaMA-Factory adapter options kept by the reference (``model/adapter.py``).
"""
from __future__ import annotations

import math
from typing import Iterable, List

import torch
import torch.nn as nn


class LoRALinear(nn.Module):
    def __init__(self, base: nn.Linear, rank: int, alpha: float):
        super().__init__()
        self.base = base
        for p in self.base.parameters():
            p.requires_grad_(False)
        self.rank, self.scaling = rank, alpha / rank
        self.enabled = True               # False: the base layer alone (reference policy of DPO / KTO)
        dev, dt = base.weight.device, base.weight.dtype
        self.lora_A = nn.Parameter(torch.empty(rank, base.in_features, device=dev, dtype=dt))
        self.lora_B = nn.Parameter(torch.zeros(base.out_features, rank, device=dev, dtype=dt))
        nn.init.kaiming_uniform_(self.lora_A, a=math.sqrt(5))

    @property
    def weight(self):
        return self.base.weight

    @property
    def bias(self):
        return self.base.bias

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        if not self.enabled:
            return self.base(x)
        return self.base(x) + (x @ self.lora_A.t()) @ self.lora_B.t() * self.scaling

    def merged_weight(self) -> torch.Tensor:
        return self.base.weight + (self.lora_B @ self.lora_A) * self.scaling


DEFAULT_TARGETS = ("q_proj", "k_proj", "v_proj", "o_proj", "gate_proj", "up_proj", "down_proj", "in_proj", "out_proj",
                   "g_proj")


def apply_lora(model: nn.Module, rank: int = 8, alpha: float = None, target: str = "all") -> List[str]:
    alpha = float(alpha if alpha is not None else 2 * rank)
    names = DEFAULT_TARGETS if target in ("all", None, "") else tuple(t.strip() for t in target.split(","))
    for p in model.parameters():
        p.requires_grad_(False)
    wrapped = []
    for parent_name, parent in list(model.named_modules()):
        for child_name, child in list(parent.named_children()):
            if isinstance(child, nn.Linear) and child_name in names and "lm_head" not in child_name:
                setattr(parent, child_name, LoRALinear(child, rank, alpha))
                wrapped.append(f"{parent_name}.{child_name}".lstrip("."))
    if not wrapped:
        raise ValueError(f"lora_target '{target}' matches no linear layer")
    return wrapped


def merge_lora(model: nn.Module) -> int:
    n = 0
    for parent in list(model.modules()):
        for child_name, child in list(parent.named_children()):
            if isinstance(child, LoRALinear):
                with torch.no_grad():
                    child.base.weight.copy_(child.merged_weight())
                setattr(parent, child_name, child.base)
                n += 1
    return n


def freeze_all_but_last(model: nn.Module, trainable_layers: int, extra: Iterable[str] = ("norm",)) -> int:
    """Trains the last ``trainable_layers`` decoder layers (and the final norm); returns the trainable count."""
    layers = model.model.layers
    keep = set(range(len(layers) - trainable_layers, len(layers)))
    for p in model.parameters():
        p.requires_grad_(False)
    for i in keep:
        for p in layers[i].parameters():
            p.requires_grad_(True)
    for name, p in model.model.named_parameters():
        if not name.startswith("layers.") and any(e in name for e in extra):
            p.requires_grad_(True)
    return sum(p.numel() for p in model.parameters() if p.requires_grad)
