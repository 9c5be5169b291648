"""Parameter-efficient fine-tuning: LoRA adapters (plain, rank-stabilised, DoRA, PiSSA initialisation), LongLoRA's
shifted sparse attention, and layer freezing (``finetuning_type: lora | freeze``).

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
    """``use_rslora``: scale ``alpha / sqrt(rank)``.  ``use_dora``: weight-decomposed update, the merged weight is
    re-normalised per output row to a trainable magnitude ``m`` (initialised to the base row norms).  ``pissa``: ``A``
    and ``B`` start as the top-``rank`` singular directions of the base weight, which keeps only the residual
    (``pissa_iters`` > 0: randomised SVD with that many power iterations, else exact)."""

    def __init__(self, base: nn.Linear, rank: int, alpha: float, use_rslora: bool = False, use_dora: bool = False,
                 pissa: bool = False, pissa_iters: int = 0):
        super().__init__()
        self.base = base
        for p in self.base.parameters():
            p.requires_grad_(False)
        self.rank, self.scaling = rank, alpha / (math.sqrt(rank) if use_rslora else rank)
        self.enabled = True               # False: the base layer alone (reference policy of DPO / KTO)
        dev, dt = base.weight.device, base.weight.dtype
        self.lora_A = nn.Parameter(torch.empty(rank, base.in_features, device=dev, dtype=dt))
        self.lora_B = nn.Parameter(torch.zeros(base.out_features, rank, device=dev, dtype=dt))
        nn.init.kaiming_uniform_(self.lora_A, a=math.sqrt(5))
        if pissa:
            with torch.no_grad():
                w = base.weight.float()
                if pissa_iters > 0:
                    U, S, V = torch.svd_lowrank(w, q=rank, niter=pissa_iters)
                    Vh = V.t()
                else:
                    U, S, Vh = torch.linalg.svd(w, full_matrices=False)
                    U, S, Vh = U[:, :rank], S[:rank], Vh[:rank]
                root = torch.sqrt(S / self.scaling)
                self.lora_B.copy_((U * root).to(dt))
                self.lora_A.copy_((root[:, None] * Vh).to(dt))
                base.weight.sub_(((self.lora_B.float() @ self.lora_A.float()) * self.scaling).to(dt))
        self.magnitude = None
        if use_dora:
            with torch.no_grad():
                self.magnitude = nn.Parameter(self.merged_direction().float().norm(dim=1).to(dt))

    def merged_direction(self) -> torch.Tensor:
        return self.base.weight + (self.lora_B @ self.lora_A) * self.scaling

    @property
    def weight(self):
        return self.base.weight

    @property
    def bias(self):
        return self.base.bias

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        if not self.enabled:
            return self.base(x)
        if self.magnitude is not None:
            return nn.functional.linear(x, self.merged_weight(), self.base.bias)
        return self.base(x) + (x @ self.lora_A.t()) @ self.lora_B.t() * self.scaling

    def merged_weight(self) -> torch.Tensor:
        w = self.merged_direction()
        if self.magnitude is None:
            return w
        # the norm is treated as a constant in the backward pass, as the DoRA paper prescribes
        norm = w.detach().float().norm(dim=1, keepdim=True).clamp_min(1e-12)
        return (w.float() * (self.magnitude.float()[:, None] / norm)).to(w.dtype)


DEFAULT_TARGETS = ("q_proj", "k_proj", "v_proj", "o_proj", "gate_proj", "up_proj", "down_proj", "in_proj", "out_proj",
                   "g_proj")


def apply_lora(model: nn.Module, rank: int = 8, alpha: float = None, target: str = "all", use_rslora: bool = False,
               use_dora: bool = False, pissa_init: bool = False, pissa_iter: int = 0) -> List[str]:
    alpha = float(alpha if alpha is not None else 2 * rank)
    names = DEFAULT_TARGETS if target in ("all", None, "") else tuple(t.strip() for t in target.split(","))
    for p in model.parameters():
        p.requires_grad_(False)
    wrapped = []
    for parent_name, parent in list(model.named_modules()):
        for child_name, child in list(parent.named_children()):
            if isinstance(child, nn.Linear) and child_name in names and "lm_head" not in child_name:
                setattr(parent, child_name, LoRALinear(child, rank, alpha, use_rslora=use_rslora, use_dora=use_dora,
                                                       pissa=pissa_init, pissa_iters=pissa_iter))
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
                    merged = child.merged_weight()
                    if hasattr(child.base, "to_linear"):          # quantised base: back to an ordinary layer
                        child.base = child.base.to_linear()
                    child.base.weight.copy_(merged)
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


def shift_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, group: int, attend) -> torch.Tensor:
    """LongLoRA's shifted sparse attention for training on long inputs: the sequence is cut into groups of ``group``
    tokens that attend only inside themselves, and the second half of the heads works on the sequence rolled by half a
    group, so information still crosses the group borders.  ``q, k, v [B, T, H, D]`` (``T`` a multiple of ``group``,
    equal head counts); ``attend(q, k, v) -> o`` is causal attention over ``[B', group, H', D]``.  Reference: the
    ``shift_attn`` option of the inherited loader (``model/model_utils/longlora.py``)."""
    B, T, H, D = q.shape
    if T % group != 0:
        raise ValueError(f"sequence length {T} is not a multiple of the attention group {group}")
    half = H // 2

    def fold(x):
        x = torch.cat([x[:, :, :half], torch.roll(x[:, :, half:], -group // 2, dims=1)], dim=2)
        return x.reshape(B * (T // group), group, H, D)
    o = attend(fold(q), fold(k), fold(v)).reshape(B, T, H, D)
    return torch.cat([o[:, :, :half], torch.roll(o[:, :, half:], group // 2, dims=1)], dim=2)


def add_neftune(model: nn.Module, alpha: float = 5.0):
    """Noisy embeddings for instruction tuning: while the model is in training mode, uniform noise in
    ``[-s, s]`` with ``s = alpha / sqrt(tokens x width)`` is added to the output of the input embedding; evaluation
    and generation are untouched.  Returns the hook handle (``handle.remove()`` switches it off).
    Reference: the ``neftune_noise_alpha`` training argument inherited from the Hugging Face trainer."""
    emb = model.get_input_embeddings() if hasattr(model, "get_input_embeddings") else model.model.embed_tokens

    def hook(module, inputs, output):
        if not module.training:
            return output
        scale = alpha / (output.shape[-2] * output.shape[-1]) ** 0.5
        return output + torch.empty_like(output).uniform_(-scale, scale)

    return emb.register_forward_hook(hook)
