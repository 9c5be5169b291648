"""Model patchers applied between loading and training: vocabulary resize, fp32 up-casts, RoPE scaling for longer
contexts, and the OFT adapter (orthogonal fine-tuning) next to LoRA / freeze in ``train/adapters.py``.

Reference: ``model/patcher.py`` (``patch_config`` / ``patch_model``), ``model/model_utils/embedding.py`` (noisy-mean
resize), ``model/model_utils/rope.py`` (scaling factor from the target length), ``model/adapter.py`` (adapter setup).
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch
import torch.nn as nn


# -- vocabulary -------------------------------------------------------------------------------------------------------
def resize_embedding_layer(model, new_vocab_size: int, pad_to_multiple_of: int = 64) -> int:
    """Grows (never shrinks) the input embedding and the output head to ``new_vocab_size`` rounded up to a multiple of
    ``pad_to_multiple_of``.  New rows are the mean of the old ones plus small noise, so new tokens start near the
    centre of the embedding cloud instead of at an arbitrary point.  Returns the new size."""
    emb = model.model.embed_tokens
    old = emb.weight.shape[0]
    target = (max(new_vocab_size, old) + pad_to_multiple_of - 1) // pad_to_multiple_of * pad_to_multiple_of
    if target == old:
        return old
    tied = model.lm_head.weight is emb.weight

    def grow(w: torch.Tensor) -> torch.Tensor:
        mean = w.float().mean(0, keepdim=True)
        noise = torch.randn(target - old, w.shape[1], device=w.device) * (1.0 / math.sqrt(w.shape[1]))
        return torch.cat([w, (mean + noise * w.float().std()).to(w.dtype)], 0)
    with torch.no_grad():
        emb.weight = nn.Parameter(grow(emb.weight.data), requires_grad=emb.weight.requires_grad)
        emb.num_embeddings = target
        if tied:
            model.lm_head.weight = emb.weight
        else:
            model.lm_head.weight = nn.Parameter(grow(model.lm_head.weight.data),
                                                requires_grad=model.lm_head.weight.requires_grad)
            if model.lm_head.bias is not None:
                b = model.lm_head.bias.data
                model.lm_head.bias = nn.Parameter(torch.cat([b, b.new_zeros(target - old)]))
        model.lm_head.out_features = target
    model.config.vocab_size = target
    return target


# -- precision ---------------------------------------------------------------------------------------------------------
def upcast_layernorm(model) -> int:
    """Keeps every 1-D norm weight in fp32 (``upcast_layernorm``); returns how many were cast."""
    n = 0
    for name, p in model.named_parameters():
        if p.dim() == 1 and "norm" in name and p.dtype != torch.float32:
            p.data = p.data.float()
            n += 1
    return n


def upcast_lmhead_output(model) -> None:
    """The logits leave the output head in fp32 (``upcast_lmhead_output``)."""
    def hook(_m, _a, out):
        return out.float()
    model.lm_head.register_forward_hook(hook)


# -- RoPE scaling ---------------------------------------------------------------------------------------------------------
def configure_rope_scaling(config, rope_scaling: Optional[str], model_max_length: Optional[int]) -> Optional[dict]:
    """``rope_scaling``: ``linear`` | ``dynamic`` | ``yarn`` | ``llama3``; the factor is the ratio of the wanted context
    (``model_max_length``) to the model's ``max_position_embeddings``, at least 1.  Writes ``config.rope_scaling`` and
    raises ``max_position_embeddings`` (call before the model is built)."""
    if not rope_scaling:
        return None
    cur = int(getattr(config, "max_position_embeddings", 0) or 0)
    if not model_max_length or not cur or model_max_length <= cur:
        factor = 1.0 if not (model_max_length and cur) else max(1.0, model_max_length / cur)
    else:
        factor = float(math.ceil(model_max_length / cur))
    rs = {"rope_type": rope_scaling, "factor": factor}
    if rope_scaling in ("dynamic", "yarn", "llama3"):
        rs["original_max_position_embeddings"] = cur
    if rope_scaling == "llama3":
        rs.update(low_freq_factor=1.0, high_freq_factor=4.0)
    config.rope_scaling = rs
    if model_max_length and cur and model_max_length > cur:
        config.max_position_embeddings = int(cur * factor)
    return rs


# -- OFT ---------------------------------------------------------------------------------------------------------------------
class OFTLinear(nn.Module):
    """``y = x (R W)^T + b`` with ``R`` block-diagonal orthogonal, ``R_b = (I + Q_b)(I - Q_b)^-1`` (Cayley transform of a
    skew-symmetric ``Q_b = S_b - S_b^T``); ``S = 0`` at the start, so the wrapped layer initially equals the frozen one.
    Only ``S`` trains: the hyperspherical energy (pairwise angles between neurons) of ``W`` is preserved."""

    def __init__(self, base: nn.Linear, block_size: int = 32):
        super().__init__()
        out = base.out_features
        assert out % block_size == 0, f"out_features {out} is not a multiple of the OFT block size {block_size}"
        self.base, self.block_size, self.n_blocks = base, block_size, out // block_size
        for p in base.parameters():
            p.requires_grad_(False)
        self.oft_s = nn.Parameter(torch.zeros(self.n_blocks, block_size, block_size, dtype=torch.float32,
                                              device=base.weight.device))

    def rotation(self) -> torch.Tensor:
        q = self.oft_s - self.oft_s.transpose(-1, -2)
        eye = torch.eye(self.block_size, device=q.device, dtype=q.dtype).expand_as(q)
        return torch.linalg.solve(eye - q, eye + q)                 # (I - Q)^-1 (I + Q), orthogonal

    def rotated_weight(self) -> torch.Tensor:
        w = self.base.weight
        wb = w.float().view(self.n_blocks, self.block_size, -1)
        return (self.rotation() @ wb).view_as(w).to(w.dtype)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return nn.functional.linear(x, self.rotated_weight(), self.base.bias)


def add_oft(model, targets=("q_proj", "k_proj", "v_proj", "o_proj", "gate_proj", "up_proj", "down_proj"),
            block_size: int = 32) -> List[str]:
    """Wraps the matching ``nn.Linear`` layers in ``OFTLinear`` and freezes everything else."""
    for p in model.parameters():
        p.requires_grad_(False)
    wrapped = []
    for name, mod in list(model.named_modules()):
        for child_name, child in list(mod.named_children()):
            if isinstance(child, nn.Linear) and ("all" in targets or child_name in targets) \
                    and child.out_features % block_size == 0 and child_name != "lm_head":
                setattr(mod, child_name, OFTLinear(child, block_size))
                wrapped.append(f"{name}.{child_name}" if name else child_name)
    return wrapped


def merge_oft(model) -> int:
    """Folds every rotation into its base weight and restores the plain ``nn.Linear`` modules."""
    n = 0
    for _, mod in list(model.named_modules()):
        for child_name, child in list(mod.named_children()):
            if isinstance(child, OFTLinear):
                with torch.no_grad():
                    child.base.weight.copy_(child.rotated_weight())
                setattr(mod, child_name, child.base)
                n += 1
    return n


# -- the whole sequence --------------------------------------------------------------------------------------------------------
def patch_model(model, *, vocab_size: Optional[int] = None, resize_vocab: bool = False, upcast_norms: bool = False,
                upcast_logits: bool = False, gradient_checkpointing: bool = True) -> Dict[str, object]:
    """Applies the post-load patches in the reference's order (``model/patcher.py:patch_model``)."""
    done: Dict[str, object] = {}
    if resize_vocab and vocab_size:
        done["vocab_size"] = resize_embedding_layer(model, vocab_size)
    if upcast_norms:
        done["upcast_norms"] = upcast_layernorm(model)
    if upcast_logits:
        upcast_lmhead_output(model)
        done["upcast_logits"] = True
    if gradient_checkpointing and hasattr(model, "gradient_checkpointing_enable"):
        model.gradient_checkpointing_enable()
        done["gradient_checkpointing"] = True
    return done
