"""Stage-1 distillation losses.

``hkd_mse_loss`` is the reference behaviour (``train/hkd/trainer.py:164-338``): the fused two-stream
model carries a student stream (hybrid mixers) and a frozen teacher stream (attention) through the
same norms / MLPs; the loss is an optional per-layer MSE (``decoder | mixer | residuals | all``,
averaged over layers) plus the MSE between the final-norm outputs of both streams
(``hybrid_distill_pre_lm_head``).  No vocabulary projection is evaluated.

``hkd_kl_loss`` distils against the logits of a separate teacher model (KL(teacher || student) over
the vocabulary, computed chunk-wise so the full logit matrix never exists).
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.nn.functional as F
from torch.utils.checkpoint import checkpoint

from ..models.modeling_hybrid import FusedDecoderLayer
from ..parallel.sp import get_sp_context

import torch.distributed as dist


def _sp_mean(loss: torch.Tensor, sp) -> torch.Tensor:
    """Average of per-rank means over the SP group (value only; gradients stay local)."""
    if sp is None or sp.size == 1:
        return loss
    total = loss.detach().clone()
    dist.all_reduce(total, group=sp.group)
    return loss / sp.size + (total / sp.size - loss / sp.size).detach()


def hkd_mse_loss(model, batch, lw_distill_target: Optional[str] = None, distill_pre_lm_head: bool = True) -> torch.Tensor:
    core = model.model
    input_ids = batch["input_ids"]
    h = core.embed_tokens(input_ids)
    B, T = h.shape[0], h.shape[1]
    position_ids = batch.get("position_ids")
    if position_ids is None:
        position_ids = torch.arange(T, device=h.device).expand(B, T)
    cos, sin = core.rotary_emb(position_ids)
    pos_emb = (cos.to(h.dtype), sin.to(h.dtype))
    hs, ha = h, h
    mse = h.new_zeros((), dtype=torch.float32)
    use_ckpt = core.gradient_checkpointing and model.training
    for layer in core.layers:
        if isinstance(layer, FusedDecoderLayer):
            if use_ckpt:
                outs = checkpoint(layer, hs, ha, pos_emb, position_ids, use_reentrant=False)
            else:
                outs = layer(hs, ha, position_embeddings=pos_emb, position_ids=position_ids)
            hs, ha, s_mix, t_mix, s_mlp, t_mlp = outs
        else:
            # plain layers are shared by both streams
            hs = layer(hs, position_embeddings=pos_emb, position_ids=position_ids)[0]
            with torch.no_grad():
                ha = layer(ha, position_embeddings=pos_emb, position_ids=position_ids)[0]
            s_mix = t_mix = s_mlp = t_mlp = None
        if lw_distill_target and s_mix is not None:
            if lw_distill_target in ("decoder", "all"):
                mse = mse + F.mse_loss(hs.float(), ha.float())
            if lw_distill_target in ("mixer", "residuals", "all"):
                mse = mse + F.mse_loss(s_mix.float(), t_mix.float())
            if lw_distill_target in ("residuals", "all"):
                mse = mse + F.mse_loss(s_mlp.float(), t_mlp.float())
    mse = mse / len(core.layers)
    if distill_pre_lm_head:
        mse = mse + F.mse_loss(core.norm(hs).float(), core.norm(ha).float())
    return _sp_mean(mse, model.sequence_parallel_group)


def hkd_kl_loss(student, teacher, batch, chunk: int = 2048, temperature: float = 1.0) -> torch.Tensor:
    """KL between teacher and student next-token distributions, averaged over tokens."""
    pos = batch.get("position_ids")
    hs = student.model(batch["input_ids"], position_ids=pos)[0]
    with torch.no_grad():
        ht = teacher.model(batch["input_ids"], position_ids=pos)[0]
    hs2, ht2 = hs.reshape(-1, hs.shape[-1]), ht.reshape(-1, ht.shape[-1])
    total = hs.new_zeros((), dtype=torch.float32)

    def piece(a, b):
        ls = F.log_softmax(student.lm_head(a).float() / temperature, dim=-1)
        with torch.no_grad():
            lt = F.log_softmax(teacher.lm_head(b).float() / temperature, dim=-1)
        return F.kl_div(ls, lt, log_target=True, reduction="sum")

    for s in range(0, hs2.shape[0], chunk):
        total = total + checkpoint(piece, hs2[s:s + chunk], ht2[s:s + chunk], use_reentrant=False)
    loss = total / hs2.shape[0] * (temperature ** 2)
    return _sp_mean(loss, student.sequence_parallel_group)


def freeze_params_hybrid(model, learnable: Optional[str]) -> int:
    """Only parameters whose name contains one of the comma-separated substrings stay trainable
    (reference: ``train/trainer_utils.py:955-1001``).  Returns the number of trainable parameters."""
    if not learnable:
        return sum(p.numel() for p in model.parameters() if p.requires_grad)
    keys = [k.strip() for k in learnable.split(",") if k.strip()]
    n = 0
    for name, p in model.named_parameters():
        p.requires_grad_(any(k in name for k in keys))
        if p.requires_grad:
            n += p.numel()
    if n == 0:
        raise ValueError(f"hybrid_learnable_params='{learnable}' matches no parameter")
    return n
