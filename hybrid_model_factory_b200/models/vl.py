"""Vision-language wrapper around a hybrid text backbone (Hybrid Qwen2.5-VL).

``HybridVLForConditionalGeneration`` = vision tower + hybrid decoder + ``lm_head``:
image features are written over the embeddings of the ``image_token_id`` placeholders, and multi-axis MRoPE
position ids ``[3|4, B, T]`` are collapsed to the temporal axis before the 1-D-RoPE text model sees them (exact
for text tokens, an approximation for vision tokens).  Reference:
``models/hybrid_qwen2_5_vl/modeling_hybrid_qwen2_5_vl.py:44-131``.

The vision tower is any module mapping ``(pixel_values, grid_thw) -> [n_image_tokens, hidden]``; when
``transformers`` provides the Qwen2.5-VL vision transformer and the config carries a ``vision_config`` it is
built from that, so released towers load unchanged.
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.nn as nn

from .configuration import HybridConfig
from .modeling_hybrid import HybridForCausalLM, build_model


def collapse_mrope_position_ids(position_ids: Optional[torch.Tensor]) -> Optional[torch.Tensor]:
    if position_ids is not None and position_ids.dim() == 3 and position_ids.shape[0] in (3, 4):
        return position_ids[0]
    return position_ids


def build_vision_tower(vision_config) -> Optional[nn.Module]:
    if vision_config is None:
        return None
    try:
        from transformers.models.qwen2_5_vl.configuration_qwen2_5_vl import Qwen2_5_VLVisionConfig
        from transformers.models.qwen2_5_vl.modeling_qwen2_5_vl import Qwen2_5_VisionTransformerPretrainedModel
        cfg = vision_config if not isinstance(vision_config, dict) else Qwen2_5_VLVisionConfig(**vision_config)
        return Qwen2_5_VisionTransformerPretrainedModel._from_config(cfg)
    except Exception:
        return None


class HybridVLForConditionalGeneration(nn.Module):
    model_type = "hybrid_qwen2_5_vl"

    def __init__(self, text_config: HybridConfig, vision_tower: Optional[nn.Module] = None, vision_config=None,
                 image_token_id: int = 151655, video_token_id: int = 151656):
        super().__init__()
        self.config = text_config
        self.language_model: HybridForCausalLM = build_model(text_config)
        self.visual = vision_tower if vision_tower is not None else build_vision_tower(vision_config)
        self.image_token_id, self.video_token_id = image_token_id, video_token_id

    @property
    def lm_head(self):
        return self.language_model.lm_head

    def merge_embeddings(self, input_ids, pixel_values=None, image_grid_thw=None, image_embeds=None):
        emb = self.language_model.model.embed_tokens(input_ids)
        if image_embeds is None and pixel_values is not None:
            if self.visual is None:
                raise ValueError("pixel_values given but the model has no vision tower")
            image_embeds = self.visual(pixel_values, grid_thw=image_grid_thw) if image_grid_thw is not None \
                else self.visual(pixel_values)
            if hasattr(image_embeds, "pooler_output"):      # transformers returns an output object
                image_embeds = image_embeds.pooler_output
        if image_embeds is not None:
            mask = (input_ids == self.image_token_id) | (input_ids == self.video_token_id)
            n = int(mask.sum())
            if n != image_embeds.shape[0]:
                raise ValueError(f"{n} image placeholder tokens but {image_embeds.shape[0]} image features")
            emb = emb.masked_scatter(mask[..., None], image_embeds.to(emb.dtype))
        return emb

    def forward(self, input_ids, labels=None, position_ids=None, pixel_values=None, image_grid_thw=None,
                image_embeds=None, **kw):
        emb = self.merge_embeddings(input_ids, pixel_values, image_grid_thw, image_embeds)
        return self.language_model(None, inputs_embeds=emb, labels=labels,
                                   position_ids=collapse_mrope_position_ids(position_ids), **kw)


def apply_vl_freezing(model: nn.Module, freeze_vision_tower: bool = True, freeze_multi_modal_projector: bool = True,
                      freeze_language_model: bool = False) -> dict:
    """Which parts of a vision-language model train: the vision tower, the projector that maps its features into the
    language model's space (``visual.merger`` in the Qwen2-VL family, else a module named ``*projector*``) and the
    language model.  Returns the trainable parameter count per part.  Reference: ``model/model_utils/visual.py``
    (``freeze_vision_tower`` / ``freeze_multi_modal_projector`` / ``freeze_language_model``)."""
    visual = getattr(model, "visual", None)
    counts = {"vision_tower": 0, "projector": 0, "language_model": 0}
    proj_ids = set()
    if visual is not None:
        for name, mod in visual.named_modules():
            if name == "merger" or "projector" in name.split(".")[-1]:
                proj_ids |= {id(p) for p in mod.parameters()}
        for p in visual.parameters():
            part = "projector" if id(p) in proj_ids else "vision_tower"
            p.requires_grad_(not (freeze_multi_modal_projector if part == "projector" else freeze_vision_tower))
            counts[part] += p.numel() if p.requires_grad else 0
    lm = getattr(model, "language_model", None)
    if lm is not None:
        for p in lm.parameters():
            if freeze_language_model:
                p.requires_grad_(False)
            counts["language_model"] += p.numel() if p.requires_grad else 0
    return counts
