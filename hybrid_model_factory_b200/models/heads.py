"""Task heads on top of :class:`HybridModel`: sequence classification, token classification and extractive question
answering, for every model family of the zoo.

Behaviour follows the generic heads the reference attaches to its decoder
(``models/hybrid_qwen3/modeling_hybrid_qwen3.py:1399-1408``, ``transformers.modeling_layers``):

* sequence classification scores the hidden state of the last non-padding token of each row with ``score``
  (``Linear(hidden, num_labels, bias=False)``); the loss follows ``config.problem_type`` (regression: MSE,
  single-label: cross entropy, multi-label: BCE with logits), inferred from ``num_labels`` and the label dtype
  when unset;
* token classification applies dropout and ``score`` (``Linear(hidden, num_labels)``) to every position;
* question answering maps every position to start / end logits (``qa_outputs``) and averages the two cross
  entropies, with out-of-range positions ignored.

The state-dict keys (``model.*``, ``score.*``, ``qa_outputs.*``) are the reference's.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch
import torch.nn as nn
import torch.nn.functional as F

from .configuration import HybridConfig


@dataclass
class HeadOutput:
    loss: Optional[torch.Tensor] = None
    logits: Optional[torch.Tensor] = None
    start_logits: Optional[torch.Tensor] = None
    end_logits: Optional[torch.Tensor] = None
    hidden_states: Optional[torch.Tensor] = None


def last_token_positions(input_ids: torch.Tensor, pad_token_id: Optional[int]) -> torch.Tensor:
    """Index of the last non-padding token of every row (the whole row counts when there is no pad id)."""
    B, T = input_ids.shape
    if pad_token_id is None:
        return torch.full((B,), T - 1, device=input_ids.device, dtype=torch.long)
    real = (input_ids != pad_token_id).long()
    return (real * torch.arange(T, device=input_ids.device)[None]).amax(-1)


class _HeadBase(nn.Module):
    config_class = HybridConfig

    def __init__(self, config: HybridConfig):
        super().__init__()
        from .modeling_hybrid import HybridModel
        self.config = config
        self.num_labels = int(getattr(config, "num_labels", 2) or 2)
        self.model = HybridModel(config)

    def _hidden(self, input_ids, position_ids=None, inputs_embeds=None):
        return self.model(input_ids=input_ids, position_ids=position_ids, inputs_embeds=inputs_embeds)[0]

    def gradient_checkpointing_enable(self, *_, **__):
        self.model.gradient_checkpointing = True


class HybridForSequenceClassification(_HeadBase):
    def __init__(self, config: HybridConfig):
        super().__init__(config)
        self.score = nn.Linear(config.hidden_size, self.num_labels, bias=False)

    def forward(self, input_ids=None, labels=None, position_ids=None, inputs_embeds=None, **_) -> HeadOutput:
        h = self._hidden(input_ids, position_ids, inputs_embeds)
        logits = self.score(h)
        B = logits.shape[0]
        if input_ids is not None:
            last = last_token_positions(input_ids, getattr(self.config, "pad_token_id", None))
        else:
            last = torch.full((B,), logits.shape[1] - 1, device=logits.device, dtype=torch.long)
        pooled = logits[torch.arange(B, device=logits.device), last]
        loss = None
        if labels is not None:
            kind = getattr(self.config, "problem_type", None)
            if kind is None:
                kind = ("regression" if self.num_labels == 1 else
                        "single_label_classification" if labels.dtype in (torch.long, torch.int) else
                        "multi_label_classification")
                self.config.problem_type = kind
            if kind == "regression":
                loss = F.mse_loss(pooled.float().squeeze(-1) if self.num_labels == 1 else pooled.float(),
                                  labels.float().squeeze(-1) if self.num_labels == 1 else labels.float())
            elif kind == "single_label_classification":
                loss = F.cross_entropy(pooled.float().view(-1, self.num_labels), labels.view(-1))
            else:
                loss = F.binary_cross_entropy_with_logits(pooled.float(), labels.float())
        return HeadOutput(loss=loss, logits=pooled, hidden_states=h)


class HybridForTokenClassification(_HeadBase):
    def __init__(self, config: HybridConfig):
        super().__init__(config)
        p = getattr(config, "classifier_dropout", None)
        p = getattr(config, "hidden_dropout", 0.1) if p is None else p
        self.dropout = nn.Dropout(float(p or 0.0))
        self.score = nn.Linear(config.hidden_size, self.num_labels)

    def forward(self, input_ids=None, labels=None, position_ids=None, inputs_embeds=None, **_) -> HeadOutput:
        h = self._hidden(input_ids, position_ids, inputs_embeds)
        logits = self.score(self.dropout(h))
        loss = None
        if labels is not None:
            loss = F.cross_entropy(logits.float().view(-1, self.num_labels), labels.view(-1), ignore_index=-100)
        return HeadOutput(loss=loss, logits=logits, hidden_states=h)


class HybridForQuestionAnswering(_HeadBase):
    def __init__(self, config: HybridConfig):
        super().__init__(config)
        self.qa_outputs = nn.Linear(config.hidden_size, 2)

    def forward(self, input_ids=None, start_positions=None, end_positions=None, position_ids=None,
                inputs_embeds=None, **_) -> HeadOutput:
        h = self._hidden(input_ids, position_ids, inputs_embeds)
        start, end = self.qa_outputs(h).float().unbind(-1)
        loss = None
        if start_positions is not None and end_positions is not None:
            T = start.shape[1]
            sp, ep = start_positions.view(-1).clamp(0, T), end_positions.view(-1).clamp(0, T)
            loss = 0.5 * (F.cross_entropy(start, sp, ignore_index=T) + F.cross_entropy(end, ep, ignore_index=T))
        return HeadOutput(loss=loss, start_logits=start, end_logits=end, hidden_states=h)


HEAD_CLASSES = {"sequence_classification": HybridForSequenceClassification,
                "token_classification": HybridForTokenClassification,
                "question_answering": HybridForQuestionAnswering}


def build_head_model(config: HybridConfig, task: str) -> nn.Module:
    """``task`` in ``sequence_classification | token_classification | question_answering``."""
    from ..ops.gemm import use_own_linear
    if task not in HEAD_CLASSES:
        raise ValueError(f"unknown task {task!r}; choose from {sorted(HEAD_CLASSES)}")
    model = HEAD_CLASSES[task](config)
    use_own_linear(model)
    return model
