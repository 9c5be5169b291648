"""Trainer of the second-generation stack.  One optimizer step consumes a list of micro-batches; each micro-batch's
loss is weighted by its share of the step's valid (non-masked) tokens over ALL data-parallel ranks, so the update
equals that of one large batch whatever the split (reference: ``v1/core/base_trainer.py:164-199``).  Sharding
(``dist``): ``zero2`` = flat AdamW with sharded gradients and states, ``zero3`` = parameters sharded too (the
counterparts of the reference's ``fsdp2`` plugin with and without ``reshard_after_forward``)."""
from __future__ import annotations

import json
import os
from dataclasses import asdict, dataclass
from typing import Dict, List, Optional

import torch
import torch.distributed as dist

from ..train.optimizer import get_lr
from ..train.trainer import Trainer, TrainingArguments
from .batching import IGNORE_INDEX, BatchGenerator


@dataclass
class V1TrainingArguments:
    output_dir: str = "output"
    micro_batch_size: int = 1
    global_batch_size: Optional[int] = None
    cutoff_len: int = 2048
    learning_rate: float = 1e-5
    lr_scheduler: str = "cosine"
    warmup_steps: int = 0
    max_steps: int = 0
    num_train_epochs: int = 1
    max_grad_norm: float = 1.0
    bf16: bool = True
    enable_activation_checkpointing: bool = True
    batching_strategy: str = "normal"
    token_budget: int = 0
    dist: str = "zero2"
    seed: int = 0


def valid_tokens(batches: List[Dict]) -> int:
    """Tokens that contribute to the loss: labels other than the ignore index, after the shift by one."""
    return int(sum((b["labels"][..., 1:] != IGNORE_INDEX).sum() for b in batches))


class SFTTrainerV1:
    def __init__(self, args: V1TrainingArguments, model: torch.nn.Module, renderer, train_dataset,
                 device: Optional[torch.device] = None):
        self.args, self.model, self.renderer = args, model, renderer
        world = dist.get_world_size() if dist.is_initialized() else 1
        rank = dist.get_rank() if dist.is_initialized() else 0
        self.dp_size, self.rank = world, rank
        self.generator = BatchGenerator(train_dataset, renderer, args.micro_batch_size, args.global_batch_size,
                                        args.batching_strategy, args.token_budget, rank, world, args.seed)
        steps = args.max_steps if args.max_steps > 0 else args.num_train_epochs * len(self.generator)
        self.num_training_steps = steps
        inner = TrainingArguments(output_dir="", learning_rate=args.learning_rate, max_steps=steps,
                                  warmup_steps=args.warmup_steps, lr_scheduler_type=args.lr_scheduler,
                                  max_grad_norm=args.max_grad_norm, bf16=args.bf16, pure_bf16=args.bf16,
                                  disable_gradient_checkpointing=not args.enable_activation_checkpointing,
                                  zero_stage=3 if args.dist == "zero3" else 2, logging_steps=0, seed=args.seed)
        self.core = Trainer(model, inner, device=device)
        self.device = self.core.device
        self.global_step = 0
        self.history: List[dict] = []

    def compute_loss(self, batch: Dict) -> torch.Tensor:
        """Sum (not mean) of the token losses of one micro-batch."""
        extra = {"cu_seqlens": batch["cu_seqlens"]} if batch.get("cu_seqlens") is not None else {}
        dev = {k: v.to(self.device, non_blocking=True) for k, v in batch.items() if isinstance(v, torch.Tensor)}
        out = self.model(input_ids=dev["input_ids"], labels=dev["labels"], position_ids=dev.get("position_ids"), **extra)
        return out.loss * max(valid_tokens([batch]), 1)

    def train_step(self, micro_batches: List[Dict]) -> float:
        self.model.train()
        self.core.optimizer.zero_grad()
        total = torch.tensor(float(valid_tokens(micro_batches)), device=self.device)
        if dist.is_initialized() and self.dp_size > 1:
            dist.all_reduce(total)
        denom = float(total) + 1e-6
        step_loss = 0.0
        for mb in micro_batches:
            # the optimizer averages gradients over the ranks, hence the factor dp_size
            loss = self.compute_loss(mb) * (self.dp_size / denom)
            loss.backward()
            step_loss += float(loss.detach()) / self.dp_size
        lr = get_lr(self.args.lr_scheduler, self.global_step, self.args.learning_rate, self.args.warmup_steps,
                    self.num_training_steps)
        self.core.optimizer.step(lr)
        self.global_step += 1
        if dist.is_initialized() and self.dp_size > 1:
            t = torch.tensor(step_loss, device=self.device)
            dist.all_reduce(t)
            step_loss = float(t)
        self.history.append({"step": self.global_step, "loss": step_loss, "lr": lr})
        return step_loss

    def fit(self) -> None:
        start_epoch = self.generator.epoch
        for epoch in range(start_epoch, max(self.args.num_train_epochs, start_epoch + 1)):
            self.generator.set_epoch(epoch)
            for micro_batches in self.generator:
                self.train_step(micro_batches)
                if self.global_step >= self.num_training_steps:
                    return
            if self.args.max_steps <= 0 and epoch + 1 >= self.args.num_train_epochs:
                return

    # -- checkpoints: model + optimizer (through the core trainer) + data position ------------------------------------
    def save_checkpoint(self, path: str) -> None:
        self.core.global_step = self.global_step
        self.core.save_checkpoint(path)
        if self.rank == 0:
            with open(os.path.join(path, "v1_state.json"), "w") as fh:
                json.dump({"global_step": self.global_step, "generator": self.generator.state_dict(),
                           "args": asdict(self.args)}, fh)

    def load_checkpoint(self, path: str) -> None:
        self.core.load_checkpoint(path)
        with open(os.path.join(path, "v1_state.json")) as fh:
            st = json.load(fh)
        self.global_step = st["global_step"]
        self.generator.load_state_dict(st["generator"])

    def save_model(self) -> None:
        from ..utils import checkpoint_io
        if self.rank == 0 or self.args.dist == "zero3":
            checkpoint_io.save_pretrained(self.model, self.args.output_dir)
