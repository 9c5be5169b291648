"""Training loop (own loop, no HF Trainer): bf16 parameters in a flat buffer, fused AdamW with
ZeRO sharding over all ranks, sequence-parallel loss reduction, per-layer activation
checkpointing, gradient accumulation, LR schedules, jsonl progress log, checkpoint save/resume.

One optimizer step over a batch is ``Trainer.train_step(batch)``: the batch is a dict of CPU
tensors (ideally pinned) holding this rank's shard (``input_ids``, ``labels``, ``position_ids``);
the method copies it to the device, runs forward/backward (micro-batches when
``gradient_accumulation_steps > 1``), steps the optimizer and returns the loss as a device tensor.

Reference behaviour: ``train/pt/trainer.py:46-195`` (SP sampler + loss), ``train/tuner.py:58-99``,
``train/trainer_utils.py:80-122`` (sharded save), ``train/callbacks.py:267-355`` (progress log).
"""
from __future__ import annotations

import json
import os
import time
from dataclasses import asdict, dataclass, field
from typing import Callable, Dict, Iterable, Optional

import torch
import torch.distributed as dist

from ..parallel.sp import SPContext, init_sp_group, set_sequence_parallel_group_recursive
from .optimizer import FlatAdamW, get_lr


@dataclass
class TrainingArguments:
    output_dir: str = "output"
    learning_rate: float = 1e-5
    weight_decay: float = 0.0
    adam_beta1: float = 0.9
    adam_beta2: float = 0.999
    adam_epsilon: float = 1e-8
    max_grad_norm: float = 1.0
    lr_scheduler_type: str = "cosine"
    warmup_steps: int = 0
    max_steps: int = 100
    per_device_train_batch_size: int = 1
    gradient_accumulation_steps: int = 1
    sequence_parallel_size: int = 1
    sequence_parallel_mode: str = "zigzag-ring"
    bf16: bool = True
    pure_bf16: bool = True
    disable_gradient_checkpointing: bool = False
    logging_steps: int = 1
    save_steps: int = 0
    eval_steps: int = 0                   # evaluate on the held-out batches every N steps (and at the end of training)
    save_only_model: bool = False
    save_max_shard_size: str = "5GB"
    seed: int = 42
    resume_from_checkpoint: Optional[str] = None
    optimizer_state_dtype: str = "auto"   # auto = parameter dtype (bf16 under pure_bf16), or float32
    master_weights: bool = False
    ddp_timeout: int = 1800
    optimizer: str = "adamw"              # adamw (flat, ZeRO-sharded, fused kernel) | muon | galore | apollo |
    #                                       badam | adam_mini | loraplus (train/memory_optimizers.py)
    optimizer_args: dict = field(default_factory=dict)
    zero_stage: int = 2                   # 2: flat AdamW with sharded states / gradients; 3: parameters sharded too
    offload_optimizer: bool = False       # ZeRO-3 only: moments and master weights in pinned host memory
    offload_checkpoints: bool = False     # checkpointed layer inputs wait in pinned host memory until the backward pass
    mics_shard_size: int = 0              # ZeRO-3 only: shard inside groups of this many ranks, replicate across them
    recompute_budget: str = "auto"        # auto: after the first step, layers whose activations fit in the free device
    #                                       memory stop being checkpointed (no second forward for them); off: every
    #                                       layer stays checkpointed; a number: fraction of the device memory to fill

    def to_dict(self):
        return asdict(self)


class Trainer:
    def __init__(self, model: torch.nn.Module, args: TrainingArguments, device: Optional[torch.device] = None,
                 loss_fn: Optional[Callable] = None, trainable: Optional[Iterable[torch.nn.Parameter]] = None,
                 callbacks: Optional[list] = None):
        self.model, self.args = model, args
        self.device = device or next(model.parameters()).device
        self.loss_fn = loss_fn
        self.callbacks = callbacks or []
        self.world = dist.get_world_size() if dist.is_initialized() else 1
        self.rank = dist.get_rank() if dist.is_initialized() else 0
        sp_size = max(1, args.sequence_parallel_size)
        self.sp: Optional[SPContext] = init_sp_group(sp_size) if (sp_size > 1 and dist.is_initialized()) else None
        if self.sp is not None and "ulysses" in (args.sequence_parallel_mode or ""):
            self.sp.mode = "ulysses"        # attention layers exchange heads instead of gathering K/V
        if self.sp is not None and torch.cuda.is_available() and os.environ.get("HMF_SP_PEER", "1") == "1":
            # recurrent states travel from inside the scan kernels over peer memory (NCCL send/recv otherwise)
            from ..parallel.peer import enable_peer_kv, enable_peer_transport
            enable_peer_transport(self.sp)
            # Opt-in: the attention forward can pull remote K/V tiles itself (no all-gather).  Every query tile then
            # re-reads its remote tiles over NVLink, which only pays for short contexts; measured 6x slower than the
            # NCCL gather at 128K tokens over 2 GPUs, so the default stays off.
            kv_bytes = int(os.environ.get("HMF_SP_PEER_KV_MB", "0")) << 20
            if kv_bytes > 0 and self.sp.mode != "ulysses":
                enable_peer_kv(self.sp, kv_bytes)
        set_sequence_parallel_group_recursive(model, self.sp)
        self.dp_size = self.world // sp_size
        if not args.disable_gradient_checkpointing and hasattr(model, "gradient_checkpointing_enable"):
            model.gradient_checkpointing_enable()
            if args.offload_checkpoints:
                from ..utils.checkpointing import set_offload
                set_offload(True)
        params = list(trainable) if trainable is not None else [p for p in model.parameters() if p.requires_grad]
        sdt = None if args.optimizer_state_dtype == "auto" else getattr(torch, args.optimizer_state_dtype)
        if args.zero_stage == 3:
            from .zero3 import Zero3Engine, mics_groups
            groups = {}
            if args.mics_shard_size and dist.is_initialized() and args.mics_shard_size < self.world:
                shard_group, replica_group = mics_groups(args.mics_shard_size)
                groups = dict(group=shard_group, replica_group=replica_group)
            self.optimizer = Zero3Engine(model, **groups, lr=args.learning_rate, betas=(args.adam_beta1, args.adam_beta2),
                                         eps=args.adam_epsilon, weight_decay=args.weight_decay,
                                         max_grad_norm=args.max_grad_norm, dp_size=self.dp_size,
                                         offload_optimizer=args.offload_optimizer)
        elif args.optimizer == "muon":
            from .muon import Muon
            ids = {id(p) for p in params}
            self.optimizer = Muon([(n, p) for n, p in model.named_parameters() if id(p) in ids], lr=args.learning_rate,
                                  betas=(args.adam_beta1, args.adam_beta2), eps=args.adam_epsilon,
                                  weight_decay=args.weight_decay, max_grad_norm=args.max_grad_norm, dp_size=self.dp_size)
        elif args.optimizer in ("galore", "apollo", "badam", "adam_mini", "loraplus"):
            from .memory_optimizers import build_optimizer
            self.optimizer = build_optimizer(args.optimizer, model, args.learning_rate, trainable=params,
                                             betas=(args.adam_beta1, args.adam_beta2), eps=args.adam_epsilon,
                                             weight_decay=args.weight_decay, max_grad_norm=args.max_grad_norm,
                                             dp_size=self.dp_size, **args.optimizer_args)
        else:
            self.optimizer = FlatAdamW(params, lr=args.learning_rate, betas=(args.adam_beta1, args.adam_beta2),
                                       eps=args.adam_epsilon, weight_decay=args.weight_decay,
                                       max_grad_norm=args.max_grad_norm, group=None, dp_size=self.dp_size,
                                       state_dtype=sdt, master_weights=args.master_weights)
        self.global_step = 0
        self._recompute_planned = False
        self.unchecked_layers: list = []
        self.status_check_steps = 50
        self.tokens_seen = 0
        self._t0 = time.time()
        self._log_file = None
        if self.rank == 0 and args.output_dir:
            os.makedirs(args.output_dir, exist_ok=True)
            self._log_file = os.path.join(args.output_dir, "trainer_log.jsonl")
        if args.resume_from_checkpoint:
            self.load_checkpoint(args.resume_from_checkpoint)

    # -- one optimizer step -----------------------------------------------------------------
    def _to_device(self, batch: Dict[str, torch.Tensor]) -> Dict[str, torch.Tensor]:
        return {k: (v.to(self.device, non_blocking=True) if isinstance(v, torch.Tensor) else v) for k, v in batch.items()}

    def compute_loss(self, batch: Dict[str, torch.Tensor]) -> torch.Tensor:
        if self.loss_fn is not None:
            return self.loss_fn(self.model, batch)
        extra = {"cu_seqlens": batch["cu_seqlens"]} if batch.get("cu_seqlens") is not None else {}
        out = self.model(input_ids=batch["input_ids"], labels=batch["labels"], position_ids=batch.get("position_ids"),
                         labels_shifted=bool(batch.get("labels_shifted", self.sp is not None)), **extra)
        return out.loss

    # -- which layers need no second forward ---------------------------------------------------------
    def _core_with_layers(self):
        for m in self.model.modules():
            if hasattr(m, "checkpoint_skip") and hasattr(m, "layers"):
                return m
        return None

    def _probe_wanted(self) -> bool:
        core = self._core_with_layers()
        return (not self._recompute_planned and str(self.args.recompute_budget) != "off" and core is not None
                and getattr(core, "gradient_checkpointing", False) and self.device.type == "cuda"
                and not self.args.offload_checkpoints)

    def plan_recompute(self, sizes: dict, total_bytes: int, peak_bytes: int) -> list:
        """Chooses the layers that run WITHOUT activation checkpointing from now on.  ``sizes``: bytes each layer's
        autograd graph held during the first (fully checkpointed) step; ``peak_bytes``: that step's peak of live
        memory.  The activations of the chosen layers must fit in what the step left free, with a margin for the
        allocator's fragmentation; sharding over more ranks frees memory, so more layers qualify and the step loses
        their second forward.  Every rank takes the same decision (smallest budget, largest sizes): a layer that one
        rank re-runs and another does not would issue its collectives a different number of times."""
        from ..utils.checkpointing import choose_unchecked_layers
        frac = 0.90 if str(self.args.recompute_budget) == "auto" else float(self.args.recompute_budget)
        budget = (frac * total_bytes - peak_bytes) * 0.8
        keys = sorted(sizes)
        if dist.is_initialized() and self.world > 1 and keys:
            t = torch.tensor([-budget] + [float(sizes[k]) for k in keys], device=self.device, dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            budget = -float(t[0])
            sizes = {k: float(v) for k, v in zip(keys, t[1:].tolist())}
        chosen = choose_unchecked_layers(sizes, budget)
        core = self._core_with_layers()
        if core is not None:
            core.checkpoint_skip = frozenset(chosen)
        self.unchecked_layers = chosen
        self._recompute_planned = True
        return chosen

    def train_step(self, batch: Dict[str, torch.Tensor]) -> torch.Tensor:
        self.model.train()
        probing = self._probe_wanted()
        if probing:
            from ..utils import checkpointing
            torch.cuda.reset_peak_memory_stats(self.device)
            checkpointing.start_probe()
        ga = max(1, self.args.gradient_accumulation_steps)
        self.optimizer.zero_grad()
        dev = self._to_device(batch)
        total = None
        # preference batches carry chosen_* / rejected_* tensors instead of input_ids
        first = dev["input_ids"] if "input_ids" in dev else next(v for v in dev.values() if isinstance(v, torch.Tensor)
                                                                   and v.dim() > 0)
        bsz = first.shape[0]
        micro = max(1, bsz // ga)
        for i in range(0, bsz, micro):
            mb = {k: (v[i:i + micro] if isinstance(v, torch.Tensor) and v.dim() > 0 and v.shape[0] == bsz else v)
                  for k, v in dev.items()}
            if isinstance(mb.get("cu_seqlens"), list) and micro == 1 and len(mb["cu_seqlens"]) == bsz:
                mb["cu_seqlens"] = [mb["cu_seqlens"][i]]
            loss = self.compute_loss(mb) * (micro / bsz)
            loss.backward()
            total = loss.detach() if total is None else total + loss.detach()
        lr = get_lr(self.args.lr_scheduler_type, self.global_step, self.args.learning_rate, self.args.warmup_steps,
                    self.args.max_steps)
        self.optimizer.step(lr)
        if probing:
            sizes = checkpointing.stop_probe()
            if self.plan_recompute(sizes, torch.cuda.mem_get_info(self.device)[1],
                                   torch.cuda.max_memory_allocated(self.device)):
                torch.cuda.empty_cache()        # the cached blocks were shaped by the fully checkpointed step
        self.global_step += 1
        self.tokens_seen += sum(int(v.numel()) for k, v in dev.items()
                                if isinstance(v, torch.Tensor) and k.endswith("input_ids")) * self.world
        self._last_lr = lr
        return total

    # -- device-side wait status -----------------------------------------------------------------
    def check_kernel_status(self, status_reader: Optional[Callable] = None) -> None:
        """Raises ``KernelError`` on every rank when any rank's kernels recorded a wait that ran out (a late or
        missing peer in the in-kernel state chain, an mbarrier that never completed).  Such a kernel returns and the
        step goes on with stale data, so the record must be read: here at logging steps, before every checkpoint
        and every ``status_check_steps`` steps (one small device-to-host read and, with several ranks, one
        all-reduce)."""
        from ..ops import _lib
        if status_reader is None:
            if not (torch.cuda.is_available() and self.device.type == "cuda" and _lib.kernels_available()):
                return
            status_reader = _lib.read_status
        code, block, detail, count = status_reader()
        worst = int(code)
        if dist.is_initialized() and self.world > 1:
            t = torch.tensor([worst], device=self.device)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            worst = int(t)
        if worst != 0:
            raise _lib.KernelError(
                f"step {self.global_step}: a device-side wait ran out on at least one rank (this rank: code={code} "
                f"block={block} detail={detail:#x} count={count}); the results of the steps since the last check are "
                f"not valid.  With sequence parallelism, HMF_SP_PEER=0 selects the NCCL state transport.")

    # -- evaluation -----------------------------------------------------------------------------
    @torch.no_grad()
    def evaluate(self, batches: Iterable[Dict[str, torch.Tensor]]) -> float:
        """Mean loss over ``batches`` (every rank evaluates its own share; the mean is taken over all ranks)."""
        was_training = self.model.training
        self.model.eval()
        total, n = 0.0, 0
        for batch in batches:
            total += float(self.compute_loss(self._to_device(batch)))
            n += 1
        self.model.train(was_training)
        if dist.is_initialized() and self.world > 1:
            t = torch.tensor([total, float(n)], device=self.device, dtype=torch.float64)
            dist.all_reduce(t)
            total, n = float(t[0]), int(t[1])
        return total / max(n, 1)

    def _maybe_evaluate(self, force: bool = False) -> None:
        fn = getattr(self, "eval_batches_fn", None)
        if fn is None:
            return
        if force or (self.args.eval_steps and self.global_step % self.args.eval_steps == 0):
            self.last_eval_loss = self.evaluate(fn())
            self.log({"eval_loss": self.last_eval_loss})

    # -- loop ---------------------------------------------------------------------------------
    def train(self, batches: Iterable[Dict[str, torch.Tensor]]) -> None:
        for batch in batches:
            if self.global_step >= self.args.max_steps:
                break
            loss = self.train_step(batch)
            logging_now = bool(self.args.logging_steps and self.global_step % self.args.logging_steps == 0)
            if logging_now or self.global_step % self.status_check_steps == 0:
                self.check_kernel_status()
            if logging_now:
                self._last_loss = float(loss.item())
                self.log({"loss": self._last_loss, "lr": self._last_lr})
            self._maybe_evaluate()
            if self.args.save_steps and self.global_step % self.args.save_steps == 0:
                self.save_checkpoint(os.path.join(self.args.output_dir, f"checkpoint-{self.global_step}"))
            for cb in self.callbacks:           # after the save, so that a callback finds this step's checkpoint
                cb(self)
        if self.args.eval_steps == 0 or self.global_step % max(self.args.eval_steps, 1) != 0:
            self._maybe_evaluate(force=True)
        for cb in self.callbacks:
            if hasattr(cb, "on_train_end"):
                cb.on_train_end(self)

    def log(self, values: dict) -> None:
        elapsed = time.time() - self._t0
        rec = {"current_steps": self.global_step, "total_steps": self.args.max_steps, "elapsed_time": round(elapsed, 2),
               "throughput": round(self.tokens_seen / max(elapsed, 1e-9), 2), **values}
        if os.environ.get("RECORD_VRAM", "0") == "1" and torch.cuda.is_available():
            rec["vram_reserved_gb"] = round(torch.cuda.max_memory_reserved() / 2 ** 30, 2)
        if self.rank == 0 and self._log_file:
            with open(self._log_file, "a") as f:
                f.write(json.dumps(rec) + "\n")

    # -- checkpoints --------------------------------------------------------------------------
    def save_checkpoint(self, path: str) -> None:
        from ..utils.checkpoint_io import save_pretrained
        self.check_kernel_status()          # never write weights that a timed-out wait may have corrupted
        zero3 = hasattr(self.optimizer, "gather_full_state")
        if zero3:                       # every rank takes part in the all-gathers
            self.optimizer.gather_full_state()
        if self.rank == 0:
            save_pretrained(self.model, path, max_shard_size=self.args.save_max_shard_size)
            with open(os.path.join(path, "trainer_state.json"), "w") as f:
                json.dump({"global_step": self.global_step, "tokens_seen": self.tokens_seen,
                           "args": self.args.to_dict()}, f, indent=2)
        if zero3:
            self.optimizer.release_all()
        if not self.args.save_only_model:
            os.makedirs(path, exist_ok=True)
            torch.save(self.optimizer.state_dict(), os.path.join(path, f"optimizer_rank{self.rank:05d}.pt"))
        if dist.is_initialized():
            dist.barrier()

    def load_checkpoint(self, path: str) -> None:
        """Restores weights, step counters and (when present) this rank's optimizer shard.

        Under ZeRO-3 the parameters are released to empty placeholders: the per-rank optimizer file carries the
        weight shards, and a model-only checkpoint is loaded into the gathered parameters and re-sliced.  A parameter
        that the checkpoint does not hold is an error (a LoRA- or OFT-wrapped model resumed as a plain one, or the
        reverse, would otherwise continue from random weights)."""
        from ..utils.checkpoint_io import load_state_dict_into
        zero3 = hasattr(self.optimizer, "gather_full_state")
        opt = os.path.join(path, f"optimizer_rank{self.rank:05d}.pt")
        has_opt = os.path.exists(opt)
        if not (zero3 and has_opt):
            if zero3:
                self.optimizer.gather_full_state()
            missing, unexpected = load_state_dict_into(self.model, path)
            if zero3:
                self.optimizer.reshard_from_full()
                self.optimizer.release_all()
            if missing:
                raise KeyError(f"{path}: {len(missing)} model parameters are not in the checkpoint "
                               f"(first: {missing[:6]})")
            if unexpected and self.rank == 0:
                import warnings
                warnings.warn(f"{path}: {len(unexpected)} checkpoint tensors match no model parameter "
                              f"(first: {unexpected[:6]})")
        st = os.path.join(path, "trainer_state.json")
        if os.path.exists(st):
            with open(st) as f:
                s = json.load(f)
            self.global_step, self.tokens_seen = int(s["global_step"]), int(s["tokens_seen"])
        if has_opt:
            self.optimizer.load_state_dict(torch.load(opt, map_location=self.device))


def get_last_checkpoint(output_dir: str) -> Optional[str]:
    """Latest ``checkpoint-<step>`` directory (auto-resume, reference: ``hparams/parser.py:383-399``)."""
    if not os.path.isdir(output_dir):
        return None
    best, best_step = None, -1
    for name in os.listdir(output_dir):
        if name.startswith("checkpoint-") and name.split("-")[-1].isdigit():
            s = int(name.split("-")[-1])
            if s > best_step:
                best, best_step = os.path.join(output_dir, name), s
    return best
