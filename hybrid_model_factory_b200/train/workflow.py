"""Training workflows: ``run_exp`` reads the configuration and dispatches on ``stage``.

  * ``pt``  : next-token pre-training / continued pre-training (stage 2 of priming, long context + SP)
  * ``sft`` : supervised fine-tuning (prompt tokens masked)
  * ``hkd`` : stage-1 distillation of a fused model (hidden-state MSE; optional logit KL to a teacher)
  * ``dpo`` / ``kto`` / ``rm`` : preference objectives on top of the same loop (``train/preference.py``)

Reference: ``train/tuner.py:58-112``, ``train/pt/workflow.py:41-127``, ``train/hkd/workflow.py:47-139``.
"""
from __future__ import annotations

import json
import os
from typing import Any, Optional

import torch
import torch.distributed as dist

from ..config.parser import get_train_args
from ..data.formats import load_tokenizer
from ..data.loader import batch_iterator, get_dataset
from ..models.configuration import HybridConfig
from ..models.modeling_hybrid import build_model
from ..utils import checkpoint_io
from ..utils.logging import get_logger, info_rank0
from .hkd import freeze_params_hybrid, hkd_kl_loss, hkd_mse_loss
from .trainer import Trainer, TrainingArguments

logger = get_logger(__name__)


def _device() -> torch.device:
    if torch.cuda.is_available():
        local = int(os.environ.get("LOCAL_RANK", "0"))
        torch.cuda.set_device(local)
        return torch.device("cuda", local)
    return torch.device("cpu")


def init_distributed(timeout_s: int = 1800) -> None:
    if dist.is_initialized() or int(os.environ.get("WORLD_SIZE", "1")) <= 1:
        return
    import datetime
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    backend = "nccl" if torch.cuda.is_available() else "gloo"
    dist.init_process_group(backend, timeout=datetime.timedelta(seconds=min(timeout_s, 7 * 24 * 3600)))


def load_model(model_args, run_args, device: torch.device):
    """Config (+ dotted overrides) -> model -> weights -> dtype/device (reference: ``model/loader.py:194-335``)."""
    path = model_args.model_name_or_path
    overrides = model_args.config_overrides()
    dtype = torch.bfloat16 if run_args.bf16 else torch.float32
    if path and os.path.isdir(path) and os.path.exists(os.path.join(path, "config.json")):
        cfg = HybridConfig.from_pretrained(path)
        cfg.apply_overrides(overrides)
        if getattr(model_args, "rope_scaling", None):
            from .patcher import configure_rope_scaling
            configure_rope_scaling(cfg, model_args.rope_scaling, getattr(model_args, "model_max_length", None))
        model = build_model(cfg).to(dtype)
        if checkpoint_io.checkpoint_files(path):
            missing, unexpected = checkpoint_io.load_state_dict_into(model, path)
            if missing:
                logger.warning("load_model: %d tensors missing in the checkpoint (e.g. %s)", len(missing), missing[:4])
    else:
        raw = json.loads(path) if path and path.strip().startswith("{") else (overrides or {})
        cfg = HybridConfig.from_dict(dict(raw))
        model = build_model(cfg).to(dtype)
    return model.to(device)


def to_trainer_args(model_args, data_args, run_args, n_batches: Optional[int]) -> TrainingArguments:
    max_steps = run_args.max_steps
    if max_steps is None or max_steps < 0:
        max_steps = int((n_batches or 0) * run_args.num_train_epochs)
    warmup = run_args.warmup_steps or int(run_args.warmup_ratio * max_steps)
    return TrainingArguments(
        output_dir=run_args.output_dir, learning_rate=run_args.learning_rate, weight_decay=run_args.weight_decay,
        adam_beta1=run_args.adam_beta1, adam_beta2=run_args.adam_beta2, adam_epsilon=run_args.adam_epsilon,
        max_grad_norm=run_args.max_grad_norm, lr_scheduler_type=run_args.lr_scheduler_type, warmup_steps=warmup,
        max_steps=max_steps, per_device_train_batch_size=run_args.per_device_train_batch_size,
        gradient_accumulation_steps=run_args.gradient_accumulation_steps,
        sequence_parallel_size=model_args.sequence_parallel_size, sequence_parallel_mode=model_args.sequence_parallel_mode,
        bf16=run_args.bf16, pure_bf16=run_args.pure_bf16,
        disable_gradient_checkpointing=run_args.disable_gradient_checkpointing,
        recompute_budget=str(run_args.recompute_budget), logging_steps=run_args.logging_steps,
        save_steps=run_args.save_steps, eval_steps=run_args.eval_steps, save_only_model=run_args.save_only_model,
        save_max_shard_size=run_args.save_max_shard_size, seed=run_args.seed,
        resume_from_checkpoint=run_args.resume_from_checkpoint, ddp_timeout=run_args.ddp_timeout,
        **zero_config(run_args.deepspeed))


def zero_config(path: Optional[str]) -> dict:
    """Reads the ZeRO stage and the optimizer offload switch from a DeepSpeed-style JSON
    (``zero_optimization.stage``, ``zero_optimization.offload_optimizer.device``); other keys are ignored."""
    if not path:
        return {}
    import json
    with open(path) as f:
        z = json.load(f).get("zero_optimization", {})
    stage = int(z.get("stage", 2))
    off = str(z.get("offload_optimizer", {}).get("device", "none")).lower() in ("cpu", "nvme")
    out = {"zero_stage": 3 if stage >= 3 else 2, "offload_optimizer": off and stage >= 3}
    if stage >= 3 and int(z.get("mics_shard_size", 0) or 0) > 0:
        out["mics_shard_size"] = int(z["mics_shard_size"])
    return out


def select_optimizer(ft_args, default: str = "adamw"):
    """Maps the ``use_*`` switches of the fine-tuning arguments to ``(optimizer name, optimizer kwargs)``
    (reference: ``train/trainer_utils.py:257-605``; at most one of GaLore / APOLLO / BAdam may be set)."""
    chosen = [k for k in ("galore", "apollo", "badam") if getattr(ft_args, f"use_{k}", False)]
    if len(chosen) > 1:
        raise ValueError("use_galore, use_apollo and use_badam exclude one another")
    if chosen and ft_args.finetuning_type == "lora":
        raise ValueError("GaLore / APOLLO / BAdam train full weights, not LoRA adapters")
    if chosen == ["galore"]:
        return "galore", dict(rank=ft_args.galore_rank, update_interval=ft_args.galore_update_interval,
                              scale=ft_args.galore_scale, proj_type=ft_args.galore_proj_type,
                              targets=tuple(t.strip() for t in ft_args.galore_target.split(",")))
    if chosen == ["apollo"]:
        return "apollo", dict(rank=ft_args.apollo_rank, update_interval=ft_args.apollo_update_interval,
                              scale=ft_args.apollo_scale, proj=ft_args.apollo_proj, proj_type=ft_args.apollo_proj_type,
                              scale_type=ft_args.apollo_scale_type,
                              targets=tuple(t.strip() for t in ft_args.apollo_target.split(",")))
    if chosen == ["badam"]:
        return "badam", dict(mode=ft_args.badam_mode, switch_mode=ft_args.badam_switch_mode,
                             switch_interval=ft_args.badam_switch_interval, start_block=ft_args.badam_start_block,
                             update_ratio=ft_args.badam_update_ratio, mask_mode=ft_args.badam_mask_mode)
    if getattr(ft_args, "use_adam_mini", False):
        return "adam_mini", {}
    if getattr(ft_args, "loraplus_lr_ratio", None) is not None:
        if ft_args.finetuning_type != "lora":
            raise ValueError("loraplus_lr_ratio is only valid for LoRA training")
        return "loraplus", dict(lr_ratio=ft_args.loraplus_lr_ratio, lr_embedding=ft_args.loraplus_lr_embedding)
    return default, {}


def build_callbacks(run_args, model_args=None) -> list:
    """Callbacks of a run: stop on a non-finite loss; ``report_to`` tensorboard (own event-file writer), wandb or
    swanlab (when importable); the base tokenizer's files re-copied into every checkpoint."""
    from .callbacks import EarlyStopCallback, PreserveTokenizerConfigCallback, ReporterCallback
    cbs = [EarlyStopCallback()]
    targets = {t.strip() for t in str(getattr(run_args, "report_to", "none") or "none").split(",")}
    if targets & {"tensorboard", "all"}:
        from ..utils.tensorboard_writer import TensorBoardCallback
        cbs.append(TensorBoardCallback(run_args.output_dir))
    for backend in ("wandb", "swanlab"):
        if targets & {backend, "all"}:
            cbs.append(ReporterCallback(backend=backend))
    src = getattr(model_args, "model_name_or_path", None)
    if src and os.path.isdir(src):
        cbs.append(PreserveTokenizerConfigCallback(src))
    return cbs


def run_ppo(model, ft_args, run_args, dataset, tokenizer, device, bsz):
    """PPO stage: prompts come from the dataset's ``input_ids`` (truncated to ``cutoff``), scores from the reward model
    of ``ft_args.reward_model`` (a checkpoint of the ``rm`` stage), the KL reference from ``ft_args.ref_model`` or the
    policy's own starting point.  Single-process (data-parallel PPO is not wired)."""
    from .ppo import PPOConfig, PPOTrainer, reward_model_fn
    if not getattr(ft_args, "reward_model", None):
        raise ValueError("`reward_model` is necessary for PPO training")
    rm = checkpoint_io.from_pretrained(ft_args.reward_model, device=device).eval()
    vh = dict(checkpoint_io.load_state_dict(ft_args.reward_model)).get("v_head.weight")
    if vh is not None:
        from .preference import attach_value_head
        with torch.no_grad():
            attach_value_head(rm).weight.copy_(vh.to(rm.v_head.weight.dtype))
    ref = checkpoint_io.from_pretrained(ft_args.ref_model, device=device).eval() if getattr(ft_args, "ref_model", None) else None
    cfg = PPOConfig(learning_rate=run_args.learning_rate, ppo_epochs=ft_args.ppo_epochs,
                    ppo_buffer_size=ft_args.ppo_buffer_size, mini_batch_size=run_args.per_device_train_batch_size,
                    ppo_score_norm=ft_args.ppo_score_norm, ppo_target=ft_args.ppo_target,
                    ppo_whiten_rewards=ft_args.ppo_whiten_rewards, max_grad_norm=run_args.max_grad_norm,
                    eos_token_id=getattr(tokenizer, "eos_token_id", None),
                    max_new_tokens=getattr(ft_args, "ppo_max_new_tokens", 64))
    trainer = PPOTrainer(model, reward_model_fn(rm), cfg, ref_model=ref)
    it = iter(dataset)
    plen = getattr(ft_args, "ppo_prompt_len", 32)
    for step in range(run_args.max_steps if run_args.max_steps > 0 else 100):
        groups = []
        for _ in range(cfg.ppo_buffer_size):
            rows = []
            while len(rows) < bsz:
                try:
                    ex = next(it)
                except StopIteration:
                    it = iter(dataset)
                    continue
                ids = torch.as_tensor(ex["input_ids"]).flatten()[:plen]
                if ids.numel() == plen:
                    rows.append(ids)
            groups.append(torch.stack(rows).to(device))
        stats = trainer.step(groups)
        info_rank0(logger, "ppo step %d: %s", step + 1, {k: round(v, 4) for k, v in stats.items()})
    os.makedirs(run_args.output_dir, exist_ok=True)
    checkpoint_io.save_pretrained(model, os.path.join(run_args.output_dir, "final"))
    torch.save(trainer.value_head.state_dict(), os.path.join(run_args.output_dir, "final", "value_head.pt"))
    return trainer


def run_prediction(model, tokenizer, data_args, run_args, gen_args):
    """``do_predict``: generate an answer for every sample of ``eval_dataset`` (or ``dataset``), write
    ``generated_predictions.jsonl`` and the text metrics to ``output_dir`` (single process)."""
    import copy
    from .predict import run_predict
    da = copy.copy(data_args)
    da.dataset = data_args.eval_dataset or data_args.dataset
    da.tokenized_path, da.synthetic, da.disable_shuffling = None, False, True      # keep the file order
    rows = get_dataset(da, tokenizer, stage="unsupervised")
    rows = [rows[i] for i in range(len(rows))]
    metrics = run_predict(model.eval(), tokenizer, rows, run_args.output_dir, max_new_tokens=gen_args.max_new_tokens,
                          temperature=gen_args.temperature if gen_args.do_sample else 0.0, top_k=gen_args.top_k,
                          max_model_len=data_args.cutoff_len + gen_args.max_new_tokens + 64)
    info_rank0(logger, "prediction metrics: %s", metrics)
    return metrics


def run_exp(args: Optional[Any] = None) -> Trainer:
    model_args, data_args, run_args, ft_args, _ = get_train_args(args)
    init_distributed(run_args.ddp_timeout)
    torch.manual_seed(run_args.seed)
    device = _device()
    world = dist.get_world_size() if dist.is_initialized() else 1
    rank = dist.get_rank() if dist.is_initialized() else 0
    sp = model_args.sequence_parallel_size
    tokenizer = load_tokenizer(model_args.model_name_or_path)
    model = load_model(model_args, run_args, device)
    from .patcher import patch_model
    tok_size = len(tokenizer) if (tokenizer is not None and hasattr(tokenizer, "__len__")) else None
    patch_model(model, vocab_size=tok_size, resize_vocab=model_args.resize_vocab,
                upcast_norms=getattr(model_args, "upcast_layernorm", False),
                upcast_logits=getattr(model_args, "upcast_lmhead_output", False), gradient_checkpointing=False)
    stage = ft_args.stage
    if run_args.do_predict and not run_args.do_train:
        return run_prediction(model, tokenizer, data_args, run_args, _)
    if stage == "hkd" or ft_args.hybrid_learnable_params:
        n = freeze_params_hybrid(model, ft_args.hybrid_learnable_params)
        info_rank0(logger, "trainable parameters: %d", n)
    if ft_args.finetuning_type == "lora":
        from .adapters import apply_lora
        wrapped = apply_lora(model, ft_args.lora_rank, ft_args.lora_alpha, ft_args.lora_target,
                             use_rslora=ft_args.use_rslora, use_dora=ft_args.use_dora, pissa_init=ft_args.pissa_init,
                             pissa_iter=ft_args.pissa_iter)
        info_rank0(logger, "LoRA adapters on %d linear layers", len(wrapped))
        if getattr(ft_args, "quantization_bit", None):
            from .qlora import quantize_adapter_bases, quantized_bytes
            qn = quantize_adapter_bases(model, int(ft_args.quantization_bit), ft_args.quantization_type)
            info_rank0(logger, "%d adapted layers keep their base weight as %d-bit codes (%.2f GB)", len(qn),
                       int(ft_args.quantization_bit), quantized_bytes(model) / 1e9)
    if getattr(ft_args, "mixture_of_depths", None) == "convert":
        from ..models.mod import apply_mixture_of_depths
        routed = apply_mixture_of_depths(model, capacity=ft_args.mod_capacity)
        info_rank0(logger, "mixture-of-depths routers on layers %s (capacity %.3f)", routed, ft_args.mod_capacity)
    if getattr(ft_args, "shift_attn", False):
        from ..layers.attention import Attention
        n_shift = 0
        for m in model.modules():
            if isinstance(m, Attention) and m.sliding_window is None:
                m.shift_group_ratio = 0.25
                n_shift += 1
        info_rank0(logger, "shifted sparse attention on %d attention layers", n_shift)
    elif ft_args.finetuning_type == "oft":
        from .patcher import add_oft
        wrapped = add_oft(model, tuple(t.strip() for t in ft_args.lora_target.split(",")), ft_args.oft_block_size)
        info_rank0(logger, "OFT rotations on %d linear layers", len(wrapped))
    elif ft_args.finetuning_type == "freeze":
        from .adapters import freeze_all_but_last
        info_rank0(logger, "trainable parameters: %d", freeze_all_but_last(model, ft_args.freeze_trainable_layers))
    if hasattr(model, "visual") and hasattr(model, "language_model"):
        from ..models.vl import apply_vl_freezing
        counts = apply_vl_freezing(model, ft_args.freeze_vision_tower, ft_args.freeze_multi_modal_projector,
                                   ft_args.freeze_language_model)
        info_rank0(logger, "vision-language model, trainable parameters per part: %s", counts)
    if getattr(run_args, "fp8", False):
        from ..ops.fp8 import use_fp8_linear
        info_rank0(logger, "fp8: %d linear layers run their GEMMs in row-wise scaled float8", use_fp8_linear(model))
    if not data_args.template and stage not in ("pt", "hkd"):
        # no template given: the one the model family speaks (`data/model_registry.py`), else the plain default
        from ..data.model_registry import template_for_model
        guess = template_for_model(getattr(model_args, "model_name_or_path", None))
        if guess:
            data_args.template = guess
            info_rank0(logger, "template '%s' chosen from the model name", guess)
    dataset = get_dataset(data_args, tokenizer, stage=("pt" if stage in ("pt", "hkd") else stage if stage in ("rm", "dpo", "kto") else "sft"), sp_size=sp,
                          vocab_size=model.config.vocab_size, seed=run_args.seed)
    bsz = run_args.per_device_train_batch_size * run_args.gradient_accumulation_steps
    held = None
    if data_args.val_size and hasattr(dataset, "rows"):
        # hold out the tail of the dataset (whole SP groups): `val_size` is a fraction below 1, a sample count above
        from ..data.loader import ListDataset
        groups = len(dataset) // sp
        n_val = int(data_args.val_size * groups) if data_args.val_size < 1 else int(data_args.val_size)
        n_val = max(1, min(n_val, groups - 1))
        held = ListDataset(dataset.rows[(groups - n_val) * sp:groups * sp], dataset.labels_shifted)
        dataset = ListDataset(dataset.rows[:(groups - n_val) * sp], dataset.labels_shifted)
    n_batches = None
    if hasattr(dataset, "__len__") and len(dataset) < (1 << 29):
        from ..data.loader import steps_per_epoch
        n_batches = steps_per_epoch(len(dataset), bsz, world, sp)      # counted after the hold-out split
    targs = to_trainer_args(model_args, data_args, run_args, n_batches)
    if ft_args.use_muon:
        targs.optimizer = "muon"
    targs.optimizer, targs.optimizer_args = select_optimizer(ft_args, targs.optimizer)
    loss_fn = None
    teacher = None
    if stage == "hkd":
        if ft_args.hybrid_distill_loss == "kl":
            if not ft_args.teacher_model_name_or_path:
                raise ValueError("hybrid_distill_loss=kl needs teacher_model_name_or_path")
            teacher = checkpoint_io.from_pretrained(ft_args.teacher_model_name_or_path, device=device).eval()
            for p in teacher.parameters():
                p.requires_grad_(False)
            loss_fn = lambda m, b: hkd_kl_loss(m, teacher, b)  # noqa: E731
        else:
            loss_fn = lambda m, b: hkd_mse_loss(m, b, ft_args.hybrid_lw_distill_target,  # noqa: E731
                                                ft_args.hybrid_distill_pre_lm_head)
    elif stage in ("dpo", "kto", "rm"):
        from .preference import NEEDS_REFERENCE, ReferencePolicy, attach_value_head, make_preference_loss
        reference = None
        if stage == "kto" or (stage == "dpo" and ft_args.pref_loss in NEEDS_REFERENCE):
            reference = ReferencePolicy.build(model, ft_args, device)     # before training touches the weights
        if stage == "rm":
            attach_value_head(model)                                      # before the optimizer collects parameters
        loss_fn = make_preference_loss(stage, ft_args, reference, getattr(tokenizer, "pad_token_id", None) or 0)
    if stage == "sft" and (ft_args.use_dft_loss or ft_args.use_eaft_loss):
        from .losses import make_weighted_sft_loss
        loss_fn = make_weighted_sft_loss("dft" if ft_args.use_dft_loss else "eaft", ft_args.eaft_alpha)
    if stage in ("pt", "sft") and loss_fn is None and getattr(ft_args, "lambda_reg", 0.0) > 0:
        from ..layers.l2a import L2AAttention
        if any(isinstance(m, L2AAttention) for m in model.modules()):
            from .l2a import L2ALoss
            loss_fn = L2ALoss(targs, ft_args.lambda_reg, ft_args.lambda_reg_scheduler)
            info_rank0(logger, "L2A objective: language-model loss + lambda(step) x router sparsity term, lambda up to "
                       "%.3g (%s ramp after warm-up)", ft_args.lambda_reg, ft_args.lambda_reg_scheduler)
    if stage == "ppo":
        return run_ppo(model, ft_args, run_args, dataset, tokenizer, device, bsz)
    trainer = Trainer(model, targs, device=device, loss_fn=loss_fn, callbacks=build_callbacks(run_args, model_args))
    if getattr(ft_args, "neftune_noise_alpha", 0.0):
        from .adapters import add_neftune
        add_neftune(model, ft_args.neftune_noise_alpha)
        info_rank0(logger, "NEFTune: uniform noise of scale %.1f / sqrt(tokens x width) on the embeddings while training",
                   ft_args.neftune_noise_alpha)
    if teacher is not None:
        from ..parallel.sp import set_sequence_parallel_group_recursive
        set_sequence_parallel_group_recursive(teacher, trainer.sp)
    pad_id = getattr(tokenizer, "pad_token_id", None) or 0
    if held is not None:
        ebs = run_args.per_device_eval_batch_size
        trainer.eval_batches_fn = lambda: batch_iterator(held, ebs, rank, world, sp, pad_id, pin=device.type == "cuda",
                                                         num_epochs=1)
    # the stream wraps around epoch by epoch (fresh order per epoch unless disable_shuffling); the trainer stops at
    # max_steps, which to_trainer_args derived from num_train_epochs when it was not given
    batches = batch_iterator(dataset, bsz, rank, world, sp, pad_id, start_step=trainer.global_step,
                             pin=device.type == "cuda", shuffle=not getattr(data_args, "disable_shuffling", False),
                             seed=run_args.seed)
    if run_args.do_train:
        trainer.train(batches)
        final = os.path.join(run_args.output_dir, "final")
        if ft_args.finetuning_type == "lora":
            from .adapters import merge_lora
            merge_lora(model)                     # the final checkpoint has the ordinary layout
        elif ft_args.finetuning_type == "oft":
            from .patcher import merge_oft
            merge_oft(model)
        trainer.args.save_only_model = True
        trainer.save_checkpoint(final)
        if getattr(run_args, "plot_loss", False) and rank == 0:
            from ..utils.ploting import plot_loss
            info_rank0(logger, "loss curves: %s", plot_loss(run_args.output_dir))
        if rank == 0:
            for fn in ("tokenizer.json", "tokenizer_config.json", "vocab.json", "merges.txt", "special_tokens_map.json"):
                src = os.path.join(model_args.model_name_or_path or "", fn)
                if os.path.exists(src):
                    import shutil
                    shutil.copy(src, os.path.join(final, fn))
    return trainer
