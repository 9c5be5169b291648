"""Run configuration: one flat YAML / JSON (plus ``key=value`` command-line overrides) split into
five argument groups.  Key names follow the reference project's training YAMLs so existing configs
keep working (``hparams/model_args.py``, ``data_args.py``, ``training_args.py``,
``finetuning_args.py``, ``generating_args.py``; surface listed in the reference's
``examples/priming/**.yaml``)."""
from __future__ import annotations

import json
from dataclasses import asdict, dataclass, fields
from typing import Any, Dict, Optional


@dataclass
class ModelArguments:
    model_name_or_path: Optional[str] = None
    config_overrides_json: Optional[str] = None      # JSON string or path: dotted keys into config.json
    trust_remote_code: bool = False
    flash_attn: str = "auto"
    enable_liger_kernel: bool = False                  # accepted for compatibility: fused kernels are always on
    sequence_parallel_size: int = 1
    sequence_parallel_mode: str = "zigzag-ring"       # zigzag-ring | ulysses (attention only)
    use_deepspeed_mics: bool = False
    preserve_tokenizer_config: bool = False
    resize_vocab: bool = False
    rope_scaling: Optional[str] = None                 # linear | dynamic | yarn | llama3
    model_max_length: Optional[int] = None             # target context for the RoPE scaling factor
    upcast_layernorm: bool = False
    upcast_lmhead_output: bool = False
    infer_dtype: str = "auto"
    adapter_name_or_path: Optional[str] = None

    def config_overrides(self) -> Dict[str, Any]:
        if not self.config_overrides_json:
            return {}
        s = self.config_overrides_json
        if isinstance(s, dict):
            return s
        try:
            return json.loads(s)
        except json.JSONDecodeError:
            with open(s) as f:
                return json.load(f)


@dataclass
class DataArguments:
    dataset: Optional[str] = None                      # comma separated names from dataset_info.json
    eval_dataset: Optional[str] = None                 # dataset(s) for `do_predict`
    dataset_dir: str = "data"
    tokenized_path: Optional[str] = None
    cutoff_len: int = 2048
    template: Optional[str] = None
    mix_strategy: str = "concat"                       # concat | interleave_under | interleave_over | interleave_fast
    interleave_probs: Optional[str] = None
    packing: Optional[bool] = None
    neat_packing: bool = False
    streaming: bool = False
    preprocessing_num_workers: Optional[int] = None
    max_samples: Optional[int] = None
    val_size: float = 0.0
    disable_shuffling: bool = False
    overwrite_cache: bool = False
    train_on_prompt: bool = False
    mask_history: bool = False
    ignore_pad_token_for_loss: bool = True
    synthetic: bool = False                            # uniform random token ids of cutoff_len (benchmarks, smoke runs)
    synthetic_vocab: int = 0


@dataclass
class RunArguments:
    """Training-loop arguments (the HF ``TrainingArguments`` subset the reference configs use)."""
    output_dir: str = "output"
    overwrite_output_dir: bool = False
    do_train: bool = True
    do_predict: bool = False                           # generate over `eval_dataset` (or `dataset`) and score the text
    predict_with_generate: bool = False                # accepted for compatibility (prediction always generates)
    per_device_train_batch_size: int = 1
    gradient_accumulation_steps: int = 1
    learning_rate: float = 1e-5
    weight_decay: float = 0.0
    adam_beta1: float = 0.9
    adam_beta2: float = 0.999
    adam_epsilon: float = 1e-8
    max_grad_norm: float = 1.0
    num_train_epochs: float = 1.0
    max_steps: int = -1
    lr_scheduler_type: str = "cosine"
    warmup_steps: int = 0
    warmup_ratio: float = 0.0
    logging_steps: int = 1
    save_steps: int = 0
    eval_steps: int = 0                                # with `val_size`: held-out loss every N steps and at the end
    eval_strategy: str = "steps"                       # accepted for compatibility
    per_device_eval_batch_size: int = 1
    save_only_model: bool = False
    save_max_shard_size: str = "5GB"
    seed: int = 42
    bf16: bool = True
    pure_bf16: bool = True
    fp8: bool = False
    disable_gradient_checkpointing: bool = False
    recompute_budget: str = "auto"             # auto | off | fraction of the device memory that un-checkpointed layers may fill
    deepspeed: Optional[str] = None                    # accepted; ZeRO stage is read from the JSON ("zero_optimization.stage")
    ddp_timeout: int = 180000000
    report_to: str = "none"
    resume_from_checkpoint: Optional[str] = None
    plot_loss: bool = False
    ray: bool = False


@dataclass
class FinetuningArguments:
    stage: str = "pt"                                  # pt | sft | hkd | rm | ppo | dpo | kto
    finetuning_type: str = "full"                      # full | freeze | lora | oft
    oft_block_size: int = 32
    hybrid_learnable_params: Optional[str] = None      # comma separated substrings, e.g. "gka,norm,self_attn"
    hybrid_lw_distill_target: Optional[str] = None     # decoder | mixer | residuals | all
    hybrid_distill_pre_lm_head: bool = True
    hybrid_distill_loss: str = "mse"                   # mse (fused two-stream model) | kl (external teacher logits)
    teacher_model_name_or_path: Optional[str] = None
    use_muon: bool = False
    use_adam_mini: bool = False
    use_galore: bool = False
    galore_target: str = "all"
    galore_rank: int = 16
    galore_update_interval: int = 200
    galore_scale: float = 2.0
    galore_proj_type: str = "std"                      # std | reverse_std | right | left
    use_apollo: bool = False
    apollo_target: str = "all"
    apollo_rank: int = 16
    apollo_update_interval: int = 200
    apollo_scale: float = 32.0
    apollo_proj: str = "random"                        # svd | random
    apollo_proj_type: str = "std"
    apollo_scale_type: str = "channel"                 # channel | tensor
    use_badam: bool = False
    badam_mode: str = "layer"                          # layer | ratio
    badam_start_block: Optional[int] = None
    badam_switch_mode: str = "ascending"               # ascending | descending | random | fixed
    badam_switch_interval: int = 50
    badam_update_ratio: float = 0.05
    badam_mask_mode: str = "adjacent"                  # adjacent | scatter
    reward_model: Optional[str] = None                 # PPO: checkpoint of the `rm` stage
    ref_model: Optional[str] = None                    # PPO / DPO reference policy (default: the starting policy)
    ppo_buffer_size: int = 1
    ppo_epochs: int = 4
    ppo_score_norm: bool = False
    ppo_target: float = 6.0
    ppo_whiten_rewards: bool = False
    ppo_max_new_tokens: int = 64
    ppo_prompt_len: int = 32
    loraplus_lr_ratio: Optional[float] = None
    loraplus_lr_embedding: float = 1e-6
    pref_beta: float = 0.1
    pref_loss: str = "sigmoid"
    lora_rank: int = 8
    lora_alpha: Optional[int] = None
    lora_target: str = "all"
    use_rslora: bool = False                   # scale alpha / sqrt(rank)
    use_dora: bool = False                     # weight-decomposed LoRA (trainable row magnitudes)
    pissa_init: bool = False                   # adapters start as the principal singular directions of the weight
    pissa_iter: int = 16                       # power iterations of the randomised SVD (0: exact SVD)
    freeze_vision_tower: bool = True           # vision-language models: which parts train
    freeze_multi_modal_projector: bool = True
    freeze_language_model: bool = False
    use_dft_loss: bool = False                 # SFT: token losses scaled by the target's (detached) probability
    use_eaft_loss: bool = False                # SFT: token losses scaled by the top-20 entropy ** eaft_alpha
    eaft_alpha: float = 1.0
    mixture_of_depths: Optional[str] = None    # "convert": add token routers to every second layer; "load": checkpoint has them
    mod_capacity: float = 0.125                # fraction of a row's tokens a routed layer processes while training
    lambda_reg: float = 0.0                    # L2A models: weight of the router sparsity term (0: plain language-model loss)
    lambda_reg_scheduler: str = "linear"       # linear | cosine | constant ramp of lambda after warm-up
    quantization_bit: Optional[int] = None     # lora: 4 or 8, the adapted layers' frozen base weights are held as codes (QLoRA)
    quantization_type: str = "nf4"             # 4-bit levels: nf4 (normal-quantile table) or int
    neftune_noise_alpha: float = 0.0           # > 0: noisy embeddings while training (scale alpha / sqrt(tokens x width))
    shift_attn: bool = False                   # LongLoRA shifted sparse attention while training (groups of 1/4 length)
    freeze_trainable_layers: int = 2
    include_effective_tokens_per_second: bool = False


@dataclass
class GeneratingArguments:
    do_sample: bool = True
    temperature: float = 0.95
    top_p: float = 0.7
    top_k: int = 50
    max_new_tokens: int = 1024
    repetition_penalty: float = 1.0


GROUPS = (ModelArguments, DataArguments, RunArguments, FinetuningArguments, GeneratingArguments)


def split_args(flat: Dict[str, Any], allow_extra: bool = False):
    """Distributes a flat dict over the five dataclasses; unknown keys raise unless allowed."""
    remaining = dict(flat)
    out = []
    for cls in GROUPS:
        names = {f.name for f in fields(cls)}
        kwargs = {k: remaining.pop(k) for k in list(remaining) if k in names}
        out.append(cls(**kwargs))
    # keys shared by two groups (sequence_parallel_size lives in ModelArguments, also read by the run loop)
    if remaining and not allow_extra:
        raise ValueError(f"unknown configuration keys: {sorted(remaining)} (set ALLOW_EXTRA_ARGS=1 to ignore)")
    return tuple(out)


def to_flat_dict(*groups) -> Dict[str, Any]:
    d: Dict[str, Any] = {}
    for g in groups:
        d.update(asdict(g))
    return d
