"""``USE_V1=1 hmf train config.yaml`` (or ``python -m hybrid_model_factory_b200.v1.launcher config.yaml``): supervised
fine-tuning on the second-generation stack.  The YAML holds ``model`` (checkpoint directory), ``train_dataset``
(dataset description file, directory or file of records), ``template``, optional ``init_config`` / ``peft_config`` /
``kernel_config`` sections (``v1/model_engine.py``) and the fields of ``V1TrainingArguments``.
Reference: ``v1/launcher.py:34-179`` and ``v1/trainers/sft_trainer.py``."""
from __future__ import annotations

import os
import sys
from dataclasses import fields
from typing import List

import torch


def run_sft(config_path: str, overrides: List[str] = ()) -> int:
    import yaml
    from . import DataEngine, SFTTrainerV1, V1TrainingArguments
    with open(config_path) as fh:
        cfg = yaml.safe_load(fh) or {}
    for ov in overrides:                      # key=value on the command line wins over the file
        k, _, v = ov.partition("=")
        cfg[k] = yaml.safe_load(v)
    known = {f.name for f in fields(V1TrainingArguments)}
    extra = set(cfg) - known - {"model", "train_dataset", "template", "resume_from", "init_config", "peft_config",
                                "kernel_config"}
    if extra:
        raise ValueError(f"unknown configuration keys: {sorted(extra)}")
    args = V1TrainingArguments(**{k: v for k, v in cfg.items() if k in known})
    world = int(os.environ.get("WORLD_SIZE", "1"))
    device = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0"))) if torch.cuda.is_available() else torch.device("cpu")
    if world > 1:
        import torch.distributed as dist
        if device.type == "cuda":
            torch.cuda.set_device(device)
            dist.init_process_group("nccl", device_id=device)
        else:
            dist.init_process_group("gloo")
    dtype = torch.bfloat16 if args.bf16 else torch.float32
    from .model_engine import ModelEngine
    engine = ModelEngine(cfg["model"], template=cfg.get("template"), cutoff_len=args.cutoff_len, dtype=dtype,
                         device=device, init_config=cfg.get("init_config"), peft_config=cfg.get("peft_config"),
                         kernel_config=cfg.get("kernel_config"))
    model, renderer = engine.model, engine.renderer
    trainer = SFTTrainerV1(args, model, renderer, DataEngine(cfg["train_dataset"]), device=device)
    if cfg.get("resume_from"):
        trainer.load_checkpoint(cfg["resume_from"])
    trainer.fit()
    if cfg.get("peft_config", {}).get("name") == "lora":
        from ..train.adapters import merge_lora
        merge_lora(model)                     # the saved model has the ordinary layout
    trainer.save_model()
    if trainer.rank == 0:
        last = trainer.history[-1] if trainer.history else {}
        print(f"v1 sft: {trainer.global_step} steps, last loss {last.get('loss', float('nan')):.4f}, "
              f"model in {args.output_dir}")
    return 0


def main(argv=None) -> int:
    argv = list(sys.argv[1:] if argv is None else argv)
    if not argv:
        print("usage: USE_V1=1 hmf train CONFIG.yaml [key=value ...]")
        return 2
    return run_sft(argv[0], argv[1:])


if __name__ == "__main__":
    raise SystemExit(main())
