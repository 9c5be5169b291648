"""Trainer callbacks: called as ``cb(trainer)`` after every optimizer step (and ``cb.on_train_end(trainer)`` once).

* ``LogCallback``        progress / throughput / optional VRAM to ``trainer_log.jsonl`` plus an abort flag file
* ``PreserveTokenizerConfigCallback``  re-copies the original tokenizer files into every checkpoint
* ``ReporterCallback``   forwards scalars to wandb / swanlab when those packages are importable
* ``EarlyStopCallback``  stops on non-finite loss
Reference: ``train/callbacks.py:98-431``.
"""
from __future__ import annotations

import json
import math
import os
import shutil
import signal
import time
from typing import Optional


class LogCallback:
    def __init__(self, output_dir: str, every: int = 1):
        self.path = os.path.join(output_dir, "trainer_log.jsonl")
        self.every, self.t0, self.aborted = every, time.time(), False
        os.makedirs(output_dir, exist_ok=True)
        try:
            signal.signal(signal.SIGABRT, self._abort)
        except (ValueError, OSError):        # not in the main thread
            pass

    def _abort(self, *_):
        self.aborted = True

    def __call__(self, trainer) -> None:
        if self.aborted:
            trainer.args.max_steps = trainer.global_step        # leave the loop at the next check
        if trainer.rank != 0 or trainer.global_step % self.every:
            return
        elapsed = time.time() - self.t0
        total = max(trainer.args.max_steps, 1)
        rec = {"current_steps": trainer.global_step, "total_steps": total,
               "percentage": round(100.0 * trainer.global_step / total, 2), "elapsed_time": round(elapsed, 1),
               "remaining_time": round(elapsed / max(trainer.global_step, 1) * (total - trainer.global_step), 1),
               "throughput": round(trainer.tokens_seen / max(elapsed, 1e-9), 2), "lr": getattr(trainer, "_last_lr", None)}
        if os.environ.get("RECORD_VRAM", "0") == "1":
            import torch
            if torch.cuda.is_available():
                rec["vram_allocated_gb"] = round(torch.cuda.max_memory_allocated() / 2 ** 30, 2)
                rec["vram_reserved_gb"] = round(torch.cuda.max_memory_reserved() / 2 ** 30, 2)
        with open(self.path, "a") as f:
            f.write(json.dumps(rec) + "\n")


class PreserveTokenizerConfigCallback:
    FILES = ("tokenizer.json", "tokenizer_config.json", "special_tokens_map.json", "vocab.json", "merges.txt",
             "chat_template.jinja", "tokenizer.model")

    def __init__(self, source_dir: str):
        self.source_dir = source_dir
        self._seen = set()

    def __call__(self, trainer) -> None:
        if trainer.rank != 0 or not trainer.args.save_steps or trainer.global_step % trainer.args.save_steps:
            return
        ckpt = os.path.join(trainer.args.output_dir, f"checkpoint-{trainer.global_step}")
        self.copy_into(ckpt)

    def copy_into(self, ckpt: str) -> None:
        if not os.path.isdir(ckpt) or ckpt in self._seen or not self.source_dir or not os.path.isdir(self.source_dir):
            return
        self._seen.add(ckpt)
        for name in self.FILES:
            src = os.path.join(self.source_dir, name)
            if os.path.exists(src):
                shutil.copy(src, os.path.join(ckpt, name))


class ReporterCallback:
    def __init__(self, project: str = "hybrid-model-factory", config: Optional[dict] = None, backend: str = "auto"):
        self.run = None
        for name in (("wandb", "swanlab") if backend == "auto" else (backend,)):
            try:
                mod = __import__(name)
                self.run = mod.init(project=project, config=config or {})
                self.log = mod.log
                break
            except Exception:
                continue

    def __call__(self, trainer) -> None:
        if self.run is None or trainer.rank != 0:
            return
        self.log({"train/step": trainer.global_step, "train/lr": getattr(trainer, "_last_lr", 0.0),
                  "train/tokens": trainer.tokens_seen}, step=trainer.global_step)


class EarlyStopCallback:
    """Stops training when the last logged loss is NaN / inf."""

    def __call__(self, trainer) -> None:
        loss = getattr(trainer, "_last_loss", None)
        if loss is not None and not math.isfinite(loss):
            trainer.args.max_steps = trainer.global_step
