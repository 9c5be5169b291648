"""Reading run configurations: ``hmf train cfg.yaml key=value ...`` or a dict.

A YAML / JSON file provides the base; ``key=value`` (or ``--key value``) tokens override it with
YAML-typed values; dotted keys address nested dicts.  The result is validated and split into the
argument groups of ``hparams.py``.  Reference: ``hparams/parser.py:57-71`` (``read_args``) and
``:207-430`` (``get_train_args``)."""
from __future__ import annotations

import json
import os
import sys
from typing import Any, Dict, Optional, Sequence

import yaml

from .hparams import (DataArguments, FinetuningArguments, GeneratingArguments, ModelArguments, RunArguments, split_args)

STAGES = ("pt", "sft", "hkd", "rm", "ppo", "dpo", "kto")


def _set_dotted(d: Dict[str, Any], key: str, value: Any) -> None:
    parts = key.split(".")
    for p in parts[:-1]:
        d = d.setdefault(p, {})
    d[parts[-1]] = value


def _typed(text: str) -> Any:
    """YAML typing plus plain scientific notation (YAML 1.1 reads ``5e-5`` as a string)."""
    v = yaml.safe_load(text)
    if isinstance(v, str):
        try:
            return float(v) if any(c in v for c in ".eE") else int(v)
        except ValueError:
            return v
    return v


def _fix_numbers(d: Dict[str, Any]) -> Dict[str, Any]:
    for k, v in list(d.items()):
        if isinstance(v, dict):
            _fix_numbers(v)
        elif isinstance(v, str) and k not in ("model_name_or_path", "dataset", "output_dir", "template"):
            try:
                d[k] = float(v) if any(c in v for c in "eE") and v.replace(".", "").replace("-", "").replace(
                    "e", "").replace("E", "").replace("+", "").isdigit() else v
            except ValueError:
                pass
    return d


def parse_overrides(tokens: Sequence[str]) -> Dict[str, Any]:
    out: Dict[str, Any] = {}
    i = 0
    tokens = list(tokens)
    while i < len(tokens):
        t = tokens[i]
        if "=" in t and not t.startswith("--"):
            k, v = t.split("=", 1)
            _set_dotted(out, k, _typed(v))
        elif t.startswith("--"):
            k = t[2:]
            if "=" in k:
                k, v = k.split("=", 1)
            elif i + 1 < len(tokens) and not tokens[i + 1].startswith("--"):
                i += 1
                v = tokens[i]
            else:
                v = "true"
            _set_dotted(out, k.replace("-", "_"), _typed(v))
        else:
            raise ValueError(f"cannot parse argument '{t}' (expected key=value)")
        i += 1
    return out


def read_args(args: Optional[Any] = None) -> Dict[str, Any]:
    """``args``: ``None`` (use ``sys.argv[1:]``), a dict, or a token list whose first element may be a
    ``.yaml`` / ``.yml`` / ``.json`` path."""
    if isinstance(args, dict):
        return dict(args)
    tokens = list(sys.argv[1:] if args is None else args)
    base: Dict[str, Any] = {}
    if tokens and tokens[0].endswith((".yaml", ".yml", ".json")):
        path = tokens.pop(0)
        with open(path) as f:
            base = _fix_numbers((json.load(f) if path.endswith(".json") else yaml.safe_load(f)) or {})
    over = parse_overrides(tokens)
    for k, v in over.items():
        if isinstance(v, dict) and isinstance(base.get(k), dict):
            base[k].update(v)
        else:
            base[k] = v
    return base


def get_train_args(args: Optional[Any] = None):
    flat = read_args(args)
    allow_extra = os.environ.get("ALLOW_EXTRA_ARGS", "0").lower() in ("1", "true", "y")
    model_args, data_args, run_args, ft_args, gen_args = split_args(flat, allow_extra)
    validate(model_args, data_args, run_args, ft_args)
    return model_args, data_args, run_args, ft_args, gen_args


def validate(model_args: ModelArguments, data_args: DataArguments, run_args: RunArguments,
             ft_args: FinetuningArguments) -> None:
    if ft_args.stage not in STAGES:
        raise ValueError(f"stage must be one of {STAGES}, got '{ft_args.stage}'")
    if run_args.do_train and not (data_args.dataset or data_args.tokenized_path or data_args.synthetic):
        raise ValueError("training needs `dataset`, `tokenized_path` or `synthetic: true`")
    sp = model_args.sequence_parallel_size
    if sp < 1:
        raise ValueError("sequence_parallel_size must be >= 1")
    if sp > 1:
        if data_args.cutoff_len % (2 * sp) != 0:
            raise ValueError(f"cutoff_len={data_args.cutoff_len} must be divisible by 2*sequence_parallel_size={2 * sp}")
        if model_args.sequence_parallel_mode not in ("zigzag-ring", "ulysses"):
            raise ValueError(f"unknown sequence_parallel_mode '{model_args.sequence_parallel_mode}'")
        if model_args.sequence_parallel_mode == "ulysses":
            raise ValueError("ulysses sequence parallelism is not supported for hybrid models")
    if ft_args.stage == "hkd" and ft_args.hybrid_lw_distill_target not in (None, "decoder", "mixer", "residuals", "all"):
        raise ValueError(f"unknown hybrid_lw_distill_target '{ft_args.hybrid_lw_distill_target}'")
    if run_args.pure_bf16 and not run_args.bf16:
        run_args.bf16 = True
    if run_args.max_steps < 0 and data_args.synthetic:
        raise ValueError("synthetic data needs an explicit max_steps")
    if (run_args.do_train and os.path.isdir(run_args.output_dir) and os.listdir(run_args.output_dir)
            and not run_args.overwrite_output_dir and run_args.resume_from_checkpoint is None):
        from ..train.trainer import get_last_checkpoint
        last = get_last_checkpoint(run_args.output_dir)
        if last is not None:
            run_args.resume_from_checkpoint = last  # auto-resume
