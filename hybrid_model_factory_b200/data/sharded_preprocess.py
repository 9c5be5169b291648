"""Parallel, sharded preprocessing for corpora that do not fit a single process (``hmf preprocess``).

Four phases, each restartable from its output directory:
  1. **align**    every dataset is read and converted to the common record format by a pool of workers, one
                  output file per (dataset, worker);
  2. **shard**    the aligned records are merged, optionally shuffled, and cut into ``num_shards`` shards;
  3. **tokenize** the shards are tokenised / packed to ``cutoff_len`` in parallel (SP pad + shift + zig-zag
                  split when ``sequence_parallel_size > 1``), one ``shard_XXXXX.pt`` each;
  4. **concatenate** the shard files are indexed (or merged into one ``dataset.pt``) under ``tokenized_path``.
Reference: ``data/sharded_preprocess_and_tokenize.py:96-501``.
"""
from __future__ import annotations

import argparse
import json
import os
import random
from concurrent.futures import ProcessPoolExecutor
from typing import List, Optional

import torch

from ..config.hparams import DataArguments
from .formats import align_dataset, get_dataset_list, get_template, load_tokenizer
from .loader import (ListDataset, pack_supervised, preprocess_sp_dataset, process_pretrain, process_supervised)


def _align_worker(job):
    dataset_dir, attr_dict, part, parts, out = job
    from .formats import DatasetAttr
    attr = DatasetAttr(**attr_dict)
    rows = align_dataset(attr, dataset_dir)
    rows = rows[part::parts]
    with open(out, "w") as f:
        for r in rows:
            f.write(json.dumps(r) + "\n")
    return out, len(rows)


def phase_align(data_args: DataArguments, work: str, workers: int) -> List[str]:
    os.makedirs(os.path.join(work, "aligned"), exist_ok=True)
    jobs = []
    for attr in get_dataset_list(data_args.dataset, data_args.dataset_dir):
        for part in range(workers):
            out = os.path.join(work, "aligned", f"{attr.name}.{part:03d}.jsonl")
            if not os.path.exists(out):
                jobs.append((data_args.dataset_dir, attr.__dict__, part, workers, out))
    if jobs:
        with ProcessPoolExecutor(max_workers=workers) as ex:
            list(ex.map(_align_worker, jobs))
    return sorted(os.path.join(work, "aligned", n) for n in os.listdir(os.path.join(work, "aligned")))


def phase_shard(aligned: List[str], work: str, num_shards: int, shuffle: bool, seed: int) -> List[str]:
    os.makedirs(os.path.join(work, "shards"), exist_ok=True)
    outs = [os.path.join(work, "shards", f"shard_{i:05d}.jsonl") for i in range(num_shards)]
    if all(os.path.exists(o) for o in outs):
        return outs
    rows = []
    for path in aligned:
        with open(path) as f:
            rows.extend(f.readlines())
    if shuffle:
        random.Random(seed).shuffle(rows)
    for i, o in enumerate(outs):
        with open(o, "w") as f:
            f.writelines(rows[i::num_shards])
    return outs


def _tokenize_worker(job):
    shard, out, tok_path, stage, cutoff_len, template, packing, sp_size, train_on_prompt = job
    tokenizer = load_tokenizer(tok_path)
    with open(shard) as f:
        examples = [json.loads(line) for line in f]
    pad_id = getattr(tokenizer, "pad_token_id", None) or getattr(tokenizer, "eos_token_id", 0) or 0
    if stage == "pt":
        rows = process_pretrain(examples, tokenizer, cutoff_len)
    else:
        rows = process_supervised(examples, tokenizer, get_template(template), cutoff_len, train_on_prompt)
        if packing:
            rows = pack_supervised(rows, cutoff_len, pad_id)
    shifted = False
    if sp_size > 1:
        rows = preprocess_sp_dataset(rows, sp_size, cutoff_len, pad_id)
        shifted = True
    torch.save({"rows": rows, "labels_shifted": shifted}, out)
    return out, len(rows)


def phase_tokenize(shards: List[str], work: str, data_args: DataArguments, tokenizer_path: Optional[str], stage: str,
                   sp_size: int, workers: int) -> List[str]:
    os.makedirs(os.path.join(work, "tokenized"), exist_ok=True)
    jobs, outs = [], []
    for s in shards:
        out = os.path.join(work, "tokenized", os.path.basename(s).replace(".jsonl", ".pt"))
        outs.append(out)
        if not os.path.exists(out):
            jobs.append((s, out, tokenizer_path, stage, data_args.cutoff_len, data_args.template, data_args.packing,
                         sp_size, data_args.train_on_prompt))
    if jobs:
        with ProcessPoolExecutor(max_workers=workers) as ex:
            list(ex.map(_tokenize_worker, jobs))
    return outs


def phase_concatenate(tokenized: List[str], tokenized_path: str) -> str:
    rows, shifted = [], False
    for t in tokenized:
        d = torch.load(t)
        rows.extend(d["rows"])
        shifted = shifted or d["labels_shifted"]
    ListDataset(rows, shifted).save(tokenized_path)
    return tokenized_path


def run(data_args: DataArguments, tokenizer_path: Optional[str], stage: str = "pt", sp_size: int = 1,
        num_shards: int = 8, workers: int = 4, seed: int = 42) -> str:
    assert data_args.tokenized_path, "tokenized_path must be set for preprocessing"
    work = os.path.join(data_args.tokenized_path, "stages")      # per-phase outputs (restartable)
    aligned = phase_align(data_args, work, workers)
    shards = phase_shard(aligned, work, num_shards, not data_args.disable_shuffling, seed)
    tokenized = phase_tokenize(shards, work, data_args, tokenizer_path, stage, sp_size, workers)
    return phase_concatenate(tokenized, data_args.tokenized_path)


def main(argv=None) -> int:
    from ..config.parser import get_train_args
    ap = argparse.ArgumentParser(prog="hmf preprocess")
    ap.add_argument("--config", required=True)
    ap.add_argument("--num-shards", type=int, default=8)
    ap.add_argument("--workers", type=int, default=4)
    a = ap.parse_args(argv)
    model_args, data_args, run_args, ft_args = get_train_args([a.config])[:4]
    stage = "pt" if ft_args.stage in ("pt", "hkd") else "sft"
    tok_path = model_args.model_name_or_path
    if tok_path and tok_path.strip().startswith("{"):      # inline JSON config: no tokenizer files, byte tokenizer
        tok_path = None
    out = run(data_args, tok_path, stage, model_args.sequence_parallel_size, a.num_shards, a.workers,
              getattr(run_args, "seed", 42))
    print(out)
    return 0
