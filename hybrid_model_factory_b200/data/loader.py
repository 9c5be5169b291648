"""Dataset construction: tokenise -> pack / mask -> (sequence-parallel) pad, shift and zig-zag split
-> batches.

Rows are dicts of equal-length int lists ``input_ids``, ``labels``, ``position_ids`` (and
``attention_mask``).  Under sequence parallelism every sample is padded to ``cutoff_len``, labels are
shifted by one *before* the split, the sequence is cut into ``2*SP`` chunks and rank ``r`` gets chunks
``r`` and ``2*SP-1-r``; the dataset stores the shards of one sample consecutively
(``[s0_r0, s0_r1, ..., s1_r0, ...]``) and rank ``r`` reads row ``i*SP + r``
(reference: ``data/processor/sequence_parallel.py:5-47``, ``data/data_utils.py:255-268``,
``data/loader.py:348-454``, ``data/processor/pretrain.py:27-60``, ``supervised.py:182-215``).
"""
from __future__ import annotations

import os
import random
from typing import Dict, Iterator, List, Optional, Sequence

import torch

from ..config.hparams import DataArguments
from .formats import align_dataset, get_dataset_list, get_template

IGNORE_INDEX = -100


# -- processors ------------------------------------------------------------------------------
def process_pretrain(examples: Sequence[dict], tokenizer, cutoff_len: int) -> List[Dict[str, List[int]]]:
    """Concatenates documents (EOS between them) and cuts blocks of ``cutoff_len`` tokens."""
    eos = getattr(tokenizer, "eos_token_id", None)
    stream: List[int] = []
    for ex in examples:
        text = ex.get("text")
        if text is None:  # chat data used for pre-training: join the turns
            text = "\n".join(m["content"] for m in ex.get("messages", []))
        stream.extend(tokenizer.encode(text, add_special_tokens=False))
        if eos is not None:
            stream.append(eos)
    rows = []
    for s in range(0, len(stream) - cutoff_len + 1, cutoff_len):
        ids = stream[s:s + cutoff_len]
        rows.append({"input_ids": ids, "labels": list(ids), "position_ids": list(range(cutoff_len))})
    return rows


def process_supervised(examples: Sequence[dict], tokenizer, template, cutoff_len: int, train_on_prompt: bool = False,
                       mask_history: bool = False) -> List[Dict[str, List[int]]]:
    rows = []
    for ex in examples:
        pairs = template.encode_multiturn(tokenizer, ex["messages"], ex.get("system", ""))
        ids, labels = [], []
        for t, (p, r) in enumerate(pairs):
            last = t == len(pairs) - 1
            ids += p + r
            labels += (p if train_on_prompt else [IGNORE_INDEX] * len(p))
            labels += r if (last or not mask_history) else [IGNORE_INDEX] * len(r)
        ids, labels = ids[:cutoff_len], labels[:cutoff_len]
        if all(l == IGNORE_INDEX for l in labels):
            continue
        rows.append({"input_ids": ids, "labels": labels, "position_ids": list(range(len(ids)))})
    return rows


def pack_supervised(rows: Sequence[Dict[str, List[int]]], cutoff_len: int, pad_id: int) -> List[Dict[str, List[int]]]:
    """Greedy first-fit packing; position ids restart for every packed sample (continuous per sample)."""
    bins: List[Dict[str, List[int]]] = []
    for row in sorted(rows, key=lambda r: -len(r["input_ids"])):
        n = len(row["input_ids"])
        for b in bins:
            if len(b["input_ids"]) + n <= cutoff_len:
                break
        else:
            b = {"input_ids": [], "labels": [], "position_ids": []}
            bins.append(b)
        b["input_ids"] += row["input_ids"]
        lab = list(row["labels"])
        lab[0] = IGNORE_INDEX  # no loss across a sample boundary
        b["labels"] += lab
        b["position_ids"] += list(range(n))
    for b in bins:
        pad = cutoff_len - len(b["input_ids"])
        b["input_ids"] += [pad_id] * pad
        b["labels"] += [IGNORE_INDEX] * pad
        b["position_ids"] += list(range(pad))
    return bins


# -- sequence-parallel split -------------------------------------------------------------------
def pad_sequence(row: Dict[str, List[int]], cutoff_len: int, pad_id: int) -> Dict[str, List[int]]:
    n = len(row["input_ids"])
    pad = cutoff_len - n
    if pad < 0:
        return {k: v[:cutoff_len] for k, v in row.items()}
    return {"input_ids": row["input_ids"] + [pad_id] * pad, "labels": row["labels"] + [IGNORE_INDEX] * pad,
            "position_ids": row["position_ids"] + list(range(n, n + pad))}


def shift_labels(row: Dict[str, List[int]]) -> Dict[str, List[int]]:
    out = dict(row)
    out["labels"] = row["labels"][1:] + [IGNORE_INDEX]
    return out


def sp_split(row: Dict[str, List[int]], sp_size: int) -> List[Dict[str, List[int]]]:
    """Zig-zag shards of one padded, label-shifted sample, in rank order."""
    L = len(row["input_ids"])
    assert L % (2 * sp_size) == 0, f"length {L} not divisible by 2*SP={2 * sp_size}"
    c = L // (2 * sp_size)
    shards = []
    for r in range(sp_size):
        a, b = r, 2 * sp_size - 1 - r
        shards.append({k: v[a * c:(a + 1) * c] + v[b * c:(b + 1) * c] for k, v in row.items()})
    return shards


def preprocess_sp_dataset(rows: Sequence[Dict[str, List[int]]], sp_size: int, cutoff_len: int, pad_id: int):
    out = []
    for row in rows:
        out.extend(sp_split(shift_labels(pad_sequence(row, cutoff_len, pad_id)), sp_size))
    return out


# -- datasets ---------------------------------------------------------------------------------
class ListDataset(torch.utils.data.Dataset):
    def __init__(self, rows: List[Dict[str, List[int]]], labels_shifted: bool = False):
        self.rows, self.labels_shifted = rows, labels_shifted

    def __len__(self):
        return len(self.rows)

    def __getitem__(self, i):
        return self.rows[i]

    def save(self, path: str) -> None:
        os.makedirs(path, exist_ok=True)
        torch.save({"rows": self.rows, "labels_shifted": self.labels_shifted}, os.path.join(path, "dataset.pt"))

    @classmethod
    def load(cls, path: str) -> "ListDataset":
        d = torch.load(os.path.join(path, "dataset.pt"), weights_only=False)
        return cls(d["rows"], d["labels_shifted"])


class SyntheticDataset(torch.utils.data.Dataset):
    """Uniform random token ids (the benchmark workload); deterministic per index."""

    def __init__(self, vocab_size: int, seq_len: int, length: int = 1 << 30, seed: int = 0):
        self.vocab_size, self.seq_len, self.length, self.seed = vocab_size, seq_len, length, seed
        self.labels_shifted = False

    def __len__(self):
        return self.length

    def __getitem__(self, i):
        g = torch.Generator().manual_seed(self.seed * 1000003 + i)
        ids = torch.randint(0, self.vocab_size, (self.seq_len,), generator=g).tolist()
        return {"input_ids": ids, "labels": list(ids), "position_ids": list(range(self.seq_len))}


def mix_datasets(parts: List[List[dict]], strategy: str = "concat", probs: Optional[List[float]] = None, seed: int = 42):
    if len(parts) == 1 or strategy == "concat":
        return [r for p in parts for r in p]
    rng = random.Random(seed)
    probs = probs or [1.0 / len(parts)] * len(parts)
    iters = [iter(p) for p in parts]
    alive = [True] * len(parts)
    out = []
    if strategy == "interleave_fast":  # round robin until the shortest ends
        n = min(len(p) for p in parts)
        for i in range(n):
            out.extend(p[i] for p in parts)
        return out
    while any(alive):
        k = rng.choices(range(len(parts)), weights=[w if a else 0 for w, a in zip(probs, alive)])[0]
        try:
            out.append(next(iters[k]))
        except StopIteration:
            if strategy == "interleave_under":
                break
            alive[k] = False
    return out


def _encode_prompt_and_answers(ex: dict, tokenizer, template, cutoff_len: int, answers: Sequence[dict]):
    """Token ids of the conversation up to the last user turn, and of each candidate answer."""
    msgs, system = template.normalise(ex["messages"], ex.get("system", ""), ex.get("tools", ""))
    outs = []
    for ans in answers:
        pairs = template.encode_multiturn(tokenizer, list(msgs) + [ans], system)
        prompt = [t for p, r in pairs[:-1] for t in p + r] + pairs[-1][0]
        outs.append((prompt, pairs[-1][1]))
    return outs


def process_pairwise(examples: Sequence[dict], tokenizer, template, cutoff_len: int) -> List[Dict[str, List[int]]]:
    """Preference pairs (``rm`` / ``dpo``): one prompt, a chosen and a rejected answer; labels cover the answers."""
    rows = []
    for ex in examples:
        if "chosen" not in ex or "rejected" not in ex:
            continue
        (pc, rc), (pr, rr) = _encode_prompt_and_answers(ex, tokenizer, template, cutoff_len, [ex["chosen"], ex["rejected"]])
        keep = max(cutoff_len - max(len(rc), len(rr)), cutoff_len // 2)
        pc, pr = pc[-keep:], pr[-keep:]                      # keep the end of a long prompt
        row = {}
        for name, p_ids, r_ids in (("chosen", pc, rc), ("rejected", pr, rr)):
            ids = (p_ids + r_ids)[:cutoff_len]
            lab = ([IGNORE_INDEX] * len(p_ids) + r_ids)[:cutoff_len]
            row[f"{name}_input_ids"], row[f"{name}_labels"] = ids, lab
        rows.append(row)
    return rows


def process_feedback(examples: Sequence[dict], tokenizer, template, cutoff_len: int) -> List[Dict[str, List[int]]]:
    """KTO: single answers tagged desirable / undesirable."""
    rows = []
    for ex, row in zip(examples, process_supervised(examples, tokenizer, template, cutoff_len)):
        row = dict(row)
        row["kto_tags"] = int(bool(ex.get("kto_tag", True)))
        rows.append(row)
    return rows


def process_unsupervised(examples: Sequence[dict], tokenizer, template, cutoff_len: int) -> List[Dict[str, List[int]]]:
    """Generation / evaluation: the prompt (up to the last user turn) as ``input_ids``, the reference answer as
    ``labels``."""
    rows = []
    for ex in examples:
        msgs = list(ex["messages"])
        answer = msgs.pop() if msgs and msgs[-1]["role"] == "assistant" else {"role": "assistant", "content": ""}
        (prompt, resp), = _encode_prompt_and_answers(dict(ex, messages=msgs), tokenizer, template, cutoff_len, [answer])
        rows.append({"input_ids": prompt[-cutoff_len:], "labels": resp[:cutoff_len]})
    return rows


def get_dataset(data_args: DataArguments, tokenizer, stage: str = "pt", sp_size: int = 1, vocab_size: int = 0,
                seed: int = 42) -> torch.utils.data.Dataset:
    """Builds (or loads from ``tokenized_path``) the training dataset for this configuration."""
    pad_id = getattr(tokenizer, "pad_token_id", None)
    if pad_id is None:
        pad_id = getattr(tokenizer, "eos_token_id", 0) or 0
    if data_args.tokenized_path and os.path.exists(os.path.join(data_args.tokenized_path, "dataset.pt")):
        return ListDataset.load(data_args.tokenized_path)
    if data_args.synthetic:
        vs = data_args.synthetic_vocab or vocab_size
        base = SyntheticDataset(vs, data_args.cutoff_len, seed=seed)
        if sp_size == 1:
            return base
        return _SPSynthetic(base, sp_size, pad_id)
    template = get_template(data_args.template)
    parts = []
    for attr in get_dataset_list(data_args.dataset, data_args.dataset_dir):
        examples = align_dataset(attr, data_args.dataset_dir, data_args.max_samples)
        if stage == "pt":
            rows = process_pretrain(examples, tokenizer, data_args.cutoff_len)
        elif stage in ("rm", "dpo"):
            rows = process_pairwise(examples, tokenizer, template, data_args.cutoff_len)
        elif stage == "kto":
            rows = process_feedback(examples, tokenizer, template, data_args.cutoff_len)
        elif stage == "unsupervised":
            rows = process_unsupervised(examples, tokenizer, template, data_args.cutoff_len)
        else:
            rows = process_supervised(examples, tokenizer, template, data_args.cutoff_len, data_args.train_on_prompt,
                                      data_args.mask_history)
            if data_args.packing or data_args.neat_packing:
                rows = pack_supervised(rows, data_args.cutoff_len, pad_id)
        parts.append(rows)
    probs = [float(x) for x in data_args.interleave_probs.split(",")] if data_args.interleave_probs else None
    rows = mix_datasets(parts, data_args.mix_strategy, probs, seed)
    if not data_args.disable_shuffling and sp_size == 1:
        random.Random(seed).shuffle(rows)
    shifted = False
    if sp_size > 1:
        rows = preprocess_sp_dataset(rows, sp_size, data_args.cutoff_len, pad_id)
        shifted = True
    ds = ListDataset(rows, shifted)
    ds.neat_packing = bool(getattr(data_args, "neat_packing", False)) and sp_size == 1
    if data_args.tokenized_path:
        ds.save(data_args.tokenized_path)
    return ds


class _SPSynthetic(torch.utils.data.Dataset):
    def __init__(self, base: SyntheticDataset, sp_size: int, pad_id: int):
        self.base, self.sp, self.pad_id, self.labels_shifted = base, sp_size, pad_id, True

    def __len__(self):
        return len(self.base) * self.sp

    def __getitem__(self, i):
        row = shift_labels(self.base[i // self.sp])
        return sp_split(row, self.sp)[i % self.sp]


# -- batching ------------------------------------------------------------------------------------
def collate(rows: Sequence[Dict[str, List[int]]], pad_id: int = 0, pin: bool = False) -> Dict[str, torch.Tensor]:
    """Pads every list-valued column to the batch maximum (``*labels`` with the ignore index, ``*input_ids`` with the
    pad id, the rest with 0); scalar columns (``kto_tags``) become 1-D tensors."""
    batch = {}
    for key in rows[0]:
        vals = [r[key] for r in rows]
        if isinstance(vals[0], (list, tuple)):
            L = max(len(v) for v in vals)
            fill = IGNORE_INDEX if key.endswith("labels") else (pad_id if key.endswith("input_ids") else 0)
            batch[key] = torch.tensor([list(v) + [fill] * (L - len(v)) for v in vals], dtype=torch.long)
        else:
            batch[key] = torch.tensor(vals, dtype=torch.long)
    if pin and torch.cuda.is_available():
        batch = {k: v.pin_memory() for k, v in batch.items()}
    return batch


def steps_per_epoch(n_rows: int, batch_size: int, world: int = 1, sp_size: int = 1) -> int:
    """Optimizer steps in one pass over the data: the same number on every rank (a tail that does not fill one batch
    on every data-parallel replica is dropped)."""
    dp = max(1, world // sp_size)
    return (n_rows // sp_size) // (dp * batch_size)


def batch_iterator(dataset, batch_size: int, rank: int = 0, world: int = 1, sp_size: int = 1, pad_id: int = 0,
                   start_step: int = 0, pin: bool = True, num_epochs: Optional[float] = None, shuffle: bool = False,
                   seed: int = 0) -> Iterator[Dict[str, torch.Tensor]]:
    """Deterministic batches, epoch after epoch.  With SP the dataset rows are already interleaved per rank:
    in step ``s`` of an epoch data-parallel replica ``d`` and SP rank ``r`` read samples ``(s*dp + d)*B + j`` (row
    ``sample*SP + r``).  Every rank sees the same number of steps per epoch, so no rank runs out of batches before
    another (ranks that disagreed would issue mismatched collectives).  ``num_epochs`` ends the stream (``None``: it
    wraps around for as long as the trainer asks, which stops at ``max_steps``); epochs after the first draw the
    samples in a fresh order when ``shuffle`` is set (reference: the per-epoch sampler seed of its trainer), the first
    keeps the dataset's own order.  Resuming is skipping ``start_step`` steps."""
    dp = max(1, world // sp_size)
    d, r = rank // sp_size, rank % sp_size
    n_samples = len(dataset) // sp_size
    spe = steps_per_epoch(len(dataset), batch_size, world, sp_size)
    if spe == 0:
        return
    total = None if num_epochs is None else int(round(num_epochs * spe))
    labels_shifted = bool(getattr(dataset, "labels_shifted", False))
    step, cur_epoch, order = start_step, -1, None
    while total is None or step < total:
        epoch, s = divmod(step, spe)
        if epoch != cur_epoch:
            cur_epoch = epoch
            order = None
            if shuffle and epoch > 0:
                g = torch.Generator().manual_seed(seed + epoch)
                order = torch.randperm(n_samples, generator=g).tolist()
        first = (s * dp + d) * batch_size
        ids = range(first, first + batch_size)
        rows = [dataset[(order[i] if order is not None else i) * sp_size + r] for i in ids]
        batch = collate(rows, pad_id, pin)
        batch["labels_shifted"] = labels_shifted
        if getattr(dataset, "neat_packing", False) and batch_size == 1 and "position_ids" in rows[0]:
            # packed samples must not attend to one another: sample boundaries are where the position ids restart
            from .collator import indices_from_position_ids, segment_boundaries
            seg = indices_from_position_ids(rows[0]["position_ids"], len(rows[0]["position_ids"]))
            batch["cu_seqlens"] = segment_boundaries(torch.tensor([seg]))
        yield batch
        step += 1
