"""``BatchGenerator``: an iterator over optimizer steps (each a list of micro-batches) whose position can be saved and
restored exactly.

Order: a permutation of the dataset drawn from ``seed + epoch``, strided over the data-parallel ranks, so every rank
sees the same number of samples and no rank runs out before another.  Strategies:

* ``normal``: ``micro_batch_size`` rows per micro-batch, padded to the longest;
* ``padding_free``: the rows of a micro-batch are concatenated into one row with ``cu_seqlens`` (no pad tokens; the
  mixers treat the samples independently);
* ``dynamic``: samples are taken while the step stays within ``token_budget`` tokens (rendered samples wait in a
  buffer, which is part of the saved state), split into ``num_micro_batch`` micro-batches of about equal tokens.

State = ``(epoch, cursor, buffer)``; ``load_state_dict`` followed by iteration continues with the very next step.
Reference: ``v1/core/utils/batching.py:62-213`` (which implements the first strategy and names the others)."""
from __future__ import annotations

import copy
from typing import Any, Dict, Iterator, List, Optional, Sequence

import torch

from .plugin import BatchingStrategy

IGNORE_INDEX = -100


class StatefulBuffer:
    """FIFO of rendered samples with a running token count."""

    def __init__(self):
        self.items: List[dict] = []

    def __len__(self) -> int:
        return len(self.items)

    @property
    def tokens(self) -> int:
        return sum(len(s["input_ids"]) for s in self.items)

    def put(self, samples: Sequence[dict]) -> None:
        self.items.extend(samples)

    def get(self, n: int) -> List[dict]:
        out, self.items = self.items[:n], self.items[n:]
        return out

    def clear(self) -> None:
        self.items = []

    def state_dict(self) -> dict:
        return {"items": copy.deepcopy(self.items)}

    def load_state_dict(self, state: dict) -> None:
        self.items = copy.deepcopy(state["items"])


def pad_collate(rows: Sequence[dict], pad_id: int = 0) -> Dict[str, torch.Tensor]:
    n = max(len(r["input_ids"]) for r in rows)
    ids = torch.full((len(rows), n), pad_id, dtype=torch.long)
    labels = torch.full((len(rows), n), IGNORE_INDEX, dtype=torch.long)
    mask = torch.zeros(len(rows), n, dtype=torch.long)
    for i, r in enumerate(rows):
        m = len(r["input_ids"])
        ids[i, :m] = torch.tensor(r["input_ids"])
        labels[i, :m] = torch.tensor(r["labels"])
        mask[i, :m] = 1
    return {"input_ids": ids, "labels": labels, "attention_mask": mask}


def packed_collate(rows: Sequence[dict]) -> Dict[str, Any]:
    """One row without padding; ``cu_seqlens`` marks the sample boundaries, positions restart at every sample and the
    first label of every sample but the first is masked (it would be predicted from the previous sample)."""
    ids, labels, pos, cu = [], [], [], [0]
    for r in rows:
        lab = list(r["labels"])
        if ids and lab:
            lab[0] = IGNORE_INDEX
        ids += r["input_ids"]
        labels += lab
        pos += list(range(len(lab)))
        cu.append(len(ids))
    return {"input_ids": torch.tensor([ids]), "labels": torch.tensor([labels]), "position_ids": torch.tensor([pos]),
            "cu_seqlens": cu}


class BatchGenerator(Iterator):
    def __init__(self, dataset, renderer, micro_batch_size: int = 1, global_batch_size: Optional[int] = None,
                 strategy: str = "normal", token_budget: int = 0, dp_rank: int = 0, dp_size: int = 1, seed: int = 0,
                 pad_id: int = 0, shuffle: bool = True):
        if strategy not in ("normal", "padding_free", "dynamic") and not BatchingStrategy.has(strategy):
            raise ValueError(f"unknown batching strategy '{strategy}' (built in: normal, padding_free, dynamic; "
                             f"registered: {', '.join(BatchingStrategy.names()) or 'none'})")
        if strategy == "dynamic" and token_budget <= 0:
            raise ValueError("the dynamic strategy needs token_budget > 0")
        self.dataset, self.renderer = dataset, renderer
        self.micro_batch_size, self.strategy, self.token_budget = micro_batch_size, strategy, token_budget
        self.dp_rank, self.dp_size, self.seed, self.pad_id, self.shuffle = dp_rank, dp_size, seed, pad_id, shuffle
        gbs = global_batch_size or dp_size * micro_batch_size
        if gbs % (dp_size * micro_batch_size):
            raise ValueError(f"global batch size {gbs} is not a multiple of dp size {dp_size} x micro batch "
                             f"{micro_batch_size}")
        self.num_micro_batch = gbs // dp_size // micro_batch_size
        self.per_rank = len(dataset) // dp_size                      # drop_last over the ranks
        self.epoch, self.cursor = 0, 0
        self.buffer = StatefulBuffer()
        self._order: Optional[List[int]] = None

    # -- order -------------------------------------------------------------------------------------
    def set_epoch(self, epoch: int) -> None:
        if epoch != self.epoch:
            self.epoch, self.cursor, self._order = epoch, 0, None
            self.buffer.clear()

    def _indices(self) -> List[int]:
        if self._order is None:
            n = len(self.dataset)
            if self.shuffle:
                g = torch.Generator().manual_seed(self.seed + self.epoch)
                perm = torch.randperm(n, generator=g).tolist()
            else:
                perm = list(range(n))
            self._order = perm[self.dp_rank:self.per_rank * self.dp_size:self.dp_size]
        return self._order

    def __len__(self) -> int:
        """Steps per epoch (exact for the fixed-size strategies, an upper bound for ``dynamic``)."""
        return self.per_rank // (self.micro_batch_size * self.num_micro_batch)

    # -- iteration -----------------------------------------------------------------------------------
    def __iter__(self):
        return self

    def _pull(self, n: int) -> bool:
        order = self._indices()
        take = order[self.cursor:self.cursor + n]
        if not take:
            return False
        self.cursor += len(take)
        self.buffer.put(self.renderer.process_samples(self.dataset[take]))
        return True

    def __next__(self) -> List[Dict[str, Any]]:
        per_step = self.micro_batch_size * self.num_micro_batch
        if self.strategy == "dynamic":
            while self.buffer.tokens < self.token_budget and self._pull(per_step):
                pass
            rows, used = [], 0
            while len(self.buffer) and (not rows or used + len(self.buffer.items[0]["input_ids"]) <= self.token_budget):
                r = self.buffer.get(1)[0]
                rows.append(r)
                used += len(r["input_ids"])
            if not rows:
                raise StopIteration
            return [packed_collate(g) for g in self._split_even(rows, self.num_micro_batch)]
        while len(self.buffer) < per_step and self._pull(per_step - len(self.buffer)):
            pass
        if len(self.buffer) < per_step:                              # drop the ragged tail of the epoch
            self.buffer.clear()
            raise StopIteration
        rows = self.buffer.get(per_step)
        groups = [rows[i * self.micro_batch_size:(i + 1) * self.micro_batch_size] for i in range(self.num_micro_batch)]
        if self.strategy == "padding_free":
            return [packed_collate(g) for g in groups]
        if self.strategy != "normal":
            return BatchingStrategy(self.strategy)(rows, self)
        return [pad_collate(g, self.pad_id) for g in groups]

    @staticmethod
    def _split_even(rows: List[dict], parts: int) -> List[List[dict]]:
        """Greedy split into ``parts`` groups of about equal token counts (longest first); empty groups are dropped."""
        groups: List[List[dict]] = [[] for _ in range(parts)]
        loads = [0] * parts
        for r in sorted(rows, key=lambda r: -len(r["input_ids"])):
            i = loads.index(min(loads))
            groups[i].append(r)
            loads[i] += len(r["input_ids"])
        return [g for g in groups if g]

    # -- state ---------------------------------------------------------------------------------------
    def state_dict(self) -> dict:
        return {"epoch": self.epoch, "cursor": self.cursor, "seed": self.seed, "buffer": self.buffer.state_dict()}

    def load_state_dict(self, state: dict) -> None:
        self.epoch, self.cursor, self.seed = state["epoch"], state["cursor"], state["seed"]
        self._order = None
        self.buffer.load_state_dict(state["buffer"])
