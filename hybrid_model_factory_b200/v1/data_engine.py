"""``DataEngine``: several datasets behind one index.

The dataset description is a mapping ``name -> {path, source, converter, size, weight, split}`` (a YAML / JSON
file, a dict, or one local file / directory of records, which becomes the dataset ``default``).  Every sample is
addressed by ``(dataset name, row)``; ``size`` resamples a dataset to exactly that many entries of the index and
``weight`` scales its share, so mixtures are fixed at construction time and reproducible.  A sample comes out in the
unified form ``{"_dataset_name", "messages": [{"role", "content", "loss_weight"}], ...}``.
Reference: ``v1/core/data_engine.py:47-174`` and ``v1/plugins/data_plugins/{loader,converter}.py``."""
from __future__ import annotations

import json
import os
from typing import Any, Dict, List, Sequence, Tuple, Union

import torch

from .plugin import DataConverter


def _read_records(path: str) -> List[dict]:
    if os.path.isdir(path):
        out: List[dict] = []
        for f in sorted(os.listdir(path)):
            if f.endswith((".json", ".jsonl")):
                out += _read_records(os.path.join(path, f))
        return out
    with open(path, encoding="utf-8") as fh:
        if path.endswith(".jsonl"):
            return [json.loads(line) for line in fh if line.strip()]
        data = json.load(fh)
    return data if isinstance(data, list) else data.get("data", [data])


def convert_alpaca(rec: dict) -> dict:
    """``instruction / input / output (/ system)`` records."""
    user = rec.get("instruction", "")
    if rec.get("input"):
        user = f"{user}\n{rec['input']}" if user else rec["input"]
    msgs = []
    if rec.get("system"):
        msgs.append({"role": "system", "content": rec["system"], "loss_weight": 0.0})
    msgs.append({"role": "user", "content": user, "loss_weight": 0.0})
    msgs.append({"role": "assistant", "content": rec.get("output", ""), "loss_weight": 1.0})
    return {"messages": msgs}


def convert_sharegpt(rec: dict) -> dict:
    """``conversations: [{from, value}]`` records."""
    roles = {"human": "user", "user": "user", "gpt": "assistant", "assistant": "assistant", "system": "system",
             "function_call": "assistant", "observation": "user", "tool": "user"}
    msgs = []
    for turn in rec.get("conversations", []):
        role = roles.get(turn.get("from", turn.get("role", "user")), "user")
        msgs.append({"role": role, "content": turn.get("value", turn.get("content", "")),
                     "loss_weight": 1.0 if role == "assistant" else 0.0})
    return {"messages": msgs}


def convert_pair(rec: dict) -> dict:
    """Preference records: ``chosen`` / ``rejected`` answers to one prompt."""
    base = convert_alpaca({**rec, "output": ""})["messages"][:-1] if "instruction" in rec else \
        [{"role": "user", "content": rec.get("prompt", ""), "loss_weight": 0.0}]
    mk = lambda text: base + [{"role": "assistant", "content": text, "loss_weight": 1.0}]  # noqa: E731
    return {"chosen_messages": mk(rec["chosen"]), "rejected_messages": mk(rec["rejected"])}


for _name, _fn in (("alpaca", convert_alpaca), ("sharegpt", convert_sharegpt), ("pair", convert_pair)):
    DataConverter(_name).register(replace=True)(_fn)


def adjust_data_index(index: List[Tuple[str, int]], size=None, weight=None) -> List[Tuple[str, int]]:
    """``size``: repeat / truncate to exactly that many entries; ``weight``: scale the count by that factor."""
    if size:
        reps = -(-int(size) // max(len(index), 1))
        index = (index * reps)[:int(size)]
    if weight:
        n = int(round(len(index) * float(weight)))
        reps = -(-n // max(len(index), 1))
        index = (index * reps)[:n]
    return index


class DataEngine(torch.utils.data.Dataset):
    def __init__(self, dataset: Union[str, Dict[str, dict]]):
        self.dataset_infos: Dict[str, dict] = self._infos(dataset)
        self.datasets: Dict[str, Sequence[dict]] = {}
        self.data_index: List[Tuple[str, int]] = []
        for name, info in self.dataset_infos.items():
            source = info.get("source", "local")
            if source == "local":
                self.datasets[name] = _read_records(info["path"])
            elif source == "memory":
                self.datasets[name] = info["records"]
            elif source == "hf_hub":
                from datasets import load_dataset           # optional dependency, needs network access
                self.datasets[name] = load_dataset(info["path"], split=info.get("split", "train"))
            else:
                raise ValueError(f"dataset {name}: unknown source '{source}'")
            idx = [(name, i) for i in range(len(self.datasets[name]))]
            self.data_index += adjust_data_index(idx, info.get("size"), info.get("weight"))

    @staticmethod
    def _infos(dataset) -> Dict[str, dict]:
        if isinstance(dataset, dict):
            return dataset
        if dataset.endswith((".yaml", ".yml")) and os.path.isfile(dataset):
            import yaml
            with open(dataset) as fh:
                infos = yaml.safe_load(fh)
            base = os.path.dirname(os.path.abspath(dataset))
            for info in infos.values():       # paths in the file are relative to it
                if info.get("source", "local") == "local" and not os.path.isabs(info["path"]):
                    info["path"] = os.path.join(base, info["path"])
            return infos
        if os.path.exists(dataset):
            return {"default": {"path": dataset, "source": "local"}}
        return {"default": {"path": dataset, "source": "hf_hub"}}

    def __len__(self) -> int:
        return len(self.data_index)

    def _convert(self, raw: dict, name: str) -> dict:
        conv = self.dataset_infos[name].get("converter")
        out = DataConverter(conv)(raw) if conv else dict(raw)
        out["_dataset_name"] = name
        return out

    def __getitem__(self, index: Union[int, slice, Sequence[int]]) -> Any:
        if isinstance(index, int):
            name, i = self.data_index[index]
            return self._convert(self.datasets[name][i], name)
        picks = self.data_index[index] if isinstance(index, slice) else [self.data_index[i] for i in index]
        return [self._convert(self.datasets[n][i], n) for n, i in picks]
