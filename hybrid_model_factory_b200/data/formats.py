"""Dataset registry, format converters and chat templates.

* ``dataset_info.json`` (same schema as the reference's ``data/dataset_info.json``): per dataset a
  ``file_name`` (json / jsonl / txt / parquet), ``formatting`` (``alpaca`` | ``sharegpt`` | ``text``) and
  optional ``columns`` / ``tags`` remappings.
* Converters normalise every example to ``{"messages": [{"role", "content"}...], "system": str}`` or
  ``{"text": str}`` for pre-training corpora (reference: ``data/parser.py``, ``data/converter.py``).
* Templates render messages to token ids and tell which spans are supervised
  (reference: ``data/template.py``, ``data/formatter.py``).
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass, field
from typing import Any, Dict, Iterable, Iterator, List, Optional, Sequence, Tuple


# ----------------------------------------------------------------------------------------
# registry
# ----------------------------------------------------------------------------------------
@dataclass
class DatasetAttr:
    name: str
    file_name: str
    formatting: str = "alpaca"
    columns: Dict[str, str] = field(default_factory=dict)
    tags: Dict[str, str] = field(default_factory=dict)
    split: str = "train"
    num_samples: Optional[int] = None


def load_dataset_info(dataset_dir: str) -> Dict[str, dict]:
    path = os.path.join(dataset_dir, "dataset_info.json")
    if not os.path.exists(path):
        return {}
    with open(path) as f:
        return json.load(f)


def get_dataset_list(names: Optional[str], dataset_dir: str) -> List[DatasetAttr]:
    if not names:
        return []
    info = load_dataset_info(dataset_dir)
    out = []
    for name in [n.strip() for n in names.split(",") if n.strip()]:
        if name in info:
            e = info[name]
            out.append(DatasetAttr(name, e.get("file_name", name), e.get("formatting", "alpaca"),
                                   e.get("columns", {}), e.get("tags", {}), e.get("split", "train"),
                                   e.get("num_samples")))
        elif os.path.exists(os.path.join(dataset_dir, name)) or os.path.exists(name):
            fmt = "text" if name.endswith(".txt") else "alpaca"
            out.append(DatasetAttr(os.path.basename(name), name, fmt))
        else:
            raise ValueError(f"dataset '{name}' is neither in {dataset_dir}/dataset_info.json nor a file")
    return out


def read_records(attr: DatasetAttr, dataset_dir: str) -> Iterator[dict]:
    path = attr.file_name if os.path.isabs(attr.file_name) or os.path.exists(attr.file_name) \
        else os.path.join(dataset_dir, attr.file_name)
    if path.endswith(".jsonl"):
        with open(path) as f:
            for line in f:
                if line.strip():
                    yield json.loads(line)
    elif path.endswith(".json"):
        with open(path) as f:
            for rec in json.load(f):
                yield rec
    elif path.endswith(".txt"):
        with open(path) as f:
            for line in f:
                if line.strip():
                    yield {"text": line.rstrip("\n")}
    elif path.endswith(".parquet"):
        import pyarrow.parquet as pq
        for rec in pq.read_table(path).to_pylist():
            yield rec
    else:
        raise ValueError(f"unsupported dataset file type: {path}")


# ----------------------------------------------------------------------------------------
# converters
# ----------------------------------------------------------------------------------------
def convert_alpaca(rec: dict, attr: DatasetAttr) -> dict:
    c = {"prompt": "instruction", "query": "input", "response": "output", "system": "system", "history": "history"}
    c.update(attr.columns)
    messages = []
    for turn in rec.get(c["history"]) or []:
        messages += [{"role": "user", "content": turn[0]}, {"role": "assistant", "content": turn[1]}]
    prompt = rec.get(c["prompt"], "") or ""
    if rec.get(c["query"]):
        prompt = f"{prompt}\n{rec[c['query']]}" if prompt else rec[c["query"]]
    messages.append({"role": "user", "content": prompt})
    messages.append({"role": "assistant", "content": rec.get(c["response"], "") or ""})
    return {"messages": messages, "system": rec.get(c["system"], "") or ""}


def convert_sharegpt(rec: dict, attr: DatasetAttr) -> dict:
    c = {"messages": "conversations", "system": "system"}
    c.update(attr.columns)
    t = {"role_tag": "from", "content_tag": "value", "user_tag": "human", "assistant_tag": "gpt", "system_tag": "system"}
    t.update(attr.tags)
    system = rec.get(c["system"], "") or ""
    messages = []
    for m in rec.get(c["messages"], []):
        role = m.get(t["role_tag"])
        content = m.get(t["content_tag"], "")
        if role == t["system_tag"]:
            system = content
        elif role in (t["user_tag"], "user"):
            messages.append({"role": "user", "content": content})
        elif role in (t["assistant_tag"], "assistant"):
            messages.append({"role": "assistant", "content": content})
        else:
            messages.append({"role": str(role), "content": content})
    return {"messages": messages, "system": system}


def convert_text(rec: dict, attr: DatasetAttr) -> dict:
    col = attr.columns.get("prompt", "text")
    return {"text": rec.get(col, "")}


CONVERTERS = {"alpaca": convert_alpaca, "sharegpt": convert_sharegpt, "openai": convert_sharegpt, "text": convert_text}


def align_dataset(attr: DatasetAttr, dataset_dir: str, max_samples: Optional[int] = None) -> List[dict]:
    conv = CONVERTERS[attr.formatting]
    out = []
    for i, rec in enumerate(read_records(attr, dataset_dir)):
        if max_samples is not None and i >= max_samples:
            break
        out.append(conv(rec, attr))
    return out


# ----------------------------------------------------------------------------------------
# templates
# ----------------------------------------------------------------------------------------
@dataclass
class Template:
    name: str
    system_fmt: str = "{content}\n"
    user_fmt: str = "Human: {content}\nAssistant:"
    assistant_fmt: str = "{content}\n"
    default_system: str = ""
    add_bos: bool = False
    efficient_eos: bool = True   # append the tokenizer's EOS after each assistant turn

    def encode_multiturn(self, tokenizer, messages: Sequence[dict], system: str = "") -> List[Tuple[List[int], List[int]]]:
        """Returns ``[(prompt_ids, response_ids), ...]`` per user/assistant exchange."""
        pairs = []
        prefix = ""
        sys_text = system or self.default_system
        if sys_text:
            prefix = self.system_fmt.format(content=sys_text)
        i = 0
        first = True
        while i < len(messages):
            user = messages[i]["content"] if messages[i]["role"] != "assistant" else ""
            if messages[i]["role"] != "assistant":
                i += 1
            answer = ""
            if i < len(messages) and messages[i]["role"] == "assistant":
                answer = messages[i]["content"]
                i += 1
            prompt_text = (prefix if first else "") + self.user_fmt.format(content=user)
            p_ids = tokenizer.encode(prompt_text, add_special_tokens=False)
            if first and self.add_bos and getattr(tokenizer, "bos_token_id", None) is not None:
                p_ids = [tokenizer.bos_token_id] + p_ids
            r_ids = tokenizer.encode(self.assistant_fmt.format(content=answer), add_special_tokens=False)
            if self.efficient_eos and getattr(tokenizer, "eos_token_id", None) is not None:
                r_ids = r_ids + [tokenizer.eos_token_id]
            pairs.append((p_ids, r_ids))
            first = False
        return pairs


TEMPLATES: Dict[str, Template] = {
    "default": Template("default"),
    "empty": Template("empty", system_fmt="{content}", user_fmt="{content}", assistant_fmt="{content}"),
    "chatml": Template("chatml", system_fmt="<|im_start|>system\n{content}<|im_end|>\n",
                       user_fmt="<|im_start|>user\n{content}<|im_end|>\n<|im_start|>assistant\n",
                       assistant_fmt="{content}<|im_end|>\n", efficient_eos=False),
    "qwen": Template("qwen", system_fmt="<|im_start|>system\n{content}<|im_end|>\n",
                     user_fmt="<|im_start|>user\n{content}<|im_end|>\n<|im_start|>assistant\n",
                     assistant_fmt="{content}<|im_end|>\n", default_system="You are a helpful assistant.",
                     efficient_eos=False),
    "qwen3": Template("qwen3", system_fmt="<|im_start|>system\n{content}<|im_end|>\n",
                      user_fmt="<|im_start|>user\n{content}<|im_end|>\n<|im_start|>assistant\n",
                      assistant_fmt="{content}<|im_end|>\n", efficient_eos=False),
    "llama3": Template("llama3", system_fmt="<|start_header_id|>system<|end_header_id|>\n\n{content}<|eot_id|>",
                       user_fmt="<|start_header_id|>user<|end_header_id|>\n\n{content}<|eot_id|>"
                                "<|start_header_id|>assistant<|end_header_id|>\n\n",
                       assistant_fmt="{content}<|eot_id|>", add_bos=True, efficient_eos=False),
    "mistral": Template("mistral", system_fmt="{content}\n\n", user_fmt="[INST] {content}[/INST]",
                        assistant_fmt=" {content}", add_bos=True),
}


def get_template(name: Optional[str]) -> Template:
    if not name:
        return TEMPLATES["default"]
    if name not in TEMPLATES:
        raise ValueError(f"unknown template '{name}'; available: {sorted(TEMPLATES)}")
    return TEMPLATES[name]


class ByteTokenizer:
    """Dependency-free byte-level tokenizer (ids 0..255 + bos/eos/pad) for tests and synthetic runs."""
    bos_token_id, eos_token_id, pad_token_id = 256, 257, 258
    vocab_size = 259

    def encode(self, text: str, add_special_tokens: bool = False) -> List[int]:
        ids = list(text.encode("utf-8"))
        return ([self.bos_token_id] + ids) if add_special_tokens else ids

    def decode(self, ids: Iterable[int], skip_special_tokens: bool = True) -> str:
        return bytes(i for i in ids if i < 256).decode("utf-8", errors="replace")

    def __call__(self, text, **kw):
        return {"input_ids": self.encode(text)}


def load_tokenizer(path: Optional[str]):
    """HF tokenizer when ``path`` holds one, else the byte tokenizer."""
    if path and any(os.path.exists(os.path.join(path, f)) for f in ("tokenizer.json", "tokenizer_config.json", "tokenizer.model")):
        from transformers import AutoTokenizer
        return AutoTokenizer.from_pretrained(path)
    return ByteTokenizer()
