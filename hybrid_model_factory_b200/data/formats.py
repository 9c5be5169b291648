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
from typing import Dict, Iterable, Iterator, List, Optional, Sequence, Tuple


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
    ranking: bool = False              # preference data: ``chosen`` / ``rejected`` answers
    hf_hub_url: Optional[str] = None   # load with ``datasets.load_dataset`` instead of from a local file
    subset: Optional[str] = None
    streaming: bool = False


PACKAGED_CATALOGUE = os.path.join(os.path.dirname(os.path.abspath(__file__)), "dataset_info.json")


def load_dataset_info(dataset_dir: str) -> Dict[str, dict]:
    """The catalogue shipped with the package (well-known instruction, preference and long-context text datasets by
    hub name), overlaid by ``<dataset_dir>/dataset_info.json`` when the user provides one."""
    info: Dict[str, dict] = {}
    for path in (PACKAGED_CATALOGUE, os.path.join(dataset_dir, "dataset_info.json")):
        if os.path.exists(path):
            with open(path) as f:
                info.update(json.load(f))
    return info


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
                                   e.get("num_samples"), bool(e.get("ranking", False)), e.get("hf_hub_url"),
                                   e.get("subset"), bool(e.get("streaming", False))))
        elif os.path.exists(os.path.join(dataset_dir, name)) or os.path.exists(name):
            fmt = "text" if name.endswith(".txt") else "alpaca"
            out.append(DatasetAttr(os.path.basename(name), name, fmt))
        else:
            raise ValueError(f"dataset '{name}' is neither in {dataset_dir}/dataset_info.json nor a file")
    return out


def read_records(attr: DatasetAttr, dataset_dir: str) -> Iterator[dict]:
    local = attr.file_name if os.path.isabs(attr.file_name) or os.path.exists(attr.file_name) \
        else os.path.join(dataset_dir, attr.file_name)
    if attr.hf_hub_url and not os.path.exists(local):
        try:
            import datasets
            ds = datasets.load_dataset(attr.hf_hub_url, attr.subset, split=attr.split, streaming=attr.streaming)
        except Exception as e:  # noqa: BLE001  (offline machine, missing package, gated dataset)
            raise RuntimeError(f"dataset '{attr.name}' is a hub dataset ({attr.hf_hub_url}) and could not be loaded: "
                               f"{type(e).__name__}: {e}; place a local copy under {dataset_dir} and set file_name") from e
        for i, rec in enumerate(ds):
            if attr.num_samples is not None and i >= attr.num_samples:
                break
            yield rec
        return
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
    out = {"system": rec.get(c["system"], "") or ""}
    chosen_col, rejected_col = c.get("chosen", "chosen"), c.get("rejected", "rejected")
    if (attr.ranking or chosen_col in rec) and rejected_col in rec:       # preference pair: two answers to one prompt
        out["messages"] = messages
        out["chosen"] = {"role": "assistant", "content": rec.get(chosen_col, "") or ""}
        out["rejected"] = {"role": "assistant", "content": rec.get(rejected_col, "") or ""}
        return out
    messages.append({"role": "assistant", "content": rec.get(c["response"], "") or ""})
    out["messages"] = messages
    kto_col = c.get("kto_tag", "kto_tag")
    if kto_col in rec:                                                    # KTO feedback: desirable / undesirable
        out["kto_tag"] = bool(rec[kto_col])
    return out


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
        elif role in (t.get("function_tag", "function_call"), "function_call", "tool_calls"):
            messages.append({"role": "function", "content": content})
        elif role in (t.get("observation_tag", "observation"), "observation", "tool"):
            messages.append({"role": "observation", "content": content})
        else:
            messages.append({"role": str(role), "content": content})
    out = {"messages": messages, "system": system, "tools": rec.get(c.get("tools", "tools"), "") or ""}
    chosen_col, rejected_col = c.get("chosen", "chosen"), c.get("rejected", "rejected")
    if (attr.ranking or chosen_col in rec) and rejected_col in rec:

        def one(m):
            if isinstance(m, dict):
                return {"role": "assistant", "content": m.get(t["content_tag"], m.get("content", ""))}
            return {"role": "assistant", "content": str(m)}
        out["chosen"], out["rejected"] = one(rec[chosen_col]), one(rec[rejected_col])
    kto_col = c.get("kto_tag", "kto_tag")
    if kto_col in rec:
        out["kto_tag"] = bool(rec[kto_col])
    return out


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
# How a model family writes tools: the tool list in the system prompt, an assistant turn that calls functions, the
# results shown back to it, and how calls are recognised in generated text ("xml": blocks between the two halves of
# ``function``; "json": the answer is a JSON object, or several separated by ";", with ``name`` and ``parameters``;
# "prefixed_list": a marker followed by a JSON list of calls).  ``joined``: all calls of a turn are one JSON list inside
# one ``function`` block instead of one block per call.  Reference: the per-family tool formats of
# ``data/tool_utils.py`` (default / qwen, llama3, mistral, glm4).
TOOL_FORMATS: Dict[str, dict] = {
    "qwen": dict(function="<tool_call>\n{content}\n</tool_call>", observation="<tool_response>\n{content}\n</tool_response>",
                 tools=("\n\n# Tools\n\nYou may call one or more functions to assist with the user query.\n"
                        "<tools>\n{content}\n</tools>\nFor each function call, return a json object with function "
                        "name and arguments within <tool_call></tool_call> XML tags."), extract="xml", joined=False,
                 arguments_key="arguments"),
    "llama3": dict(function="{content}", observation="{content}",
                   tools=("\n\nYou have access to the following functions. To call a function, please respond with JSON "
                          "for a function call. Respond in the format {{\"name\": function name, \"parameters\": dictionary "
                          "of argument name and its value}}. Do not use variables.\n\n{content}"), extract="json",
                   joined=False, arguments_key="parameters"),
    "mistral": dict(function="[TOOL_CALLS] {content}", observation="[TOOL_RESULTS] {{\"content\": {content}}}[/TOOL_RESULTS]",
                    tools="[AVAILABLE_TOOLS] {content}[/AVAILABLE_TOOLS]", extract="prefixed_list", joined=True,
                    arguments_key="arguments"),
    "glm4": dict(function="{content}", observation="<|observation|>\n{content}",
                 tools=("\n\n# 可用工具\n{content}\n在调用上述函数时，请使用 Json 格式表示调用的参数。"), extract="name_then_json",
                 joined=False, arguments_key="arguments"),
}


@dataclass
class Template:
    name: str
    system_fmt: str = "{content}\n"
    user_fmt: str = "Human: {content}\nAssistant:"
    assistant_fmt: str = "{content}\n"
    default_system: str = ""
    add_bos: bool = False
    efficient_eos: bool = True   # append the tokenizer's EOS after each assistant turn
    function_fmt: str = "<tool_call>\n{content}\n</tool_call>"            # assistant turn that calls tools
    observation_fmt: str = "<tool_response>\n{content}\n</tool_response>"  # tool results, shown as a user turn
    tools_fmt: str = ("\n\n# Tools\n\nYou may call one or more functions to assist with the user query.\n"
                      "<tools>\n{content}\n</tools>\nFor each function call, return a json object with function "
                      "name and arguments within <tool_call></tool_call> XML tags.")

    tool_format: str = "qwen"

    def __post_init__(self):
        spec = TOOL_FORMATS.get(self.tool_format)
        if spec is None:
            raise ValueError(f"template {self.name}: unknown tool format '{self.tool_format}' ({sorted(TOOL_FORMATS)})")
        if self.tool_format != "qwen":      # the family's own way of writing tools
            self.function_fmt, self.observation_fmt, self.tools_fmt = spec["function"], spec["observation"], spec["tools"]

    def _render_calls(self, calls: list) -> str:
        """Text of an assistant turn that makes ``calls`` (``[{name, arguments}]``) in this family's format."""
        import json as _json
        spec = TOOL_FORMATS[self.tool_format]
        key = spec["arguments_key"]
        objs = [{"name": c["name"], key: c.get("arguments", c.get("parameters", {}))} for c in calls]
        if spec["extract"] == "name_then_json":
            return "\n".join(f"{o['name']}\n{_json.dumps(o[key], ensure_ascii=False)}" for o in objs)
        if spec["joined"]:
            return self.function_fmt.format(content=_json.dumps(objs, ensure_ascii=False))
        sep = "; " if spec["extract"] == "json" else "\n"
        return sep.join(self.function_fmt.format(content=_json.dumps(o, ensure_ascii=False)) for o in objs)

    def normalise(self, messages: Sequence[dict], system: str = "", tools: str = ""):
        """Tool turns become ordinary ones: a ``function`` turn is an assistant turn wrapped in ``function_fmt``, an
        ``observation`` a user turn wrapped in ``observation_fmt``; a tool list is appended to the system prompt."""
        out = []
        for m in messages:
            if m["role"] == "function":
                content = m["content"]
                try:                                   # a JSON list of calls: one block per call
                    import json as _json
                    calls = _json.loads(content)
                    calls = calls if isinstance(calls, list) else [calls]
                    if all(isinstance(c_, dict) and "name" in c_ for c_ in calls):
                        content = self._render_calls(calls)
                    else:
                        content = "\n".join(self.function_fmt.format(content=_json.dumps(c_, ensure_ascii=False))
                                            for c_ in calls)
                    out.append({"role": "assistant", "content": content})
                    continue
                except (ValueError, TypeError):
                    pass
                out.append({"role": "assistant", "content": self.function_fmt.format(content=content)})
            elif m["role"] == "observation":
                out.append({"role": "user", "content": self.observation_fmt.format(content=m["content"])})
            else:
                out.append(m)
        if tools:
            system = (system or self.default_system) + self.tools_fmt.format(content=tools if isinstance(tools, str)
                                                                             else __import__("json").dumps(tools))
        return out, system

    def extract_tool_calls(self, text: str):
        """``(remaining text, [{"name": ..., "arguments": {...}}, ...])``: the function calls an answer makes, in this
        family's format; anything that does not parse stays text."""
        import json as _json
        import re
        spec = TOOL_FORMATS[self.tool_format]

        def as_call(obj):
            if isinstance(obj, dict) and "name" in obj:
                return {"name": obj["name"], "arguments": obj.get("arguments", obj.get("parameters", {}))}
            return None

        kind = spec["extract"]
        if kind == "json":                                  # the whole answer: one JSON object, or several after ";"
            try:
                objs = [_json.loads(text)]
            except ValueError:
                try:
                    objs = [_json.loads(part) for part in text.split("; ")]
                except ValueError:
                    return text, []
            calls = [as_call(o) for o in objs]
            return ("", calls) if calls and all(calls) else (text, [])
        if kind == "prefixed_list":
            marker = self.function_fmt.partition("{content}")[0].strip()
            at = text.find(marker)
            if at < 0:
                return text, []
            try:
                objs = _json.loads(text[at + len(marker):].strip())
            except ValueError:
                return text, []
            calls = [as_call(o) for o in (objs if isinstance(objs, list) else [objs])]
            return (text[:at].strip(), calls) if calls and all(calls) else (text, [])
        if kind == "name_then_json":                        # a function name on one line, its arguments on the next
            m = re.fullmatch(r"\s*([\w.\-]+)\n(\{.*\})\s*", text, flags=re.S)
            if not m:
                return text, []
            try:
                return "", [{"name": m.group(1), "arguments": _json.loads(m.group(2))}]
            except ValueError:
                return text, []
        head, _, tail = self.function_fmt.partition("{content}")
        head, tail = head.strip(), tail.strip()
        if not head or not tail:
            return text, []
        calls, rest, pos = [], [], 0
        for m in re.finditer(re.escape(head) + r"\s*(.*?)\s*" + re.escape(tail), text, flags=re.S):
            try:
                call = as_call(_json.loads(m.group(1)))
            except ValueError:
                continue
            if call is None:
                continue
            calls.append(call)
            rest.append(text[pos:m.start()])
            pos = m.end()
        rest.append(text[pos:])
        return "".join(rest).strip() if calls else text, calls

    def encode_multiturn(self, tokenizer, messages: Sequence[dict], system: str = "") -> List[Tuple[List[int], List[int]]]:
        """Returns ``[(prompt_ids, response_ids), ...]`` per user/assistant exchange."""
        pairs = []
        prefix = ""
        if any(m["role"] in ("function", "observation") for m in messages):
            messages, system = self.normalise(messages, system)
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
                       assistant_fmt="{content}<|eot_id|>", add_bos=True, efficient_eos=False, tool_format="llama3"),
    "mistral": Template("mistral", system_fmt="{content}\n\n", user_fmt="[INST] {content}[/INST]",
                        assistant_fmt=" {content}", add_bos=True, tool_format="mistral"),
    "ministral": Template("ministral", system_fmt="[SYSTEM_PROMPT]{content}[/SYSTEM_PROMPT]",
                          user_fmt="[INST]{content}[/INST]", assistant_fmt="{content}", add_bos=True,
                          tool_format="mistral"),
    "qwen3_nothink": Template("qwen3_nothink", system_fmt="<|im_start|>system\n{content}<|im_end|>\n",
                              user_fmt="<|im_start|>user\n{content}<|im_end|>\n<|im_start|>assistant\n<think>\n\n</think>\n\n",
                              assistant_fmt="{content}<|im_end|>\n", efficient_eos=False),
    "llama2": Template("llama2", system_fmt="<<SYS>>\n{content}\n<</SYS>>\n\n", user_fmt="[INST] {content} [/INST]",
                       assistant_fmt=" {content} ", add_bos=True),
    "llama4": Template("llama4", system_fmt="<|header_start|>system<|header_end|>\n\n{content}<|eot|>",
                       user_fmt="<|header_start|>user<|header_end|>\n\n{content}<|eot|>"
                                "<|header_start|>assistant<|header_end|>\n\n",
                       assistant_fmt="{content}<|eot|>", add_bos=True, efficient_eos=False),
    "gemma": Template("gemma", system_fmt="{content}\n\n",
                      user_fmt="<start_of_turn>user\n{content}<end_of_turn>\n<start_of_turn>model\n",
                      assistant_fmt="{content}<end_of_turn>\n", add_bos=True, efficient_eos=False),
    "phi": Template("phi", system_fmt="<|system|>\n{content}<|end|>\n", user_fmt="<|user|>\n{content}<|end|>\n<|assistant|>\n",
                    assistant_fmt="{content}<|end|>\n", efficient_eos=False),
    "phi4": Template("phi4", system_fmt="<|im_start|>system<|im_sep|>{content}<|im_end|>",
                     user_fmt="<|im_start|>user<|im_sep|>{content}<|im_end|><|im_start|>assistant<|im_sep|>",
                     assistant_fmt="{content}<|im_end|>", efficient_eos=False),
    "deepseek": Template("deepseek", system_fmt="{content}\n\n", user_fmt="User: {content}\n\nAssistant:",
                         assistant_fmt=" {content}", add_bos=True),
    "deepseek3": Template("deepseek3", system_fmt="{content}", user_fmt="<\uff5cUser\uff5c>{content}<\uff5cAssistant\uff5c>",
                          assistant_fmt="{content}", add_bos=True),
    "glm4": Template("glm4", system_fmt="<|system|>\n{content}", user_fmt="<|user|>\n{content}<|assistant|>\n",
                     assistant_fmt="{content}", default_system="", efficient_eos=True),
    "yi": Template("yi", system_fmt="<|im_start|>system\n{content}<|im_end|>\n",
                   user_fmt="<|im_start|>user\n{content}<|im_end|>\n<|im_start|>assistant\n",
                   assistant_fmt="{content}<|im_end|>\n", efficient_eos=False),
    "zephyr": Template("zephyr", system_fmt="<|system|>\n{content}</s>\n", user_fmt="<|user|>\n{content}</s>\n<|assistant|>\n",
                       assistant_fmt="{content}</s>\n", default_system="You are a friendly chatbot.", efficient_eos=False),
    "vicuna": Template("vicuna", system_fmt="{content} ", user_fmt="USER: {content} ASSISTANT:", assistant_fmt="{content}",
                       default_system="A chat between a curious user and an artificial intelligence assistant. "
                                      "The assistant gives helpful, detailed, and polite answers to the user's questions."),
    "alpaca": Template("alpaca", system_fmt="{content}\n\n", user_fmt="### Instruction:\n{content}\n\n### Response:\n",
                       assistant_fmt="{content}\n\n",
                       default_system="Below is an instruction that describes a task. "
                                      "Write a response that appropriately completes the request."),
    "openchat": Template("openchat", system_fmt="{content}", user_fmt="GPT4 Correct User: {content}<|end_of_turn|>"
                                                                      "GPT4 Correct Assistant:",
                         assistant_fmt="{content}<|end_of_turn|>", add_bos=True, efficient_eos=False),
    "falcon": Template("falcon", system_fmt="{content}\n", user_fmt="User: {content}\nFalcon:", assistant_fmt="{content}\n"),
    "granite3": Template("granite3", system_fmt="<|start_of_role|>system<|end_of_role|>{content}<|end_of_text|>\n",
                         user_fmt="<|start_of_role|>user<|end_of_role|>{content}<|end_of_text|>\n"
                                  "<|start_of_role|>assistant<|end_of_role|>",
                         assistant_fmt="{content}<|end_of_text|>\n", efficient_eos=False),
}


from .template_zoo import register_all as _register_zoo  # noqa: E402

_register_zoo(TEMPLATES, Template)


def register_template(template: Template) -> None:
    """Adds a user-defined template (the name must be new)."""
    if template.name in TEMPLATES:
        raise ValueError(f"template '{template.name}' already exists")
    TEMPLATES[template.name] = template


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
