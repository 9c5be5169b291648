"""``Renderer``: unified chat samples -> token ids, labels and loss weights, through this package's chat templates
(``data/formats.py``).  Reference: ``v1/core/utils/rendering.py`` and ``v1/plugins/model_plugins/rendering.py``."""
from __future__ import annotations

from typing import Dict, List, Sequence

from ..data.formats import get_template

IGNORE_INDEX = -100


class Renderer:
    def __init__(self, tokenizer, template: str = "default", cutoff_len: int = 2048):
        self.tokenizer, self.cutoff_len = tokenizer, cutoff_len
        self.template = get_template(template)

    def render_messages(self, messages: Sequence[dict]) -> Dict[str, List[int]]:
        """Tokens of the whole conversation; labels only where the turn's ``loss_weight`` is positive."""
        system = next((m["content"] for m in messages if m["role"] == "system"), "")
        turns = [m for m in messages if m["role"] != "system"]
        plain = [{"role": m["role"], "content": m["content"]} for m in turns]
        if plain and plain[-1]["role"] != "assistant":
            plain.append({"role": "assistant", "content": ""})
            turns = turns + [{"role": "assistant", "content": "", "loss_weight": 0.0}]
        pairs = self.template.encode_multiturn(self.tokenizer, plain, system)
        ids: List[int] = []
        labels: List[int] = []
        answers = [m for m in turns if m["role"] == "assistant"]
        for (p, r), ans in zip(pairs, answers):
            ids += p + r
            labels += [IGNORE_INDEX] * len(p)
            labels += r if float(ans.get("loss_weight", 1.0)) > 0 else [IGNORE_INDEX] * len(r)
        ids, labels = ids[:self.cutoff_len], labels[:self.cutoff_len]
        return {"input_ids": ids, "labels": labels, "attention_mask": [1] * len(ids)}

    def process_samples(self, samples: Sequence[dict]) -> List[Dict[str, List[int]]]:
        out = []
        for s in samples:
            if "messages" in s:
                out.append(self.render_messages(s["messages"]))
            elif "chosen_messages" in s:
                c, r = self.render_messages(s["chosen_messages"]), self.render_messages(s["rejected_messages"])
                out.append({**{f"chosen_{k}": v for k, v in c.items()}, **{f"rejected_{k}": v for k, v in r.items()}})
            else:
                raise ValueError(f"sample of dataset {s.get('_dataset_name')} has no messages")
        return out
