"""``hmf eval``: multiple-choice benchmark evaluation (MMLU / C-Eval / CMMLU style) of a hybrid checkpoint.

Task layout under ``task_dir/<task>/``: ``mapping.json`` (``{subject: {"name": ..., "category": ...}}``) and, per
subject, ``<subject>.json`` with the splits ``{"train": [...], "validation": [...], "test": [...]}``; every example is
``{"question": str, "A": str, "B": str, "C": str, "D": str, "answer": "A".."D"}``.  ``task`` is ``<task>_<split>``
(``mmlu_test``).  For every test question the prompt is the subject header, ``n_shot`` solved exemplars from the
``train`` split and the question; the prediction is the choice letter with the largest logit at the last prompt
position.  Results: accuracy per category, per subject and on average, written to ``save_dir/results.json`` and
``results.log``.  Sequences are evaluated one by one or in right-padded batches; since the recurrent layers cannot skip
padding, a batch groups prompts of equal length only.

Reference: ``eval/evaluator.py:60-160`` and ``eval/template.py`` (few-shot formats for ``en`` / ``zh``).
"""
from __future__ import annotations

import json
import os
import random
from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence

import torch

CHOICES = ["A", "B", "C", "D"]


@dataclass
class EvaluationArguments:
    task: str = "mmlu_test"
    task_dir: str = "evaluation"
    batch_size: int = 4
    seed: int = 42
    lang: str = "en"
    n_shot: int = 5
    save_dir: Optional[str] = None


@dataclass
class EvalTemplate:
    system: str
    choice: str
    answer: str

    def _example(self, ex: dict) -> str:
        return ex["question"] + "".join(self.choice.format(choice=c, content=ex[c]) for c in CHOICES if c in ex) + self.answer

    def format_example(self, target: dict, support: Sequence[dict], subject_name: str) -> List[Dict[str, str]]:
        """Chat messages: the exemplars as solved user / assistant turns, then the target question."""
        messages = []
        for ex in support:
            messages += [{"role": "user", "content": self._example(ex)}, {"role": "assistant", "content": ex["answer"]}]
        messages += [{"role": "user", "content": self._example(target)}, {"role": "assistant", "content": target["answer"]}]
        messages[0]["content"] = self.system.format(subject=subject_name) + messages[0]["content"]
        return messages


EVAL_TEMPLATES = {
    "en": EvalTemplate(system="The following are multiple choice questions (with answers) about {subject}.\n\n",
                       choice="\n{choice}. {content}", answer="\nAnswer:"),
    "zh": EvalTemplate(system="以下是中国关于{subject}考试的单项选择题，请选出其中的正确答案。\n\n",
                       choice="\n{choice}. {content}", answer="\n答案："),
}


class Evaluator:
    def __init__(self, model, tokenizer, template, args: EvaluationArguments):
        self.model, self.tok, self.tpl, self.args = model.eval(), tokenizer, template, args
        self.device = next(model.parameters()).device
        self.eval_template = EVAL_TEMPLATES[args.lang]
        # the last token of " A" style encodings is the letter itself for byte-level and BPE vocabularies alike
        self.choice_ids = [tokenizer.encode(c, add_special_tokens=False)[-1] for c in CHOICES]

    def encode_prompt(self, messages: List[Dict[str, str]]) -> List[int]:
        pairs = self.tpl.encode_multiturn(self.tok, messages)
        ids: List[int] = []
        for i, (p, r) in enumerate(pairs):
            ids += p + (r if i < len(pairs) - 1 else [])
        return ids

    @torch.no_grad()
    def predict(self, prompts: List[List[int]]) -> List[str]:
        """Choice letters for a list of prompts (grouped into batches of equal length)."""
        order = sorted(range(len(prompts)), key=lambda i: len(prompts[i]))
        out: Dict[int, str] = {}
        i = 0
        while i < len(order):
            j = i
            while j < len(order) and j - i < self.args.batch_size and len(prompts[order[j]]) == len(prompts[order[i]]):
                j += 1
            ids = torch.tensor([prompts[k] for k in order[i:j]], dtype=torch.long, device=self.device)
            logits = self.model(ids, logits_to_keep=1).logits[:, -1].float()
            best = logits[:, self.choice_ids].argmax(-1).tolist()
            for k, b in zip(order[i:j], best):
                out[k] = CHOICES[b]
            i = j
        return [out[i] for i in range(len(prompts))]

    def evaluate(self) -> Dict[str, float]:
        a = self.args
        task, split = a.task.rsplit("_", 1)
        root = os.path.join(a.task_dir, task)
        with open(os.path.join(root, "mapping.json"), encoding="utf-8") as f:
            mapping: Dict[str, Dict[str, str]] = json.load(f)
        rng = random.Random(a.seed)
        per_subject: Dict[str, List[bool]] = {}
        outputs: Dict[str, Dict[str, str]] = {}
        for subject, info in mapping.items():
            with open(os.path.join(root, f"{subject}.json"), encoding="utf-8") as f:
                data = json.load(f)
            train = list(data.get("train", []))
            prompts, labels = [], []
            for ex in data[split]:
                support = rng.sample(train, min(a.n_shot, len(train)))
                msgs = self.eval_template.format_example(ex, support, info["name"])
                prompts.append(self.encode_prompt(msgs))
                labels.append(ex["answer"])
            preds = self.predict(prompts)
            per_subject[subject] = [p == l for p, l in zip(preds, labels)]
            outputs[subject] = {str(i): p for i, p in enumerate(preds)}
        results: Dict[str, float] = {}
        cats: Dict[str, List[bool]] = {}
        for subject, ok in per_subject.items():
            results[f"subject/{subject}"] = 100.0 * sum(ok) / max(len(ok), 1)
            cats.setdefault(mapping[subject].get("category", "Other"), []).extend(ok)
            cats.setdefault("Average", []).extend(ok)
        for cat, ok in cats.items():
            results[cat] = 100.0 * sum(ok) / max(len(ok), 1)
        if a.save_dir:
            os.makedirs(a.save_dir, exist_ok=True)
            with open(os.path.join(a.save_dir, "results.json"), "w", encoding="utf-8") as f:
                json.dump(outputs, f, indent=2)
            with open(os.path.join(a.save_dir, "results.log"), "w", encoding="utf-8") as f:
                f.write("\n".join(f"{k:>40}: {v:.2f}" for k, v in results.items() if not k.startswith("subject/")))
        return results


def main(argv=None) -> int:
    import argparse
    from ..data.formats import get_template, load_tokenizer
    from ..utils import checkpoint_io
    ap = argparse.ArgumentParser(prog="hmf eval")
    ap.add_argument("model")
    ap.add_argument("--task", default="mmlu_test")
    ap.add_argument("--task-dir", default="evaluation")
    ap.add_argument("--template", default=None)
    ap.add_argument("--lang", default="en", choices=sorted(EVAL_TEMPLATES))
    ap.add_argument("--n-shot", type=int, default=5)
    ap.add_argument("--batch-size", type=int, default=4)
    ap.add_argument("--seed", type=int, default=42)
    ap.add_argument("--save-dir", default=None)
    ap.add_argument("--config", default=None, help="YAML file whose keys (task, task_dir, n_shot, ...) replace the defaults")
    pre, _ = ap.parse_known_args(argv)
    if pre.config:
        import yaml
        with open(pre.config) as f:
            given = yaml.safe_load(f) or {}
        known = {act.dest for act in ap._actions}
        bad = sorted(k for k in given if k not in known)
        if bad:
            raise ValueError(f"{pre.config}: unknown keys {bad}")
        ap.set_defaults(**given)
    a = ap.parse_args(argv)
    device = torch.device("cuda", 0) if torch.cuda.is_available() else torch.device("cpu")
    model = checkpoint_io.from_pretrained(a.model, device=device, init="meta")
    ev = Evaluator(model, load_tokenizer(a.model), get_template(a.template),
                   EvaluationArguments(a.task, a.task_dir, a.batch_size, a.seed, a.lang, a.n_shot, a.save_dir))
    res = ev.evaluate()
    print("\n".join(f"{k:>40}: {v:.2f}" for k, v in res.items() if not k.startswith("subject/")))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
