"""Batch generation over a dataset with text-similarity metrics (the ``do_predict`` / ``predict_with_generate`` path of
the reference's SFT workflow, ``train/sft/workflow.py`` and ``train/sft/metric.py``).

Prompts come from the ``unsupervised`` processor (conversation up to the last user turn, reference answer as label), run
through the serving engine (continuous batching, paged cache, CUDA-graph decode on the GPU) and are written to
``generated_predictions.jsonl`` (``prompt`` / ``predict`` / ``label``).  Metrics: exact match, ROUGE-1 / ROUGE-2 /
ROUGE-L F-scores and BLEU-4 with add-one smoothing over whitespace tokens (characters for text without spaces, e.g.
Chinese), averaged over the samples and written to ``predict_results.json``.
"""
from __future__ import annotations

import json
import math
import os
from collections import Counter
from typing import Dict, List, Optional, Sequence


def _tokens(text: str) -> List[str]:
    text = text.strip()
    return text.split() if (" " in text or not text) else list(text)


def _ngrams(toks: Sequence[str], n: int) -> Counter:
    return Counter(tuple(toks[i:i + n]) for i in range(len(toks) - n + 1))


def _f1(overlap: int, n_pred: int, n_ref: int) -> float:
    if overlap == 0 or n_pred == 0 or n_ref == 0:
        return 0.0
    p, r = overlap / n_pred, overlap / n_ref
    return 2 * p * r / (p + r)


def rouge_n(pred: Sequence[str], ref: Sequence[str], n: int) -> float:
    a, b = _ngrams(pred, n), _ngrams(ref, n)
    return _f1(sum((a & b).values()), sum(a.values()), sum(b.values()))


def rouge_l(pred: Sequence[str], ref: Sequence[str]) -> float:
    """F-score of the longest common subsequence."""
    if not pred or not ref:
        return 0.0
    prev = [0] * (len(ref) + 1)
    for x in pred:
        cur = [0]
        for j, y in enumerate(ref, 1):
            cur.append(prev[j - 1] + 1 if x == y else max(prev[j], cur[j - 1]))
        prev = cur
    return _f1(prev[-1], len(pred), len(ref))


def bleu4(pred: Sequence[str], ref: Sequence[str]) -> float:
    """Sentence BLEU with uniform 1..4-gram weights, add-one smoothing above unigrams and the brevity penalty."""
    if not pred or not ref:
        return 0.0
    logs = 0.0
    for n in range(1, 5):
        a, b = _ngrams(pred, n), _ngrams(ref, n)
        match, total = sum((a & b).values()), sum(a.values())
        if n == 1:
            if match == 0:
                return 0.0
            prec = match / total
        else:
            prec = (match + 1) / (total + 1)
        logs += 0.25 * math.log(prec)
    bp = 1.0 if len(pred) > len(ref) else math.exp(1 - len(ref) / len(pred))
    return bp * math.exp(logs)


def text_metrics(preds: Sequence[str], labels: Sequence[str]) -> Dict[str, float]:
    keys = ("exact_match", "rouge-1", "rouge-2", "rouge-l", "bleu-4")
    acc = {k: 0.0 for k in keys}
    for p, l in zip(preds, labels):
        pt, lt = _tokens(p), _tokens(l)
        acc["exact_match"] += float(p.strip() == l.strip())
        acc["rouge-1"] += rouge_n(pt, lt, 1)
        acc["rouge-2"] += rouge_n(pt, lt, 2)
        acc["rouge-l"] += rouge_l(pt, lt)
        acc["bleu-4"] += bleu4(pt, lt)
    n = max(len(preds), 1)
    return {f"predict_{k}": round(100.0 * v / n, 4) for k, v in acc.items()}


END_MARKERS = ("<|im_end|>", "<|eot_id|>", "<|eot|>", "</s>", "<|end|>", "<end_of_turn>", "<|end_of_text|>",
               "<|end_of_turn|>")


def _clean(text: str) -> str:
    """Cuts a decoded answer at the first end-of-turn marker of the chat template."""
    cut = min((text.find(m) for m in END_MARKERS if m in text), default=-1)
    return (text if cut < 0 else text[:cut]).strip()


def run_predict(model, tokenizer, rows: Sequence[dict], output_dir: Optional[str] = None, max_new_tokens: int = 128,
                temperature: float = 0.0, top_k: int = 0, max_num_seqs: int = 16, max_model_len: int = 8192) -> Dict[str, float]:
    """``rows``: output of ``data.loader.process_unsupervised`` (``input_ids`` = prompt, ``labels`` = reference answer)."""
    from ..serving.engine import SamplingParams, ServingEngine
    engine = ServingEngine(model, max_num_seqs=max_num_seqs, max_model_len=max_model_len,
                           max_num_batched_tokens=max(2048, min(max_model_len, 16384)))
    params = SamplingParams(max_new_tokens=max_new_tokens, temperature=temperature, top_k=top_k,
                            eos_token_id=getattr(tokenizer, "eos_token_id", None), ignore_eos=False)
    outs = engine.generate([list(r["input_ids"]) for r in rows], params)
    eos = getattr(tokenizer, "eos_token_id", None)
    strip = lambda ids: [t for t in ids if t != eos and t >= 0]  # noqa: E731
    preds = [_clean(tokenizer.decode(strip(o))) for o in outs]
    labels = [_clean(tokenizer.decode(strip(r["labels"]))) for r in rows]
    prompts = [tokenizer.decode(strip(r["input_ids"])) for r in rows]
    metrics = text_metrics(preds, labels)
    if output_dir:
        os.makedirs(output_dir, exist_ok=True)
        with open(os.path.join(output_dir, "generated_predictions.jsonl"), "w", encoding="utf-8") as f:
            for pr, p, l in zip(prompts, preds, labels):
                f.write(json.dumps({"prompt": pr, "predict": p, "label": l}, ensure_ascii=False) + "\n")
        with open(os.path.join(output_dir, "predict_results.json"), "w", encoding="utf-8") as f:
            json.dump(metrics, f, indent=2)
    return metrics
