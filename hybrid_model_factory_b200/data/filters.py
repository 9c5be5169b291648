"""Quality filters applied to aligned records before tokenisation (reference: ``data/filter.py``).

Each filter maps a text to ``True`` (keep) / ``False`` (drop); ``apply_filters`` runs a list of them over the
response text of every record and reports how many each one removed.
"""
from __future__ import annotations

from collections import Counter
from typing import Callable, Iterable, List, Sequence, Tuple


def ngram_repetition_ratio(text: str, n: int = 4) -> float:
    """Fraction of word n-grams that are repeats of an earlier n-gram."""
    words = text.split()
    if len(words) < n + 1:
        return 0.0
    grams = [tuple(words[i:i + n]) for i in range(len(words) - n + 1)]
    counts = Counter(grams)
    return sum(c - 1 for c in counts.values()) / len(grams)


def max_ngram_count(text: str, n: int = 8) -> int:
    words = text.split()
    if len(words) < n:
        return 0
    return max(Counter(tuple(words[i:i + n]) for i in range(len(words) - n + 1)).values())


def char_repetition_run(text: str) -> int:
    best = run = 1 if text else 0
    for a, b in zip(text, text[1:]):
        run = run + 1 if a == b else 1
        best = max(best, run)
    return best


def make_filters(max_repetition_ratio: float = 0.3, max_same_ngram: int = 8, max_char_run: int = 64,
                 min_chars: int = 1, max_chars: int = 0) -> List[Tuple[str, Callable[[str], bool]]]:
    fs = [("ngram_repetition", lambda t: ngram_repetition_ratio(t) <= max_repetition_ratio),
          ("repeated_ngram", lambda t: max_ngram_count(t) <= max_same_ngram),
          ("char_run", lambda t: char_repetition_run(t) <= max_char_run),
          ("too_short", lambda t: len(t) >= min_chars)]
    if max_chars:
        fs.append(("too_long", lambda t: len(t) <= max_chars))
    return fs


def record_text(rec: dict) -> str:
    if "text" in rec:
        return rec["text"]
    msgs = rec.get("messages") or []
    return "\n".join(m.get("content", "") for m in msgs if m.get("role") == "assistant") or rec.get("response", "")


def apply_filters(records: Iterable[dict], filters: Sequence[Tuple[str, Callable[[str], bool]]] = None):
    filters = make_filters() if filters is None else filters
    kept, dropped = [], Counter()
    for rec in records:
        text = record_text(rec)
        for name, f in filters:
            if not f(text):
                dropped[name] += 1
                break
        else:
            kept.append(rec)
    return kept, dict(dropped)
