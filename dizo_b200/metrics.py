"""Evaluation metrics: accuracy (multi-gold aware), exact match and token-level F1 with the
SQuAD answer normalisation.  Same definitions as the reference (large_models/metrics.py:7-77)."""
from __future__ import annotations

import re
import string
from collections import Counter

import numpy as np

_ARTICLES = re.compile(r"\b(a|an|the)\b")
_PUNCT = set(string.punctuation)
_UNANSWERABLE = ("CANNOTANSWER", "no answer")


def normalize_answer(s: str) -> str:
    """Lower-case, drop punctuation and articles, collapse whitespace."""
    s = "".join(ch for ch in s.lower() if ch not in _PUNCT)
    return " ".join(_ARTICLES.sub(" ", s).split())


def _token_f1(pred: str, gold: str) -> float:
    p, g = normalize_answer(pred).split(), normalize_answer(gold).split()
    same = sum((Counter(p) & Counter(g)).values())
    if same == 0:
        return 0.0
    precision, recall = same / len(p), same / len(g)
    return 2 * precision * recall / (precision + recall)


def f1(pred: str, gold: list) -> float:
    """Best token F1 of ``pred`` against any gold answer (the non-differentiable SQuAD objective)."""
    if gold[0] in _UNANSWERABLE:
        return float(normalize_answer(gold[0]) == normalize_answer(pred))
    return max(_token_f1(pred, ans) for ans in gold)


def calculate_metric(predictions, metric_name: str) -> float:
    if metric_name == "accuracy":
        if isinstance(predictions[0].correct_candidate, list):
            return float(np.mean([p.predicted_candidate in p.correct_candidate for p in predictions]))
        return float(np.mean([p.correct_candidate == p.predicted_candidate for p in predictions]))
    if metric_name == "em":
        return float(np.mean([any(normalize_answer(a) == normalize_answer(p.predicted_candidate)
                                  for a in p.correct_candidate) for p in predictions]))
    if metric_name == "f1":
        return float(np.mean([f1(p.predicted_candidate, p.correct_candidate) for p in predictions]))
    raise ValueError(f"unknown metric {metric_name!r}")
