"""LongBench (English) task metrics, dependency-free: token F1 for QA, ROUGE-L F for summarisation, class
match for TREC, paragraph-number match for retrieval / counting, edit similarity for code completion.
Same task -> metric table and aggregation as LongBench's eval (reference scripts/longbench_metrics.py:112-145);
ROUGE-L and the code similarity are computed here instead of through the rouge / fuzzywuzzy packages."""
from __future__ import annotations

import difflib
import re
import string
from collections import Counter


def normalize_answer(s: str) -> str:
    s = s.lower()
    s = "".join(ch for ch in s if ch not in set(string.punctuation))
    s = re.sub(r"\b(a|an|the)\b", " ", s)
    return " ".join(s.split())


def _f1(pred_tokens: list[str], ref_tokens: list[str]) -> float:
    common = Counter(pred_tokens) & Counter(ref_tokens)
    same = sum(common.values())
    if same == 0:
        return 0.0
    p, r = same / len(pred_tokens), same / len(ref_tokens)
    return 2 * p * r / (p + r)


def qa_f1_score(prediction: str, ground_truth: str, **_) -> float:
    return _f1(normalize_answer(prediction).split(), normalize_answer(ground_truth).split())


def _lcs(a: list[str], b: list[str]) -> int:
    prev = [0] * (len(b) + 1)
    for x in a:
        cur = [0]
        for j, y in enumerate(b, 1):
            cur.append(prev[j - 1] + 1 if x == y else max(prev[j], cur[j - 1]))
        prev = cur
    return prev[-1]


def rouge_score(prediction: str, ground_truth: str, **_) -> float:
    """ROUGE-L F-measure over whitespace tokens."""
    p, r = prediction.split(), ground_truth.split()
    if not p or not r:
        return 0.0
    lcs = _lcs(p, r)
    if lcs == 0:
        return 0.0
    prec, rec = lcs / len(p), lcs / len(r)
    return 2 * prec * rec / (prec + rec)


def classification_score(prediction: str, ground_truth: str, all_classes=None, **_) -> float:
    matches = [c for c in (all_classes or []) if c in prediction]
    matches = [m for m in matches if not (m in ground_truth and m != ground_truth)]
    return 1.0 / len(matches) if ground_truth in matches else 0.0


def retrieval_score(prediction: str, ground_truth: str, **_) -> float:
    m = re.findall(r"Paragraph (\d+)", ground_truth)
    if not m:
        return 0.0
    numbers = re.findall(r"\d+", prediction)
    return sum(1 for n in numbers if n == m[0]) / len(numbers) if numbers else 0.0


def count_score(prediction: str, ground_truth: str, **_) -> float:
    numbers = re.findall(r"\d+", prediction)
    return sum(1 for n in numbers if n == str(ground_truth)) / len(numbers) if numbers else 0.0


def code_sim_score(prediction: str, ground_truth: str, **_) -> float:
    first = ""
    for line in prediction.lstrip("\n").split("\n"):
        if "`" not in line and "#" not in line and "//" not in line:
            first = line
            break
    return difflib.SequenceMatcher(None, first, ground_truth).ratio()


DATASET2METRIC = {
    "narrativeqa": qa_f1_score, "qasper": qa_f1_score, "multifieldqa_en": qa_f1_score, "hotpotqa": qa_f1_score,
    "2wikimqa": qa_f1_score, "musique": qa_f1_score, "gov_report": rouge_score, "qmsum": rouge_score,
    "multi_news": rouge_score, "trec": classification_score, "triviaqa": qa_f1_score, "samsum": rouge_score,
    "passage_retrieval_en": retrieval_score, "passage_count": count_score, "lcc": code_sim_score,
    "repobench-p": code_sim_score,
}
# few-shot tasks whose generations are cut at the first newline before scoring
FIRST_LINE_ONLY = {"trec", "triviaqa", "samsum"}


def scorer(dataset: str, predictions: list[str], answers: list[list[str]], all_classes) -> float:
    metric = DATASET2METRIC[dataset]
    total = 0.0
    for pred, refs in zip(predictions, answers):
        if dataset in FIRST_LINE_ONLY:
            pred = pred.lstrip("\n").split("\n")[0]
        total += max((metric(pred, r, all_classes=all_classes) for r in refs), default=0.0)
    return round(100.0 * total / max(1, len(predictions)), 2)
