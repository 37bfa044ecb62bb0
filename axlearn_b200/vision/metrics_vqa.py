"""Visual question answering accuracy with the standard answer normalisation.

Counterpart of axlearn/vision/metrics_vqa.py: an answer scores ``min(1, matching human answers / 3)``,
averaged over the ten leave-one-out subsets of the human answers; before matching, answers are
lower-cased, punctuation is stripped, number words become digits, articles are dropped and
contractions are restored.
"""

from __future__ import annotations

import re
from typing import Sequence

_NUMBERS = {"none": "0", "zero": "0", "one": "1", "two": "2", "three": "3", "four": "4", "five": "5", "six": "6",
            "seven": "7", "eight": "8", "nine": "9", "ten": "10"}
_ARTICLES = {"a", "an", "the"}
_CONTRACTIONS = {"dont": "don't", "doesnt": "doesn't", "isnt": "isn't", "arent": "aren't", "cant": "can't",
                 "couldnt": "couldn't", "didnt": "didn't", "hasnt": "hasn't", "havent": "haven't", "im": "i'm",
                 "ive": "i've", "wasnt": "wasn't", "werent": "weren't", "wont": "won't", "wouldnt": "wouldn't",
                 "shouldnt": "shouldn't", "thats": "that's", "theres": "there's", "whats": "what's", "youre": "you're"}
_PUNCT = re.compile(r"[;/\[\]\"{}()=+\\_\-><@`,?!*#%^&$~|:]")
_PERIOD = re.compile(r"(?!<=\d)(\.)(?!\d)")
_COMMA_IN_NUMBER = re.compile(r"(\d)(,)(\d)")


def normalize_answer(answer: str) -> str:
    a = answer.lower().replace("\n", " ").replace("\t", " ").strip()
    a = _COMMA_IN_NUMBER.sub(r"\1\3", a)
    a = _PUNCT.sub(" ", a)
    a = _PERIOD.sub("", a)
    words = []
    for w in a.split():
        w = _NUMBERS.get(w, w)
        if w in _ARTICLES:
            continue
        words.append(_CONTRACTIONS.get(w, w))
    return " ".join(words)


def vqa_accuracy(prediction: str, human_answers: Sequence[str]) -> float:
    """Mean over leave-one-out subsets of ``min(1, matches / 3)``."""
    pred = normalize_answer(prediction)
    answers = [normalize_answer(a) for a in human_answers]
    if not answers:
        return 0.0
    if len(answers) == 1:
        return float(pred == answers[0])
    scores = []
    for i in range(len(answers)):
        others = answers[:i] + answers[i + 1:]
        scores.append(min(1.0, sum(a == pred for a in others) / 3.0))
    return sum(scores) / len(scores)


def vqa_accuracy_batch(predictions: Sequence[str], answers: Sequence[Sequence[str]]) -> dict:
    scores = [vqa_accuracy(p, a) for p, a in zip(predictions, answers)]
    return {"vqa_accuracy": sum(scores) / max(1, len(scores)), "num_examples": len(scores)}
