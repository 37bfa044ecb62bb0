"""Word error rate of decoded hypotheses against reference transcripts.

Reference: axlearn/audio/evaler_asr.py (``compute_word_errors`` :24, ``WordErrorRateMetricCalculator``
:84-243).  Every batch is decoded with a model method (beam search by default), the best hypothesis
and the labels are detokenised with the vocabulary, and substitutions / deletions / insertions are
counted by word-level edit distance; the summaries are sums over the evaluation set, so the rate
is exact whatever the batching.
"""

from __future__ import annotations

from typing import Any, Optional, Sequence

import torch

from axlearn_b200.common import prng
from axlearn_b200.common.config import REQUIRED, InstantiableConfig, Required, config_class, maybe_instantiate
from axlearn_b200.common.evaler import BaseMetricCalculator
from axlearn_b200.common.metrics import WeightedSummary


def word_errors(hypothesis: Sequence[str], reference: Sequence[str]) -> dict:
    """Minimum-edit alignment counts: ``substitutions``, ``deletions``, ``insertions``."""
    h, r = list(hypothesis), list(reference)
    # cost[i][j] = (edits, subs, dels, ins) turning r[:i] into h[:j].
    prev = [(j, 0, 0, j) for j in range(len(h) + 1)]
    for i in range(1, len(r) + 1):
        cur = [(i, 0, i, 0)]
        for j in range(1, len(h) + 1):
            if r[i - 1] == h[j - 1]:
                best = prev[j - 1]
            else:
                e, s, d, n = prev[j - 1]
                best = (e + 1, s + 1, d, n)
            e, s, d, n = prev[j]
            if e + 1 < best[0]:
                best = (e + 1, s, d + 1, n)
            e, s, d, n = cur[j - 1]
            if e + 1 < best[0]:
                best = (e + 1, s, d, n + 1)
            cur.append(best)
        prev = cur
    _, s, d, n = prev[-1]
    return dict(substitutions=s, deletions=d, insertions=n)


def compute_word_errors(hypotheses: Sequence[str], references: Sequence[str]) -> dict:
    """Totals over pairs of sentences; examples with an empty reference are skipped."""
    out = dict(num_words=0, substitutions=0, deletions=0, insertions=0, num_examples=0)
    for hyp, ref in zip(hypotheses, references):
        words = ref.split()
        if not words:
            continue
        e = word_errors(hyp.split(), words)
        out["num_words"] += len(words)
        out["num_examples"] += 1
        for k in ("substitutions", "deletions", "insertions"):
            out[k] += e[k]
    return out


class WordErrorRateMetricCalculator(BaseMetricCalculator):
    @config_class
    class Config(BaseMetricCalculator.Config):
        vocab: Required[Any] = REQUIRED                 # config or object with decode(ids) -> str
        model_method: str = "beam_search_decode"
        model_method_kwargs: dict = {}

    def __init__(self, cfg, *, parent=None, **kwargs):
        super().__init__(cfg, parent=parent, **kwargs)
        self._vocab = maybe_instantiate(cfg.vocab) if isinstance(cfg.vocab, InstantiableConfig) else cfg.vocab

    def init_state(self, *, prng_key, model_params):
        return {"prng_key": prng_key}

    def _texts(self, ids: torch.Tensor, paddings: Optional[torch.Tensor]) -> list[str]:
        out = []
        for i in range(ids.shape[0]):
            row = ids[i]
            keep = ~paddings[i].bool() if paddings is not None else (row >= 0)
            out.append(self._vocab.decode([int(t) for t in row[keep].tolist()]))
        return out

    def forward(self, input_batch, *, model_params, state):
        cfg = self._config
        key, next_key = prng.split(state["prng_key"], 2)
        outputs, _ = self._call_model(method=cfg.model_method, prng_key=key, model_params=model_params,
                                      input_batch=input_batch, **cfg.model_method_kwargs)
        if isinstance(outputs, list):       # per-utterance lists of (tokens, score), best first
            hyps = [self._vocab.decode(list(beams[0][0] if beams and isinstance(beams[0], tuple) else beams))
                    for beams in outputs]
        else:
            hyps = self._texts(outputs.sequences[:, 0], outputs.paddings[:, 0])
        labels = input_batch["target_labels"]
        eos = getattr(self._vocab, "eos_id", None)
        label_pad = (labels < 0) | (labels >= getattr(self._vocab, "vocab_size", 1 << 30))
        if eos is not None:
            label_pad = label_pad | (labels == eos)
        errors = compute_word_errors(hyps, self._texts(labels, label_pad))
        return {"state": {"prng_key": next_key}, "output": errors}

    def get_summaries(self, *, model_params, state, all_forward_outputs):
        total = {k: sum(o[k] for o in all_forward_outputs) for k in
                 ("num_words", "substitutions", "deletions", "insertions", "num_examples")}
        words = max(1, total["num_words"])
        t = lambda v: torch.tensor(float(v))
        return {
            "word_errors/wer": WeightedSummary(
                t((total["substitutions"] + total["deletions"] + total["insertions"]) / words), words),
            "word_errors/substitutions": WeightedSummary(t(total["substitutions"] / words), words),
            "word_errors/deletions": WeightedSummary(t(total["deletions"] / words), words),
            "word_errors/insertions": WeightedSummary(t(total["insertions"] / words), words),
            "word_errors/num_examples": WeightedSummary(t(total["num_examples"]), 1),
        }
