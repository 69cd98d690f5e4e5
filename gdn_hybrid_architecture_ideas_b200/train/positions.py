"""Position masks drawn per (seed, step, row): uniform random subsets of a row's valid targets, and causal answer
spans.

Every mask is a pure function of (data seed, step, row) and the batch's own valid mask, drawn from counter-based
generators, so resume needs only the step and every process computes the same masks. The answer-span rule decides
position t from the RNG and the document structure at positions <= t only, so a scored position never learns where its
document ends: walk the row; a position may start a span once its document has `min_context` earlier positions; skip a
geometric number of eligible positions (mean `gap_mean`), open a span of a length from [span_min, span_max], cut it at
the document's end, continue after it; finally AND with the valid targets
(reference: ced/train/positions.py:109-353).
"""

from __future__ import annotations

import math
from dataclasses import dataclass

import torch

from ..data.synthetic import counter_generator

DEC_POSITION_STREAM = 100_000
AUX_POSITION_STREAM = 200_000
ANSWER_SPAN_STREAM = 300_000


def random_subset_mask(valid: torch.Tensor, size: int, seed: int, step: int, stream: int) -> torch.Tensor:
    """Per row, a uniform random subset of min(size, |valid|) of the row's valid positions."""
    B, L = valid.shape
    out = torch.zeros(B, L, dtype=torch.bool)
    for b in range(B):
        g = counter_generator(seed, step, stream + b)
        idx = valid[b].nonzero()[:, 0]
        take = min(size, idx.numel())
        if take:
            out[b, idx[torch.randperm(idx.numel(), generator=g)[:take]]] = True
    return out


@dataclass(frozen=True)
class AnswerSpanRule:
    min_context: int = 64
    gap_mean: float = 256.0
    span_min: int = 8
    span_max: int = 128


def answer_span_mask(doc_ids: torch.Tensor, valid: torch.Tensor, rule: AnswerSpanRule, seed: int, step: int) -> torch.Tensor:
    B, L = doc_ids.shape
    out = torch.zeros(B, L, dtype=torch.bool)
    p = 1.0 / max(rule.gap_mean, 1.0)
    for b in range(B):
        g = counter_generator(seed, step, ANSWER_SPAN_STREAM + b)
        docs = doc_ids[b].tolist()
        t, doc_pos, prev_doc = 0, 0, None
        u = float(torch.rand(1, generator=g))
        skip = int(math.floor(math.log(max(1.0 - u, 1e-12)) / math.log(max(1.0 - p, 1e-12))))
        while t < L:
            if docs[t] != prev_doc:
                prev_doc, doc_pos = docs[t], 0
            if doc_pos >= rule.min_context:
                if skip == 0:
                    n = int(torch.randint(rule.span_min, rule.span_max + 1, (1,), generator=g))
                    end = t
                    while end < L and end - t < n and docs[end] == prev_doc:
                        end += 1
                    out[b, t:end] = True
                    doc_pos += end - t
                    t = end
                    u = float(torch.rand(1, generator=g))
                    skip = int(math.floor(math.log(max(1.0 - u, 1e-12)) / math.log(max(1.0 - p, 1e-12))))
                    continue
                skip -= 1
            doc_pos += 1
            t += 1
    return out & valid


class PositionSampler:
    """Decoder / auxiliary-head positions of a training batch ("all", "random", or "answer_spans")."""

    def __init__(self, mode: str, seed: int, capacity: int | None = None, rule: AnswerSpanRule | None = None):
        if mode not in ("all", "random", "answer_spans"):
            raise ValueError(f"data.decoder_positions {mode!r}: 'all', 'random' or 'answer_spans'")
        self.mode, self.seed, self.capacity, self.rule = mode, seed, capacity, rule or AnswerSpanRule()

    def mask(self, doc_ids: torch.Tensor, valid: torch.Tensor, step: int) -> torch.Tensor:
        if self.mode == "all":
            return valid.clone()
        if self.mode == "random":
            return random_subset_mask(valid, self.capacity or valid.shape[1], self.seed, step, DEC_POSITION_STREAM)
        return answer_span_mask(doc_ids, valid, self.rule, self.seed, step)
