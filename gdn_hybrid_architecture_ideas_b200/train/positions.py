"""Position masks drawn per (seed, step, row): uniform random subsets of a row's valid targets, causal answer spans,
and fixed-count span masks; the positions a restricted scoring regime adds around scored spans (sinks, replay).

Every mask is a pure function of (data seed, step, row) and the batch's own valid mask, drawn from counter-based
generators, so resume needs only the step and every process computes the same masks. The answer-span rule decides
position t from the RNG and the document structure at positions <= t only, so a scored position never learns where its
document ends: walk the row; a position may start a span once its document has `min_context` earlier positions; skip a
geometric number of eligible positions (mean `gap_mean`), open a span of a length from [span_min, span_max], cut it at
the document's end, continue after it; finally AND with the valid targets
(reference: ced/train/positions.py:109-353).

`span_mask` marks EXACTLY `count` positions of a row in spans whose lengths follow a truncated log-normal (or uniform)
law, placed by the RNG alone (never by tokens or document boundaries: a placement that depended on where a document ends
would tell earlier positions about the future). It is what fixed-seed evaluation rows with a given number of scored
positions use (`eval/span_bpb.build_span_rows`) (reference: ced/train/data.py:73-150, own construction: lengths by the
inverse CDF restricted to the interval, then the free positions dealt to the gaps as a uniform random composition).
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


def truncated_lognormal(g: torch.Generator, n: int, lo: int, hi: int, median: float, sigma: float) -> torch.Tensor:
    """n integer draws in [lo, hi] from a log-normal truncated (not clamped) to the interval that rounds into it."""
    mu = math.log(median)
    cdf = lambda x: torch.special.ndtr(torch.tensor((math.log(max(x, 1e-9)) - mu) / sigma, dtype=torch.float64))
    a, b = cdf(lo - 0.5), cdf(hi + 0.5)
    u = a + (b - a) * torch.rand(n, generator=g, dtype=torch.float64)
    x = torch.exp(mu + sigma * torch.special.ndtri(u.clamp(1e-15, 1 - 1e-15)))
    return x.round().clamp(lo, hi).long()


def span_mask(length: int, count: int, g: torch.Generator, distribution: str = "lognormal", median: float = 230.0, sigma: float = 1.16,
              span_min: int = 16, span_max: int = 4096) -> torch.Tensor:
    """(length,) bool with exactly `count` true positions in spans of lengths from [span_min, min(count, span_max)]; a span
    that would overshoot is cut to the remainder and a remainder shorter than span_min joins the span before it; neighbouring
    spans are at least one position apart when the row has room."""
    if not 0 <= count <= length:
        raise ValueError(f"{count} span positions do not fit a row of {length}")
    mask = torch.zeros(length, dtype=torch.bool)
    if count == 0:
        return mask
    lo = max(1, min(span_min, count))
    hi = max(lo, min(span_max, count))
    spans, left = [], count
    while left > 0:
        need = max(1, -(-left // lo))
        if distribution == "uniform":
            draws = torch.randint(lo, hi + 1, (need,), generator=g).tolist()
        elif distribution == "lognormal":
            draws = truncated_lognormal(g, need, lo, hi, median, sigma).tolist()
        else:
            raise ValueError(f"unknown span distribution {distribution!r}")
        for n in draws:
            if n >= left or left - n < lo:
                n = left
            spans.append(n)
            left -= n
            if left == 0:
                break
    k = len(spans)
    free = length - count
    apart = 1 if free >= k - 1 else 0
    spare = free - apart * (k - 1)
    # a uniform random composition of `spare` into k + 1 gaps (before the first span, between spans, after the last)
    cuts = torch.sort(torch.randint(0, spare + 1, (k,), generator=g)).values.tolist()
    at, prev = 0, 0
    for i, n in enumerate(spans):
        at += (cuts[i] - prev) + (apart if i else 0)
        prev = cuts[i]
        mask[at:at + n] = True
        at += n
    assert int(mask.sum()) == count
    return mask


def document_positions(doc_ids: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    """Per position of (B, L) document ids: its index inside its document's part of the row, and that part's first position."""
    B, L = doc_ids.shape
    idx = torch.arange(L).expand(B, L)
    new = torch.ones(B, L, dtype=torch.bool)
    new[:, 1:] = doc_ids[:, 1:] != doc_ids[:, :-1]
    first = torch.where(new, idx, torch.zeros_like(idx)).cummax(dim=1).values
    return idx - first, first


def sink_positions(doc_ids: torch.Tensor, n_sinks: int) -> torch.Tensor:
    """The first n_sinks positions of every document's part of a row."""
    return document_positions(doc_ids)[0] < n_sinks


def span_starts(doc_ids: torch.Tensor, scored: torch.Tensor) -> torch.Tensor:
    """Scored positions whose previous position in the same document is not scored."""
    prev = torch.zeros_like(scored)
    prev[:, 1:] = scored[:, :-1] & (doc_ids[:, 1:] == doc_ids[:, :-1])
    return scored & ~prev


def replay_positions(doc_ids: torch.Tensor, scored: torch.Tensor, window: int) -> torch.Tensor:
    """The min(window, available) positions immediately before every span start, inside its document; never a scored one."""
    B, L = scored.shape
    starts = span_starts(doc_ids, scored)
    within, _ = document_positions(doc_ids)
    out = torch.zeros_like(scored)
    for b, t in starts.nonzero().tolist():
        lo = max(t - window, t - int(within[b, t]))
        out[b, lo:t] = True
    return out & ~scored


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
