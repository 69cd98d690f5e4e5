"""Decoder-position spans of a pretraining row for the looped encoder-decoder: exactly n positions of a row marked in spans.

Span lengths come from `data.span_distribution` inside [span_min, min(n, span_max)]: uniform, or a log-normal of median
`span_median` and log-deviation `span_sigma` TRUNCATED to that range (one inverse-CDF draw over the interval that rounds into
it, so the shape inside the range is the fitted one even where the range holds little mass). Lengths are drawn until n
positions are covered; the last span is cut to what remains, and a span that would leave fewer than span_min positions
takes them too (no tiny trailing span). The spans are then placed uniformly at random with one context position between
neighbours when the row has room: the free positions are dealt to the gaps through sorted uniform cuts. The placement reads
the row's length and the generator alone, never tokens or document boundaries, so which kind of key a position offers
carries no information about the future. Draw for draw the reference's sampler (ced/train/data.py:74-145).
"""

from __future__ import annotations

import math

import torch

DISTRIBUTIONS = ("lognormal", "uniform")


def truncated_lognormal(g: torch.Generator, lo: int, hi: int, median: float, sigma: float) -> int:
    """One length in [lo, hi] from the log-normal restricted to [lo - 0.5, hi + 0.5]."""
    mu = math.log(median)
    cdf = lambda x: torch.special.ndtr(torch.tensor((math.log(x) - mu) / sigma, dtype=torch.float64))        # noqa: E731
    below, above = cdf(max(lo - 0.5, 1e-9)), cdf(hi + 0.5)
    u = below + (above - below) * torch.rand((), generator=g, dtype=torch.float64)
    return min(hi, max(lo, round(math.exp(mu + sigma * float(torch.special.ndtri(u))))))


def span_lengths(n: int, g: torch.Generator, distribution: str, median: float, sigma: float, span_min: int, span_max: int) -> list:
    if distribution not in DISTRIBUTIONS:
        raise ValueError(f"data.span_distribution {distribution!r}: one of {DISTRIBUTIONS}")
    lo = max(1, min(span_min, n))
    hi = max(lo, min(span_max, n))
    out, left = [], n
    while left > 0:
        if distribution == "uniform":
            span = int(torch.randint(lo, hi + 1, (1,), generator=g))
        else:
            span = truncated_lognormal(g, lo, hi, median, sigma)
        if left - span < lo:          # the rest would be a span shorter than the minimum (or nothing): this one takes it
            span = left
        out.append(span)
        left -= span
    return out


def place_spans(length: int, lengths: list, g: torch.Generator) -> torch.Tensor:
    """(length,) bool with the spans placed in order; span i starts at cuts[i] + the spans before it + i separators."""
    n, covered = len(lengths), sum(lengths)
    free = length - covered
    apart = 1 if free >= n - 1 else 0
    cuts = torch.randint(0, free - apart * (n - 1) + 1, (n,), generator=g).sort().values
    sizes = torch.tensor(lengths)
    starts = cuts + (sizes.cumsum(0) - sizes) + apart * torch.arange(n)
    edges = torch.zeros(length + 1, dtype=torch.long)
    edges.scatter_add_(0, starts, torch.ones(n, dtype=torch.long))
    edges.scatter_add_(0, starts + sizes, -torch.ones(n, dtype=torch.long))
    return edges.cumsum(0)[:length] > 0


def sample_spans(length: int, n_dec: int, g: torch.Generator, *, distribution: str = "lognormal", median: float = 230.0, sigma: float = 1.16,
                 span_min: int = 16, span_max: int = 4096) -> torch.Tensor:
    if not 0 <= n_dec <= length:
        raise ValueError(f"{n_dec} decoder positions in a row of {length}")
    if n_dec == 0:
        return torch.zeros(length, dtype=torch.bool)
    return place_spans(length, span_lengths(n_dec, g, distribution, median, sigma, span_min, span_max), g)
