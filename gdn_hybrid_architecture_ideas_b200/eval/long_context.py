"""Long-context scoring: cross-entropy by position bucket.

A long document is one row; positions are grouped into buckets with edges base, 2 base, 4 base, ... and bits per byte
are reported per bucket, with ratio-estimator standard errors over documents. A model that uses its context gets
lower bpb in later buckets (reference: ced/eval/long_context.py:73-112 buckets, :207-253 position CE, :475-575 tables).
"""

from __future__ import annotations

import math

import torch

from .span_bpb import ratio_se, token_cross_entropy

BASE_LEN = 2048


def default_edges(base: int = BASE_LEN, top: int = 1 << 20) -> tuple[int, ...]:
    edges, e = [], base
    while e <= top:
        edges.append(e)
        e *= 2
    return tuple(edges)


def length_label(n: int) -> str:
    return f"{n // 1024}k" if n and n % 1024 == 0 else str(n)


def bucket_names(edges) -> list[str]:
    lo = [0] + list(edges)
    return [f"{length_label(a)}-{length_label(b)}" for a, b in zip(lo[:-1], edges)] + [f">{length_label(edges[-1])}"]


def bucket_index(positions: torch.Tensor, edges) -> torch.Tensor:
    return torch.bucketize(positions, torch.tensor(list(edges), device=positions.device), right=True)


def bucket_sums(values: torch.Tensor, positions: torch.Tensor, edges, weight: torch.Tensor | None = None) -> torch.Tensor:
    """Sum of `values` (times weight) per bucket: (len(edges) + 1,) float64."""
    out = torch.zeros(len(edges) + 1, dtype=torch.float64, device=values.device)
    v = values.double() if weight is None else values.double() * weight.double()
    return out.index_add_(0, bucket_index(positions, edges).reshape(-1), v.reshape(-1))


@torch.no_grad()
def position_ce(model, ids: torch.Tensor, chunk: int = 8192, autocast_dtype=None) -> torch.Tensor:
    """Per-position CE of one long document (ids (n,)), read in chunks through the cache so memory stays flat.
    Returns (n - 1,) float32 on the CPU."""
    dev = next(model.parameters()).device
    tok = ids[:-1].to(dev)[None]
    tgt = ids[1:].to(dev)[None]
    doc = torch.zeros_like(tok)
    cache, parts = None, []
    for s in range(0, tok.shape[1], chunk):
        with torch.autocast(dev.type, dtype=autocast_dtype, enabled=autocast_dtype is not None):
            out = model.forward(tok[:, s:s + chunk], doc[:, s:s + chunk], cache=cache, return_cache=True)
        cache = out.cache
        parts.append(token_cross_entropy(out.logits, tgt[:, s:s + chunk])[0].cpu())
    return torch.cat(parts)


def bucket_table(records: list[dict], edges) -> list[dict]:
    """records: per document {"nats": (buckets,), "bytes": (buckets,)}. One line per bucket: bpb, its standard error over
    documents, and the number of documents reaching the bucket."""
    names = bucket_names(edges)
    y = torch.stack([r["nats"] for r in records]).double()
    x = torch.stack([r["bytes"] for r in records]).double()
    rows = []
    for b, name in enumerate(names):
        r, se, n = ratio_se(y[:, b], x[:, b])
        rows.append({"bucket": name, "bpb": r / math.log(2.0) if n else None, "se": se / math.log(2.0) if n > 1 else None, "docs": n})
    return rows


@torch.no_grad()
def score_position_bpb(model, docs: list[dict], edges=None, base: int = BASE_LEN, max_len: int | None = None, chunk: int = 8192,
                       autocast_dtype=None) -> dict:
    """docs: {"ids": LongTensor (n,), "byte_lens": LongTensor (n,)}. Returns the bucket table and the records."""
    edges = edges or default_edges(base, max(base, max_len or max(len(d["ids"]) for d in docs)))
    records = []
    for d in docs:
        ids = d["ids"][:max_len] if max_len else d["ids"]
        ce = position_ce(model, ids, chunk, autocast_dtype)
        pos = torch.arange(1, len(ids))
        by = d["byte_lens"][1:len(ids)]
        records.append({"nats": bucket_sums(ce, pos, edges), "bytes": bucket_sums(by.double(), pos, edges), "tokens": len(ids) - 1})
    return {"edges": list(edges), "table": bucket_table(records, edges), "records": records}
