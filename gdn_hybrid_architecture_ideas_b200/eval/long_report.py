"""Long-context summary and the degradation rule: what breaks first as length grows.

Metrics (reference: ced/eval/long_report.py:1-40 defines the rule and the thresholds):

    bpb.<set>     bpb(full context) - bpb(the same targets with only the last `window` tokens of context), per position
                  bucket: a difference on the same target tokens, so it does not include the ordinary drop of bpb with
                  position. Beyond the training length it should stay <= 0; above +0.010 bpb the long context hurts.
    gdn.<stat>    the worst GDN layer's factor max(r, 1 / r), r = the layer's statistic in the bucket over its value in
                  the reference bucket (state norm, effective rank, relative change per token); above 1.5 it drifted.

A metric is "degraded" at a length when its value exceeds its threshold and "clear" when it does so by more than twice
its standard error (factors without a standard error count as clear; a difference over one document never does).
"""

from __future__ import annotations

import math

import torch

from .long_context import bucket_names, bucket_sums, position_ce
from .span_bpb import ratio_se

THRESHOLDS = {"bpb": 0.010, "gdn": 1.5}


@torch.no_grad()
def context_gain(model, docs: list[dict], edges, window: int, chunk: int = 8192, autocast_dtype=None, full_records: list[dict] | None = None) -> list[dict]:
    """Per bucket [lo, hi) beyond `window`: bpb of the bucket's targets with the full context minus the same targets scored
    from a fresh start `window` tokens before the bucket. One line per bucket: {"bucket", "length", "full", "short", "diff",
    "se", "docs"} (se over documents of the per-document difference ratio)."""
    names = bucket_names(edges)
    rows = []
    for b in range(len(edges) - 1):
        lo, hi = edges[b], edges[b + 1]
        if lo < window:
            continue
        dn, by = [], []
        for i, d in enumerate(docs):
            ids = d["ids"]
            if len(ids) <= lo + 1:
                continue
            end = min(hi, len(ids))
            if full_records is not None:
                full = float(full_records[i]["nats"][b + 1])      # bucket_sums: index b + 1 holds positions in [edges[b], edges[b + 1])
            else:
                ce = position_ce(model, ids[:end], chunk, autocast_dtype)
                full = float(bucket_sums(ce, torch.arange(1, end), edges)[b + 1])
            start = lo - window
            ce_s = position_ce(model, ids[start:end], chunk, autocast_dtype)          # targets start + 1 .. end - 1
            pos = torch.arange(start + 1, end)
            short = float(ce_s[pos >= max(lo, 1)].sum())
            nbytes = float(d["byte_lens"][max(lo, 1):end].sum())
            dn.append((full, short))
            by.append(nbytes)
        if not dn:
            continue
        f = torch.tensor([x[0] for x in dn], dtype=torch.float64)
        s = torch.tensor([x[1] for x in dn], dtype=torch.float64)
        x = torch.tensor(by, dtype=torch.float64)
        diff, se, n = ratio_se(f - s, x)
        ln2 = math.log(2.0)
        rows.append({"bucket": names[b + 1], "length": hi, "full": float(f.sum() / x.sum()) / ln2, "short": float(s.sum() / x.sum()) / ln2,
                     "diff": diff / ln2, "se": se / ln2 if n > 1 else None, "docs": n})
    return rows


def gdn_factors(diag: dict, ref_bucket: int = 0) -> list[dict]:
    """From per-layer statistics by bucket ({"layers": [{"norm": [...], "erank": [...], "rel_delta": [...]}], "edges": [...]}):
    per bucket and statistic the worst layer's factor max(r, 1 / r) against the reference bucket."""
    out = []
    edges = diag["edges"]
    for b in range(len(edges) - 1):
        if b == ref_bucket:
            continue
        for stat in ("norm", "erank", "rel_delta"):
            worst, layer_at = 1.0, None
            for li, layer in enumerate(diag["layers"]):
                vals = layer.get(stat)
                if not vals or vals[b] is None or not vals[ref_bucket]:
                    continue
                r = vals[b] / vals[ref_bucket]
                f = max(r, 1.0 / r) if r > 0 else float("inf")
                if f > worst:
                    worst, layer_at = f, li
            out.append({"length": edges[b + 1], "stat": stat, "factor": worst, "layer": layer_at})
    return out


def _entry(metric, length, value, se, threshold, kind="difference"):
    if value is None or (isinstance(value, float) and math.isnan(value)):
        return None
    degraded = value > threshold
    clear = degraded and (kind == "factor" or (se is not None and value - threshold > 2 * se))
    return {"metric": metric, "length": length, "value": value, "se": se, "threshold": threshold, "degraded": degraded, "clear": clear, "kind": kind}


def degradations(summary: dict, thresholds: dict | None = None, train_len: int = 0) -> list[dict]:
    """summary: {"bpb": {set: context_gain rows}, "gdn": gdn_factors rows}. Entries beyond the training length."""
    th = {**THRESHOLDS, **(thresholds or {})}
    out = []
    for name, rows in summary.get("bpb", {}).items():
        for r in rows:
            if r["length"] > train_len:
                out.append(_entry(f"bpb.{name}", r["length"], r["diff"], r["se"], th["bpb"]))
    for r in summary.get("gdn", []):
        if r["length"] > train_len:
            out.append(_entry(f"gdn.{r['stat']}", r["length"], r["factor"], None, th["gdn"], "factor"))
    return [e for e in out if e is not None]


def breaks_first(entries: list[dict], clear_only: bool = False) -> dict:
    """The shortest length at which anything degrades, and what does there."""
    bad = [e for e in entries if e["degraded"] and (e["clear"] or not clear_only)]
    if not bad:
        return {"length": None, "metrics": []}
    at = min(e["length"] for e in bad)
    return {"length": at, "metrics": sorted(e["metric"] for e in bad if e["length"] == at)}


def render(summary: dict, entries: list[dict]) -> str:
    """Markdown: the context-gain table per set and the list of degradations."""
    lines = []
    for name, rows in summary.get("bpb", {}).items():
        lines += [f"### {name}: bpb with the full context minus the same targets with a short context", "",
                  "| bucket | full | short | difference | docs |", "|---|---|---|---|---|"]
        for r in rows:
            se = "" if r["se"] is None else f" +- {r['se']:.4f}"
            lines.append(f"| {r['bucket']} | {r['full']:.4f} | {r['short']:.4f} | {r['diff']:+.4f}{se} | {r['docs']} |")
        lines.append("")
    first = breaks_first(entries)
    lines.append("Nothing degrades." if first["length"] is None else f"Breaks first at {first['length']}: {', '.join(first['metrics'])}.")
    for e in entries:
        if e["degraded"]:
            lines.append(f"- {e['metric']} at {e['length']}: {e['value']:.4f} over {e['threshold']} ({'clear' if e['clear'] else 'within noise'})")
    return "\n".join(lines) + "\n"
