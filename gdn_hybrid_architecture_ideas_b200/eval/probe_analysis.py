"""Analysis of per-item probe results: item metrics from the per-token record, pooled values with their item-sampling
standard error, clustered pooling for items that share content, first-error histograms and marginal tables.

An item's record is the teacher-forced result over its answer tokens: ok[i] (the argmax is the gold token) and
nats[i] (-log p of the gold token), as `probes.score_probes(..., keep_tokens=True)` returns them.

    exact, token_acc, nats_per_token         the whole answer
    nats_first, first_acc                    the first answer token alone (the one that decides what is read)
    nats_per_token_rest, token_acc_rest, exact_rest   tokens 2..n (an item of one token has none)
    first_err_frac                           the position of the first wrong token / n (1.0: none wrong)
    exp_exact_t1                             exp(-sum nats): the chance that sampling at temperature 1 writes the answer

A pooled value is the item mean with SE = std / sqrt(n). Items that share their content (the two directions of one
transcode base) form a cluster: its value is the mean of its members, the SE is over clusters, and the difference
between the members carries its own paired SE (reference: ced/eval/probe_copy_analysis.py:1-37, 139-175,
ced/eval/probe_transcode_analysis.py:33-98).
"""

from __future__ import annotations

import math
from collections import defaultdict

REST_KEYS = ("nats_per_token_rest", "token_acc_rest", "exact_rest")
COMPANION_KEYS = REST_KEYS + ("nats_first", "first_acc")
TABLE_METRICS = ("exact", "token_acc", "nats_per_token", "first_err_frac", "exp_exact_t1") + COMPANION_KEYS


def item_metrics(ok: list[bool], nats: list[float]) -> dict:
    n = len(ok)
    assert n == len(nats) and n > 0
    wrong = next((i for i, o in enumerate(ok) if not o), n)
    out = {"exact": float(all(ok)), "token_acc": sum(ok) / n, "nats_per_token": sum(nats) / n, "nats_first": nats[0],
           "first_acc": float(ok[0]), "first_err_frac": wrong / n, "exp_exact_t1": math.exp(-sum(nats)), "tokens": n}
    if n > 1:
        out.update(nats_per_token_rest=sum(nats[1:]) / (n - 1), token_acc_rest=sum(ok[1:]) / (n - 1), exact_rest=float(all(ok[1:])))
    return out


def mean_se(values: list[float]):
    n = len(values)
    if n == 0:
        return None, None
    mean = sum(values) / n
    if n == 1:
        return mean, None
    return mean, math.sqrt(sum((v - mean) ** 2 for v in values) / (n - 1) / n)


def with_metrics(items: list[dict]) -> list[dict]:
    """Items of `score_probes(keep_tokens=True)` with their metrics merged in."""
    return [{**it, **item_metrics(it["ok"], it["nats"])} for it in items]


def pooled(items: list[dict], metric: str = "nats_per_token", where=None) -> dict | None:
    vals = [it[metric] for it in items if metric in it and (where is None or where(it))]
    if not vals:
        return None
    m, se = mean_se(vals)
    return {"value": m, "se": se, "n": len(vals)}


def clusters(items: list[dict], key) -> dict:
    out = defaultdict(list)
    for it in items:
        out[key(it)].append(it)
    return dict(out)


def pooled_clustered(items: list[dict], key, metric: str = "nats_per_token") -> dict | None:
    """The mean over clusters of each cluster's member mean; SE over clusters."""
    vals = [sum(m[metric] for m in ms) / len(ms) for ms in clusters(items, key).values() if all(metric in m for m in ms)]
    if not vals:
        return None
    m, se = mean_se(vals)
    return {"value": m, "se": se, "clusters": len(vals)}


def paired_difference(items: list[dict], key, member, a, b, metric: str = "nats_per_token") -> dict | None:
    """Member a minus member b inside each cluster that holds both (member(item) names the member), with its paired SE."""
    diffs = []
    for ms in clusters(items, key).values():
        by = {member(m): m for m in ms}
        if a in by and b in by and metric in by[a] and metric in by[b]:
            diffs.append(by[a][metric] - by[b][metric])
    if not diffs:
        return None
    m, se = mean_se(diffs)
    return {"diff": m, "se": se, "pairs": len(diffs)}


def paired_between_runs(a: list[dict], b: list[dict], metric: str = "nats_per_token", ident=lambda it: it["id"]) -> dict | None:
    """Run a minus run b on the items both scored, matched by id."""
    other = {ident(it): it for it in b}
    diffs = [it[metric] - other[ident(it)][metric] for it in a if ident(it) in other and metric in it and metric in other[ident(it)]]
    if not diffs:
        return None
    m, se = mean_se(diffs)
    return {"diff": m, "se": se, "n": len(diffs)}


def marginal_table(items: list[dict], by: tuple[str, ...], metrics=TABLE_METRICS, where=None) -> dict:
    """{"<by values joined by |>": {metric: {"value", "se", "n"}}} over the items that pass `where`."""
    groups = defaultdict(list)
    for it in items:
        if where is None or where(it):
            groups["|".join(str(it.get(k)) for k in by)].append(it)
    return {g: {m: pooled(ms, m) for m in metrics if pooled(ms, m) is not None} for g, ms in sorted(groups.items())}


def first_error_hist(items: list[dict], bins=(0.0, 0.25, 0.5, 0.75, 1.0), where=None) -> dict:
    """Where the first wrong token falls, as a share of the answer: counts per [bins[i], bins[i+1]) among the items with
    an error, and the share of items with none."""
    sel = [it for it in items if where is None or where(it)]
    counts = [0] * (len(bins) - 1)
    for it in sel:
        f = it["first_err_frac"]
        if f < 1.0:
            counts[max(i for i in range(len(bins) - 1) if f >= bins[i])] += 1
    return {"bins": list(bins), "counts": counts, "no_error": sum(it["first_err_frac"] >= 1.0 for it in sel) / max(len(sel), 1), "n": len(sel)}
