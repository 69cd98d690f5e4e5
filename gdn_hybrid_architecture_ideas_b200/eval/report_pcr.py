"""Evaluations beyond bits per byte: loss by token position inside the training length, and copy loss on a repeated
random token sequence.

(1) LOSS BY POSITION. Input: the per-position cross-entropy ce (N, L) of a model on the rows of an eval set. Two
position measures, bucketed by the same lower edges POS_EDGES (the last bucket runs to the row's end): "doc" = the
number of earlier positions of the same document in the row (the tokens the model can read: documents are isolated,
so this is the true context length) and "row" = the index in the row. Two masks: "scored" = the positions the set's
bpb scores (their bucket sums add up to the evaluation's own row sums, `check_sums`) and "valid" = every position
with a target in its document. Per set, bucket, measure and mask: nats, bytes, tokens, bpb = nats / (ln 2 bytes) and
the bucket's share of the set's bpb (nats_bucket / (ln 2 bytes_set); the shares add up to the set's bpb). The value
over several sets is the mean of the sets' bucket bpb, defined only where every set holds bytes in the bucket.

(2) COPY LOSS. Item: n ids drawn uniformly from the vocabulary's allowed ids from a fixed seed (one stream per
(variant, n, index)); the item is s s ("pcr_copy2"), s s s ("pcr_copy3") or s t with t an independent draw
("pcr_fresh": what the model pays on random ids it cannot copy). Scored: every token of the copies after the first,
teacher-forced, in nats per token with the argmax-correct share beside it, bucketed by the token's position in its
copy (COPY_EDGES). Bucket 0, the copy's first token, is a fresh draw for the second copy and predictable by induction
for the third, so the copies are kept apart and `nats_after_first` leaves bucket 0 out
(reference: ced/eval/report_pcr.py:1-60; its retrieval cells inside the training length are the needle, multi-key and
variable-tracking items of `eval/probes.py` and `eval/recall_ruler.py` at lengths up to the training length).
"""

from __future__ import annotations

import math

import numpy as np
import torch

from . import tst_diag as TD
from .span_bpb import EvalRows, token_cross_entropy

LN2 = math.log(2.0)
POS_EDGES = (0, 64, 256, 1024, 2048, 4096)
POS_KINDS = ("row", "doc")
MASKS = ("scored", "valid")
WHATS = ("nats", "bytes", "tokens")
COPY_EDGES = (0, 1, 4, 16, 64, 256, 1024)
COPY_VARIANTS = ("pcr_copy2", "pcr_copy3", "pcr_fresh")
COPY_SEED = 20261011


def bucket_names(edges, end: str = "end") -> list[str]:
    return [f"{a}-{b - 1}" if b is not None else f"{a}-{end}" for a, b in zip(edges, list(edges[1:]) + [None])]


# ------------------------------------------------------------------------------------------------ loss by position
@torch.no_grad()
def position_ce(model, rows: EvalRows, batch_size: int = 8, autocast_dtype=None) -> torch.Tensor:
    """(N, L) float32 cross-entropy of every position's target (0-targets of the padding included: mask them)."""
    dev = next(model.parameters()).device
    was_training = model.training
    model.eval()
    out = []
    for s in range(0, rows.tokens.shape[0], batch_size):
        tok, tgt, doc = (t[s:s + batch_size].to(dev) for t in (rows.tokens, rows.targets, rows.doc_ids))
        with torch.autocast(dev.type, dtype=autocast_dtype, enabled=autocast_dtype is not None):
            logits = model(tok, doc).logits
        out.append(token_cross_entropy(logits, tgt).float().cpu())
    model.train(was_training)
    return torch.cat(out)


def bucket_sums(ce, rows: EvalRows, edges=POS_EDGES) -> dict[str, np.ndarray]:
    """{"<kind>_<mask>_<what>": (N, K) float64}: per-row sums over the positions of each bucket."""
    ce = torch.as_tensor(np.array(ce)).double() if not torch.is_tensor(ce) else ce.double()
    N, L = ce.shape
    assert tuple(rows.tokens.shape) == (N, L), f"ce {tuple(ce.shape)} against rows {tuple(rows.tokens.shape)}"
    valid = rows.doc_index >= 0
    masks = {"scored": valid & rows.scored, "valid": valid}
    measures = {"row": torch.arange(L).expand(N, L), "doc": TD.context_in_document(rows.doc_ids)}
    values = {"nats": ce, "bytes": rows.target_bytes.double(), "tokens": torch.ones(N, L, dtype=torch.float64)}
    out = {}
    for kind, x in measures.items():
        key = TD.bucket_of(x, edges)
        for mname, m in masks.items():
            for what, val in values.items():
                out[f"{kind}_{mname}_{what}"] = TD.sum_by(key, len(edges), m, val).numpy()
    return out


def check_sums(sums: dict[str, np.ndarray], row_nats, row_bytes, row_tokens, rtol: float = 1e-5) -> None:
    """The scored buckets of a row add up to the evaluation's own row sums (nats to rtol; bytes and tokens exactly), and
    the valid buckets hold at least as much."""
    for kind in POS_KINDS:
        np.testing.assert_allclose(sums[f"{kind}_scored_nats"].sum(1), np.asarray(row_nats, dtype=np.float64), rtol=rtol, atol=1e-6)
        np.testing.assert_array_equal(sums[f"{kind}_scored_bytes"].sum(1), np.asarray(row_bytes, dtype=np.float64))
        np.testing.assert_array_equal(sums[f"{kind}_scored_tokens"].sum(1), np.asarray(row_tokens, dtype=np.float64))
        for what in ("bytes", "tokens"):
            assert (sums[f"{kind}_valid_{what}"].sum(1) >= sums[f"{kind}_scored_{what}"].sum(1)).all()


def bpb(nats, nbytes) -> float:
    return float(nats) / (LN2 * float(nbytes)) if float(nbytes) > 0 else float("nan")


def set_record(sums: dict[str, np.ndarray]) -> dict:
    """Totals over rows of one set: {kind: {mask: {nats, bytes, tokens, bpb, share: [K], bpb_total, tokens_total}}}."""
    out: dict = {}
    for kind in POS_KINDS:
        out[kind] = {}
        for mname in MASKS:
            n, b, t = (sums[f"{kind}_{mname}_{w}"].sum(0) for w in WHATS)
            bt = float(b.sum())
            out[kind][mname] = {"nats": n.tolist(), "bytes": b.tolist(), "tokens": t.tolist(), "bpb": [bpb(x, y) for x, y in zip(n, b)],
                                "share": [float(x) / (LN2 * bt) if bt > 0 else float("nan") for x in n],
                                "bpb_total": bpb(n.sum(), bt), "tokens_total": int(t.sum())}
    return out


def all_sets(records: dict[str, dict]) -> dict:
    """The mean over sets of each bucket's bpb and share (NaN where a set holds no bytes in the bucket), and of the totals."""
    out: dict = {}
    names = sorted(records)
    for kind in POS_KINDS:
        out[kind] = {}
        for mname in MASKS:
            per = [records[s][kind][mname] for s in names]
            K = len(per[0]["bpb"])
            out[kind][mname] = {
                "bpb": [float(np.mean([p["bpb"][k] for p in per])) for k in range(K)],
                "share": [float(np.mean([p["share"][k] for p in per])) for k in range(K)],
                "bpb_total": float(np.mean([p["bpb_total"] for p in per])), "sets": names}
    return out


def row_clustered_se(sums: dict[str, np.ndarray], kind: str = "doc", mask: str = "scored") -> list[float]:
    """Standard error of each bucket's bpb with the row as the unit (ratio estimator over rows)."""
    n, b = sums[f"{kind}_{mask}_nats"], sums[f"{kind}_{mask}_bytes"]
    out = []
    for k in range(n.shape[1]):
        keep = b[:, k] > 0
        y, x = n[keep, k], b[keep, k]
        if len(y) < 2:
            out.append(float("nan"))
            continue
        r = y.sum() / x.sum()
        out.append(float(np.sqrt(len(y) / (len(y) - 1) * ((y - r * x) ** 2).sum()) / x.sum() / LN2))
    return out


# ------------------------------------------------------------------------------------------------ copy loss
def allowed_ids(vocab_size: int, special_ids=()) -> np.ndarray:
    return np.setdiff1d(np.arange(vocab_size), np.asarray(list(special_ids), dtype=np.int64))


def _copy_rng(variant: str, n: int, index: int, stream: int) -> np.random.Generator:
    return np.random.default_rng([COPY_SEED, COPY_VARIANTS.index(variant), n, index, stream])


def copy_item(allowed: np.ndarray, variant: str, n: int, index: int) -> tuple[np.ndarray, int]:
    """(ids, index of the first scored token). copy2 and fresh share their first half; copy3 repeats it twice."""
    if variant not in COPY_VARIANTS:
        raise ValueError(f"copy variant {variant!r}: one of {COPY_VARIANTS}")
    s = allowed[_copy_rng("pcr_copy2", n, index, 0).integers(0, len(allowed), n)]
    if variant == "pcr_fresh":
        t = allowed[_copy_rng("pcr_fresh", n, index, 1).integers(0, len(allowed), n)]
        return np.concatenate([s, t]), n
    return np.concatenate([s] * (2 if variant == "pcr_copy2" else 3)), n


def copy_item_id(variant: str, n: int, index: int) -> str:
    return f"{variant}/n={n}/{index:04d}"


@torch.no_grad()
def score_copy_items(model, vocab_size: int, lengths=(64, 256, 1024), per_length: int = 8, variants=COPY_VARIANTS,
                     special_ids=(), batch_size: int = 8, autocast_dtype=None) -> list[dict]:
    """One result per item: {"id", "variant", "n", "nats": [...], "correct": [...]} over the scored tokens in order."""
    dev = next(model.parameters()).device
    was_training = model.training
    model.eval()
    allowed = allowed_ids(vocab_size, special_ids)
    results = []
    for variant in variants:
        for n in lengths:
            items = [copy_item(allowed, variant, n, i) for i in range(per_length)]
            for s in range(0, per_length, batch_size):
                ids = torch.as_tensor(np.stack([it[0] for it in items[s:s + batch_size]])).long().to(dev)
                with torch.autocast(dev.type, dtype=autocast_dtype, enabled=autocast_dtype is not None):
                    logits = model(ids[:, :-1], torch.zeros_like(ids[:, :-1])).logits
                ce = token_cross_entropy(logits, ids[:, 1:]).float().cpu()
                ok = (logits.argmax(-1) == ids[:, 1:]).cpu()
                for b in range(ids.shape[0]):
                    results.append({"id": copy_item_id(variant, n, s + b), "variant": variant, "n": n,
                                    "nats": ce[b, n - 1:].tolist(), "correct": ok[b, n - 1:].tolist()})
    model.train(was_training)
    return results


def copy_table(results: list[dict], edges=COPY_EDGES) -> dict:
    """{variant: {n: {"copies": [{"nats": [K], "correct": [K], "tokens": [K]} per scored copy], "nats_per_token",
    "nats_after_first", "correct", "items"}}}: means per bucket of the position inside the copy."""
    K, out = len(edges), {}
    cells: dict = {}
    for r in results:
        cells.setdefault((r["variant"], r["n"]), []).append(r)
    for (variant, n), rs in sorted(cells.items()):
        nats = np.asarray([r["nats"] for r in rs], dtype=np.float64)           # (items, copies * n)
        ok = np.asarray([r["correct"] for r in rs], dtype=np.float64)
        copies = nats.shape[1] // n
        key = np.searchsorted(np.asarray(edges[1:]), np.arange(n), side="right")
        rec = {"copies": [], "items": len(rs)}
        for c in range(copies):
            a, b = nats[:, c * n:(c + 1) * n], ok[:, c * n:(c + 1) * n]
            cnt = np.bincount(key, minlength=K).astype(np.float64) * len(rs)
            with np.errstate(invalid="ignore", divide="ignore"):
                rec["copies"].append({"nats": (np.bincount(key, weights=a.sum(0), minlength=K) / cnt).tolist(),
                                      "correct": (np.bincount(key, weights=b.sum(0), minlength=K) / cnt).tolist(),
                                      "tokens": cnt.tolist()})
        rec["nats_per_token"] = float(nats.mean())
        after = np.concatenate([nats[:, c * n + 1:(c + 1) * n] for c in range(copies)], axis=1)
        rec["nats_after_first"] = float(after.mean()) if after.size else float("nan")
        rec["correct"] = float(ok.mean())
        out.setdefault(variant, {})[n] = rec
    return out


def copy_gain(table: dict) -> dict:
    """Per length: nats per token saved by the repeat, fresh minus copy2 (after the first token)."""
    out = {}
    for n, rec in table.get("pcr_copy2", {}).items():
        fresh = table.get("pcr_fresh", {}).get(n)
        if fresh:
            out[n] = fresh["nats_after_first"] - rec["nats_after_first"]
    return out
