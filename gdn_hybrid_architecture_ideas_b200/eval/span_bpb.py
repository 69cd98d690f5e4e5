"""Bits per byte at scored positions.

Documents (token ids, byte length per token, a scored mask) are packed into rows of `seq_len`; a document never
crosses a row and gets its own document id, so it reads nothing of its neighbours. `evaluate` returns per-row sums of
nats and bytes (rows can be scored on several ranks and joined), `bpb = nats / (bytes ln 2)`, and a ratio-estimator
standard error over rows (reference: ced/eval/span_bpb.py:118-260 packing, :703-1060 evaluation and joining,
:1106-1194 standard errors).
"""

from __future__ import annotations

import math
from dataclasses import dataclass, field

import torch


@dataclass
class TokenizedDoc:
    ids: list[int]
    byte_lens: list[int]                 # bytes each token stands for
    scored: list[bool] | None = None     # which TARGET tokens count (None: all but the first)
    name: str = ""


@dataclass
class EvalRows:
    tokens: torch.Tensor        # (R, L) inputs
    targets: torch.Tensor       # (R, L) next token (0 where none)
    doc_ids: torch.Tensor       # (R, L); padding is its own document
    scored: torch.Tensor        # (R, L) bool: the target at this position counts
    target_bytes: torch.Tensor  # (R, L) bytes of the target token
    doc_index: torch.Tensor     # (R, L) index into the document list (-1 padding)
    n_docs: int = 0
    skipped: list[int] = field(default_factory=list)    # documents longer than a row


def build_eval_rows(docs: list[TokenizedDoc], seq_len: int, pad_id: int = 0) -> EvalRows:
    """First-fit in order: a document of n tokens takes n - 1 positions (inputs ids[:-1], targets ids[1:])."""
    rows, cur, used, skipped = [], [], 0, []
    for i, d in enumerate(docs):
        n = len(d.ids) - 1
        if n < 1:
            continue
        if n > seq_len:
            skipped.append(i)
            continue
        if used + n > seq_len:
            rows.append(cur)
            cur, used = [], 0
        cur.append(i)
        used += n
    if cur:
        rows.append(cur)
    R = len(rows)
    tokens = torch.full((R, seq_len), pad_id, dtype=torch.long)
    targets = torch.zeros(R, seq_len, dtype=torch.long)
    doc_ids = torch.zeros(R, seq_len, dtype=torch.long)
    scored = torch.zeros(R, seq_len, dtype=torch.bool)
    tbytes = torch.zeros(R, seq_len, dtype=torch.long)
    dindex = torch.full((R, seq_len), -1, dtype=torch.long)
    for r, members in enumerate(rows):
        at = 0
        for slot, i in enumerate(members):
            d = docs[i]
            n = len(d.ids) - 1
            ids = torch.tensor(d.ids, dtype=torch.long)
            tokens[r, at:at + n], targets[r, at:at + n] = ids[:-1], ids[1:]
            doc_ids[r, at:at + n] = slot
            sc = torch.ones(n, dtype=torch.bool) if d.scored is None else torch.tensor(d.scored[1:], dtype=torch.bool)
            scored[r, at:at + n] = sc
            tbytes[r, at:at + n] = torch.tensor(d.byte_lens[1:], dtype=torch.long)
            dindex[r, at:at + n] = i
            at += n
        doc_ids[r, at:] = len(members)          # the padding tail is one more document
    return EvalRows(tokens, targets, doc_ids, scored, tbytes, dindex, n_docs=len(docs), skipped=skipped)


@dataclass
class SpanEval:
    row_nats: torch.Tensor      # (R,) float64 sum of CE over scored positions
    row_bytes: torch.Tensor     # (R,) bytes of the scored targets
    row_tokens: torch.Tensor    # (R,)
    doc_nats: torch.Tensor      # (n_docs,)
    doc_bytes: torch.Tensor

    @property
    def bpb(self) -> float:
        return bpb(self.row_nats.sum(), self.row_bytes.sum())

    @property
    def ce(self) -> float:
        return float(self.row_nats.sum() / self.row_tokens.sum().clamp_min(1))


def bpb(nats, n_bytes) -> float:
    return float(nats) / (max(float(n_bytes), 1.0) * math.log(2.0))


def token_cross_entropy(logits: torch.Tensor, targets: torch.Tensor, chunk: int = 1024) -> torch.Tensor:
    """CE per position in fp32, the vocabulary reduced a chunk of positions at a time."""
    flat, t = logits.reshape(-1, logits.shape[-1]), targets.reshape(-1)
    out = torch.empty(flat.shape[0], dtype=torch.float32, device=logits.device)
    for s in range(0, flat.shape[0], chunk):
        lg = flat[s:s + chunk].float()
        out[s:s + chunk] = torch.logsumexp(lg, -1) - lg.gather(1, t[s:s + chunk, None])[:, 0]
    return out.view(targets.shape)


@torch.no_grad()
def evaluate(model, rows: EvalRows, batch_size: int = 8, autocast_dtype=None, row_indices: list[int] | None = None) -> SpanEval:
    """Scores `row_indices` (default: all rows); rows not scored keep zero sums, so partial results add up."""
    dev = next(model.parameters()).device
    was_training = model.training
    model.eval()
    R = rows.tokens.shape[0]
    idx = list(range(R)) if row_indices is None else list(row_indices)
    row_nats = torch.zeros(R, dtype=torch.float64)
    doc_nats = torch.zeros(rows.n_docs, dtype=torch.float64)
    for s in range(0, len(idx), batch_size):
        sel = torch.tensor(idx[s:s + batch_size], dtype=torch.long)
        tok, tgt, doc = (t[sel].to(dev) for t in (rows.tokens, rows.targets, rows.doc_ids))
        with torch.autocast(dev.type, dtype=autocast_dtype, enabled=autocast_dtype is not None):
            logits = model(tok, doc).logits
        ce = token_cross_entropy(logits, tgt).double().cpu() * rows.scored[sel]
        row_nats[sel] = ce.sum(1)
        di = rows.doc_index[sel]
        keep = di >= 0
        doc_nats.index_add_(0, di[keep], ce[keep])
    model.train(was_training)
    mask = torch.zeros(R, dtype=torch.bool)
    mask[idx] = True
    sc = rows.scored & mask[:, None]
    row_bytes = (rows.target_bytes * sc).sum(1).double()
    doc_bytes = torch.zeros(rows.n_docs, dtype=torch.float64)
    keep = (rows.doc_index >= 0) & sc
    doc_bytes.index_add_(0, rows.doc_index[keep], rows.target_bytes[keep].double())
    return SpanEval(row_nats, row_bytes, sc.sum(1).double(), doc_nats, doc_bytes)


def join_batches(parts: list[SpanEval]) -> SpanEval:
    """Sum of partial results over disjoint row sets (sharded evaluation)."""
    first = parts[0]
    out = SpanEval(*(torch.zeros_like(getattr(first, f)) for f in ("row_nats", "row_bytes", "row_tokens", "doc_nats", "doc_bytes")))
    for p in parts:
        for f in ("row_nats", "row_bytes", "row_tokens", "doc_nats", "doc_bytes"):
            getattr(out, f).add_(getattr(p, f))
    return out


def ratio_se(y: torch.Tensor, x: torch.Tensor) -> tuple[float, float, int]:
    """(ratio, standard error, n) of sum(y) / sum(x) over units with x > 0 (linearised ratio estimator)."""
    keep = x > 0
    y, x = y[keep].double(), x[keep].double()
    n = int(keep.sum())
    if n < 2:
        return (float(y.sum() / x.sum().clamp_min(1e-30)), float("nan"), n)
    r = y.sum() / x.sum()
    resid = y - r * x
    var = n / (n - 1) * (resid * resid).sum() / (x.sum() ** 2)
    return float(r), float(var.sqrt()), n


def bpb_se(e: SpanEval, by: str = "doc") -> float:
    y, x = (e.doc_nats, e.doc_bytes) if by == "doc" else (e.row_nats, e.row_bytes)
    return ratio_se(y, x)[1] / math.log(2.0)


@dataclass
class PairedDifference:
    diff_bpb: float
    se: float
    n: int


def paired_difference(a: SpanEval, b: SpanEval) -> PairedDifference:
    """bpb(a) - bpb(b) on the same documents with the standard error of the paired per-document differences."""
    keep = (a.doc_bytes > 0) & (b.doc_bytes > 0)
    x = a.doc_bytes[keep]
    d = (a.doc_nats[keep] - b.doc_nats[keep])
    r, se, n = ratio_se(d, x)
    return PairedDifference(r / math.log(2.0), se / math.log(2.0), n)
