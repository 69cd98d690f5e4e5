"""Multiple choice by likelihood: each (context, choice) pair is a document whose choice tokens are scored; the
predicted choice has the lowest summed CE (also reported normalised by bytes)
(reference: ced/eval/multiple_choice.py:36-240)."""

from __future__ import annotations

from dataclasses import dataclass

import torch

from .span_bpb import TokenizedDoc, build_eval_rows, evaluate


@dataclass
class Item:
    context: list[int]
    choices: list[list[int]]
    answer: int
    choice_bytes: list[int] | None = None


def build_documents(items: list[Item]) -> tuple[list[TokenizedDoc], list[tuple[int, int]]]:
    """One document per (item, choice); index[d] = (item, choice)."""
    docs, index = [], []
    for i, it in enumerate(items):
        for c, ch in enumerate(it.choices):
            ids = it.context + ch
            scored = [False] * len(it.context) + [True] * len(ch)
            nb = (it.choice_bytes[c] if it.choice_bytes else len(ch))
            per = max(nb // max(len(ch), 1), 1)
            docs.append(TokenizedDoc(ids, [1] * len(it.context) + [per] * len(ch), scored))
            index.append((i, c))
    return docs, index


def score_items(model, items: list[Item], seq_len: int = 8192, batch_size: int = 1, autocast_dtype=None) -> dict:
    docs, index = build_documents(items)
    rows = build_eval_rows(docs, seq_len)
    ev = evaluate(model, rows, batch_size, autocast_dtype)
    correct = correct_norm = 0
    for i, it in enumerate(items):
        ds = [d for d, (ii, _) in enumerate(index) if ii == i]
        nats = torch.stack([ev.doc_nats[d] for d in ds])
        norm = nats / torch.stack([ev.doc_bytes[d] for d in ds]).clamp_min(1)
        correct += int(int(nats.argmin()) == it.answer)
        correct_norm += int(int(norm.argmin()) == it.answer)
    n = max(len(items), 1)
    return {"acc": correct / n, "acc_norm": correct_norm / n, "n": len(items), "skipped_docs": len(rows.skipped)}
