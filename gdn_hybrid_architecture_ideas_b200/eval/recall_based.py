"""The Based recall suite (SWDE, FDA, SQuAD completion): evaluation only.

Protocol of the Based evaluation harness (Arora et al. 2024, arXiv 2402.18668), as the reference restates it
(ced/eval/recall_based.py:1-60): the prompt is the item's text as given, greedy decoding of at most 48 new tokens, the
input left-truncated to its last `max_length - 48` tokens (a long document keeps its end, where the question is), the
generation cut at the first newline, and the metric "contains": 1 when the gold value is found in the generation by a
case-insensitive search, nothing else normalised. One labelled change kept from the reference: the generation is also
cut before the first end-of-document token (a fixed number of steps would otherwise run on into a "new document" that
can copy the gold); every record keeps the hit without that cut too.

Items live in `<task>.items.jsonl.gz` (one JSON object per line: id, text, value) with a manifest holding each set's
sha256; the sets are downloaded for scoring and never redistributed.
"""

from __future__ import annotations

import gzip
import hashlib
import json
import re
from dataclasses import dataclass
from pathlib import Path
from typing import Callable, Iterable, Sequence

TASKS = ("squad", "swde", "fda")
MAX_GEN_TOKS = 48
STOP = ("\n",)
MANIFEST_NAME = "manifest.json"


@dataclass
class Item:
    task: str
    id: str
    text: str
    value: str


def format_item(task: str, row: dict, index: int) -> Item:
    if task not in TASKS:
        raise ValueError(f"unknown task {task!r}: one of {TASKS}")
    return Item(task, str(row.get("doc_id", row.get("id", f"{index:05d}"))), row["text"], row["value"])


def item_sha256(it: Item) -> str:
    return hashlib.sha256(json.dumps([it.task, it.id, it.text, it.value], ensure_ascii=False).encode()).hexdigest()


def set_sha256(items: Sequence[Item]) -> str:
    return hashlib.sha256("\n".join(item_sha256(i) for i in items).encode()).hexdigest()


def write_items(path, items: Sequence[Item]) -> str:
    data = "".join(json.dumps({"id": i.id, "text": i.text, "value": i.value}, ensure_ascii=False) + "\n" for i in items).encode()
    with open(path, "wb") as f:
        with gzip.GzipFile(fileobj=f, mode="wb", mtime=0) as z:      # mtime 0: the same items give the same file
            z.write(data)
    return set_sha256(items)


def read_items(path, task: str) -> list[Item]:
    with gzip.open(path, "rt", encoding="utf-8") as f:
        return [format_item(task, json.loads(line), n) for n, line in enumerate(f) if line.strip()]


def write_set(directory, items_by_task: dict[str, Sequence[Item]]) -> dict:
    directory = Path(directory)
    directory.mkdir(parents=True, exist_ok=True)
    manifest = {t: {"n": len(items), "set_sha256": write_items(directory / f"{t}.items.jsonl.gz", items)} for t, items in items_by_task.items()}
    (directory / MANIFEST_NAME).write_text(json.dumps(manifest, indent=1))
    return manifest


def load_set(directory, task: str) -> list[Item]:
    """Items of a task, checked against the manifest's sha256."""
    directory = Path(directory)
    manifest = json.loads((directory / MANIFEST_NAME).read_text())
    items = read_items(directory / f"{task}.items.jsonl.gz", task)
    if set_sha256(items) != manifest[task]["set_sha256"] or len(items) != manifest[task]["n"]:
        raise ValueError(f"{task}: the items file does not match its manifest entry")
    return items


def contains_score(prediction: str, value: str) -> int:
    return int(bool(re.search(re.escape(value), prediction, re.IGNORECASE)))


def cut_at_stop(text: str, until: Sequence[str] = STOP) -> str:
    for s in until:
        text = text.split(s)[0]
    return text


def cut_at_eos(ids: Sequence[int], eos_id: int | None):
    ids = list(ids)
    if eos_id is not None and eos_id in ids:
        at = ids.index(eos_id)
        return ids[:at], at
    return ids, -1


def left_truncate(ids: Sequence[int], max_length: int, max_gen: int = MAX_GEN_TOKS):
    keep = max_length - max_gen
    ids = list(ids)
    return (ids[-keep:], True) if len(ids) > keep else (ids, False)


def score_items(model, items: Sequence[Item], encode: Callable[[str], list[int]], decode: Callable[[Sequence[int]], str], max_length: int,
                eos_id: int | None = None, batch: int = 8, autocast_dtype=None) -> list[dict]:
    """One record per item: hit, hit_no_eos_cut, eos_at, truncated, n_tokens, generation."""
    from .generate import generate_greedy_batched

    order = sorted(range(len(items)), key=lambda i: len(items[i].text))       # similar lengths share a batch (less padding)
    records: list[dict | None] = [None] * len(items)
    for lo in range(0, len(order), batch):
        idx = order[lo:lo + batch]
        prompts = [left_truncate(encode(items[i].text), max_length) for i in idx]
        gens = generate_greedy_batched(model, [p for p, _ in prompts], MAX_GEN_TOKS, autocast_dtype=autocast_dtype)
        for i, (p, cut), g in zip(idx, prompts, gens):
            kept, at = cut_at_eos(g, eos_id)
            text, text_all = cut_at_stop(decode(kept)), cut_at_stop(decode(g))
            records[i] = {"id": items[i].id, "task": items[i].task, "hit": contains_score(text, items[i].value),
                          "hit_no_eos_cut": contains_score(text_all, items[i].value), "eos_at": at, "truncated": cut, "n_tokens": len(p),
                          "generation": text}
    return records


def cell_key(task: str) -> str:
    return f"based|{task}|all|acc"


def values_json(run: str, records_by_task: dict[str, Sequence[dict]], code_sha: str = "local", exclude: Iterable[str] = ()) -> dict:
    skip = set(exclude)
    cells, n_items = {}, {}
    for task, recs in records_by_task.items():
        kept = [r for r in recs if f"{task}:{r['id']}" not in skip]
        if kept:
            cells[cell_key(task)] = sum(r["hit"] for r in kept) / len(kept)
            n_items[cell_key(task)] = len(kept)
    return {"run": run, "family": "based", "code_sha": code_sha, "cells": cells, "n_items": n_items, "excluded": sorted(skip)}
