#!/usr/bin/env python
"""Build the RULER subset's items once (`eval/recall_ruler.py`), so every checkpoint of a comparison generates from the
same stored prompts (reference: tools/build_recall_ruler.py).

    python scripts/build_recall_ruler.py --out items/ --tokenizer tokenizer.json|bytes --docs web.docs.jsonl.gz [--docs ...] \\
        [--tasks ...] [--lengths 2048 4096 8192] [--per-cell 500]

CPU only. Reads held-out documents (JSON lines {"id", "text"}, gzip or plain; never part of a training shard) for the
open-haystack tasks and writes under --out:
    items/<task>.jsonl.gz          one JSON per item (id, task, length, index, prompt, refs, gen_tokens, tokens, meta), by length then index
    manifest.json                  seed, counts and token lengths per cell, items that found no fit, sha256 of every file, the pool, the tokenizer
    haystack-docs-used.json        ids of the documents the open-haystack items were cut from, per task and in all
    item-hashes.json               {"<item id>": sha256 of the prompt}: what a contamination check of training data compares against
Deterministic: the same inputs give the same files. An item of an index below the per-cell count is the same whatever the
count, so a build with 500 items a cell holds the build with 250 as its first 250 indices. A build in which an item's token
count under the tokenizer differs from the builder's own exits 1 after writing the manifest.
Score with `scripts/recall_ruler_score.py --items <out>`.
"""

from __future__ import annotations

import argparse
import gzip
import hashlib
import json
import os
import sys
from collections import defaultdict
from dataclasses import asdict
from pathlib import Path

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from gdn_hybrid_architecture_ideas_b200.data.tokenizers import open_tokenizer, tokenizer_sha256  # noqa: E402
from gdn_hybrid_architecture_ideas_b200.eval import recall_ruler as RR  # noqa: E402


def gz_text_writer(path: Path):
    """A gzip text stream whose bytes depend on the content alone (no file name, no modification time in the header)."""
    import io

    raw = open(path, "wb")
    return io.TextIOWrapper(gzip.GzipFile(filename="", mode="wb", fileobj=raw, mtime=0), encoding="utf-8")


def sha256_file(path: Path) -> str:
    h = hashlib.sha256()
    with open(path, "rb") as f:
        for block in iter(lambda: f.read(1 << 20), b""):
            h.update(block)
    return h.hexdigest()


def read_docs(paths) -> list[dict]:
    docs = []
    for p in paths:
        opener = gzip.open if str(p).endswith(".gz") else open
        with opener(p, "rt", encoding="utf-8") as f:
            for n, line in enumerate(f):
                if line.strip():
                    d = json.loads(line)
                    docs.append({"id": str(d.get("id", f"{Path(p).name}:{n}")), "text": d["text"]})
    return docs


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--out", required=True)
    ap.add_argument("--tokenizer", required=True)
    ap.add_argument("--eos-token")
    ap.add_argument("--docs", action="append", default=[])
    ap.add_argument("--tasks", nargs="*", default=None)
    ap.add_argument("--lengths", nargs="*", type=int, default=list(RR.LENGTHS))
    ap.add_argument("--per-cell", type=int, default=500)
    a = ap.parse_args(argv)
    tok = open_tokenizer(a.tokenizer, a.eos_token)
    docs = read_docs(a.docs)
    pool = [d["text"] for d in docs] or None
    tasks = a.tasks or [t for t in RR.TASKS if pool or RR.SPEC[t]["haystack"] != "open"]
    count = lambda text: len(tok.encode(text))
    out = Path(a.out)
    (out / "items").mkdir(parents=True, exist_ok=True)
    files, cells, no_fit, hashes, mismatches = {}, {}, [], {}, []
    used = defaultdict(set)
    for task in tasks:
        path = out / "items" / f"{task}.jsonl.gz"
        with gz_text_writer(path) as f:
            for length in a.lengths:
                lens = []
                for i in range(a.per_cell):
                    try:
                        it = RR.make_item(task, length, i, count, pool)
                    except RR.NoFitError as e:
                        no_fit.append({"task": task, "length": length, "index": i, "why": str(e)})
                        continue
                    true = count(it.prompt) + it.gen_tokens
                    if it.tokens and it.tokens != true:
                        mismatches.append({"id": it.id, "builder": it.tokens, "tokenizer": true})
                    lens.append(true)
                    hashes[it.id] = hashlib.sha256(it.prompt.encode("utf-8")).hexdigest()
                    if RR.SPEC[task]["haystack"] == "open":       # which pool documents the haystack's first `units` words came from
                        order = RR.rng_for(task, length, i, 2).permutation(len(docs))
                        left = int(it.meta["units"])
                        for j in order:
                            if left <= 0:
                                break
                            used[task].add(docs[int(j)]["id"])
                            left -= len(docs[int(j)]["text"].split())
                    f.write(json.dumps({"id": it.id, **asdict(it)}, ensure_ascii=False) + "\n")
                cells[f"{task}|{length}"] = {"items": len(lens), "min_tokens": min(lens, default=0), "max_tokens": max(lens, default=0)}
        files[str(path.relative_to(out))] = sha256_file(path)
    side = {"haystack-docs-used.json": {"per_task": {t: sorted(v) for t, v in used.items()}, "all": sorted(set().union(*used.values())) if used else []},
            "item-hashes.json": hashes}
    for name, blob in side.items():
        (out / name).write_text(json.dumps(blob, indent=1, sort_keys=True))
        files[name] = sha256_file(out / name)
    manifest = {"seed": RR.BASE_SEED, "tasks": tasks, "lengths": a.lengths, "per_cell": a.per_cell, "cells": cells, "no_fit": no_fit,
                "token_count_mismatches": mismatches, "sha256": files,
                "pool": {"documents": len(docs), "files": {str(p): sha256_file(Path(p)) for p in a.docs}},
                "tokenizer": {"name": getattr(tok, "name", a.tokenizer), "vocab_size": tok.vocab_size,
                              "sha256": tokenizer_sha256(a.tokenizer) if a.tokenizer != "bytes" else None}}
    (out / "manifest.json").write_text(json.dumps(manifest, indent=1))
    print(json.dumps({"items": sum(c["items"] for c in cells.values()), "no_fit": len(no_fit), "token_count_mismatches": len(mismatches)}))
    return 1 if mismatches else 0


if __name__ == "__main__":
    sys.exit(main())
