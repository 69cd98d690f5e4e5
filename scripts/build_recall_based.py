#!/usr/bin/env python
"""Build the Based recall suite's item files (SQuAD completion, SWDE, FDA) from raw files already on disk. EVALUATION ONLY.
The protocol is in `eval/recall_based.py` (reference: tools/data/build_recall_based.py; that tool also fetches the files at
pinned revisions, which needs a network: here the downloaded files are given).

    python scripts/build_recall_based.py --raw RAW --out ITEMS [--tasks squad,swde,fda] [--tokenizer tokenizer.json|bytes] [--texts]
        [--expect-sha256 squad=<sha256 of the raw file> ...]

RAW/<task>/ holds the task's rows as one file: *.parquet (needs pyarrow), *.jsonl or *.jsonl.gz, each row with the fields of the
public release ("doc_id", "text", "value"). A file's sha256 is recorded, and compared with --expect-sha256 when given (a
mismatch stops the build). SQuAD 2.0 is CC BY-SA 4.0; SWDE and FDA state no licence: the items are built for scoring and are
not to be redistributed (keep the raw files and the built items out of any repository).

Writes under --out:
    <task>.items.jsonl.gz            the items (raw text: the tokenizer is applied at scoring), a fixed gzip header
    manifest.json                    per task: item count and set sha256 (what `eval.recall_based.load_set` verifies), the raw file and its sha256
    recall_based.contamination.json  per set: item count and item-text hashes (hashes, no text)
    report.json                      counts, repeated ids / texts, and with --tokenizer the prompt token counts per task
    itemtexts/<task>.jsonl.gz        with --texts: {id, text, value} a line, for an n-gram contamination scan
"""

from __future__ import annotations

import argparse
import gzip
import hashlib
import json
import os
import statistics
import sys
from pathlib import Path

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from gdn_hybrid_architecture_ideas_b200.eval import recall_based as RB  # noqa: E402


def sha256_file(path: Path) -> str:
    h = hashlib.sha256()
    with open(path, "rb") as f:
        for block in iter(lambda: f.read(1 << 20), b""):
            h.update(block)
    return h.hexdigest()


def read_rows(path: Path) -> list[dict]:
    if path.suffix == ".parquet":
        import pyarrow.parquet as pq

        return pq.read_table(path).to_pylist()
    opener = gzip.open if path.name.endswith(".gz") else open
    with opener(path, "rt", encoding="utf-8") as f:
        return [json.loads(line) for line in f if line.strip()]


def raw_file(raw: Path, task: str) -> Path:
    found = sorted(p for p in (raw / task).glob("*") if p.suffix in (".parquet", ".jsonl") or p.name.endswith(".jsonl.gz"))
    if len(found) != 1:
        raise SystemExit(f"{raw / task}: expected exactly one raw file (*.parquet, *.jsonl, *.jsonl.gz), found {[p.name for p in found]}")
    return found[0]


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--raw", required=True)
    ap.add_argument("--out", required=True)
    ap.add_argument("--tasks", default=",".join(RB.TASKS))
    ap.add_argument("--tokenizer")
    ap.add_argument("--texts", action="store_true")
    ap.add_argument("--expect-sha256", action="append", default=[], metavar="TASK=SHA256")
    a = ap.parse_args(argv)
    tasks = a.tasks.split(",")
    expect = dict(x.split("=", 1) for x in a.expect_sha256)
    raw, out = Path(a.raw), Path(a.out)
    items_by_task, sources = {}, {}
    for task in tasks:
        path = raw_file(raw, task)
        digest = sha256_file(path)
        if task in expect and expect[task] != digest:
            raise SystemExit(f"{path}: sha256 {digest} is not the expected {expect[task]}")
        rows = read_rows(path)
        items_by_task[task] = [RB.format_item(task, r, i) for i, r in enumerate(rows)]
        sources[task] = {"file": path.name, "sha256": digest, "rows": len(rows)}
    manifest = RB.write_set(out, items_by_task)
    for task in tasks:
        manifest[task]["source"] = sources[task]
    (out / RB.MANIFEST_NAME).write_text(json.dumps(manifest, indent=1))
    contamination = {t: {"items": len(v), "source": sources[t], "item_text_sha256": [hashlib.sha256(i.text.encode("utf-8")).hexdigest() for i in v],
                         "note": "hashes only; the items are not redistributed"} for t, v in items_by_task.items()}
    (out / "recall_based.contamination.json").write_text(json.dumps(contamination, indent=1))
    report = {}
    tok = None
    if a.tokenizer:
        from gdn_hybrid_architecture_ideas_b200.data.tokenizers import open_tokenizer

        tok = open_tokenizer(a.tokenizer)
    for t, v in items_by_task.items():
        rec = {"items": len(v), "repeated_ids": len(v) - len({i.id for i in v}), "repeated_texts": len(v) - len({i.text for i in v}),
               "empty_values": sum(not i.value for i in v)}
        if tok is not None and v:
            lens = [len(tok.encode(i.text)) for i in v]
            rec["prompt_tokens"] = {"min": min(lens), "median": statistics.median(lens), "max": max(lens)}
        report[t] = rec
    (out / "report.json").write_text(json.dumps(report, indent=1))
    if a.texts:
        (out / "itemtexts").mkdir(exist_ok=True)
        for t, v in items_by_task.items():
            with open(out / "itemtexts" / f"{t}.jsonl.gz", "wb") as f, gzip.GzipFile(fileobj=f, mode="wb", mtime=0) as z:
                z.write("".join(json.dumps({"id": i.id, "text": i.text, "value": i.value}, ensure_ascii=False) + "\n" for i in v).encode())
    print(json.dumps({t: r["items"] for t, r in report.items()}))
    return 0


if __name__ == "__main__":
    sys.exit(main())
