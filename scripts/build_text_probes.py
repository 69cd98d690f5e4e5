#!/usr/bin/env python
"""Build text-level probe sets (`eval/probe_text.py`) from held-out documents and tokenize them.

    python scripts/build_text_probes.py --out probes/ --tokenizer t64k=tokenizer.json [--tokenizer bytes=bytes] \\
        --docs web.docs.jsonl.gz --docs general_web.docs.jsonl.gz [--probes uuid_needle,multikey,path_copy,depth,mf_chain,mf_concat] \\
        [--lengths 8192,16384] [--per-cell 20] [--needle-distances 2048:61440:2048 --distance-per-cell 40 --distance-keys 4]

Writes
    <out>/text/<probe>.jsonl.gz      the text items, one JSON per line (tokenizer-independent)
    <out>/<tok>/<probe>.pt           {"probes": [...]} in the stored form `scripts/eval_probes.py --set` scores
    <out>/<tok>/manifest.json        counts, token lengths per cell, failed per-item checks, sha256 of the files
    <out>/manifest.json              seed, probes, length measure, the document pool, sha256 of everything written

`--preset pcr`: the retrieval-inside-the-training-length set: uuid_needle, multikey and vt at 2,048 / 4,096 / 8,192 tokens,
plus the copy-loss sequences of `eval/report_pcr.py` (pcr_copy2, pcr_copy3, pcr_fresh: random token sequences repeated, so
they are written per tokenizer only) at --copy-lengths, --copy-per-length items each.

`--docs`: JSON lines {"id", "text"} (gzip or plain) of documents that are in no training shard. An item's length is the
largest of its token counts under the tokenizers given, so an item of nominal length T has at most T tokens under each.
Per-item checks under every tokenizer (counted in the manifest; the build fails on a miss unless --allow-misses): context
and answer tokenize at a clean boundary; a needle's or path's answer tokens occur once in the context; depth candidates
are single tokens; multi-fact pieces add up to the answer. Reference: tools/build_probes.py, tools/build_probes_multifact.py.
"""

from __future__ import annotations

import argparse
import gzip
import hashlib
import json
import os
import sys
from collections import defaultdict
from pathlib import Path

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from gdn_hybrid_architecture_ideas_b200.data.tokenizers import open_tokenizer  # noqa: E402
from gdn_hybrid_architecture_ideas_b200.eval import probe_text as T  # noqa: E402


def gz_text_writer(path: Path):
    """A gzip text stream whose bytes depend on the content alone (no file name, no modification time in the header)."""
    import io

    raw = open(path, "wb")
    return io.TextIOWrapper(gzip.GzipFile(filename="", mode="wb", fileobj=raw, mtime=0), encoding="utf-8")


def sha256(path: Path) -> str:
    h = hashlib.sha256()
    with open(path, "rb") as f:
        for block in iter(lambda: f.read(1 << 20), b""):
            h.update(block)
    return h.hexdigest()


def read_docs(paths) -> list[str]:
    docs = []
    for p in paths:
        opener = gzip.open if str(p).endswith(".gz") else open
        with opener(p, "rt", encoding="utf-8") as f:
            docs += [json.loads(line)["text"] for line in f if line.strip()]
    return docs


def parse_distances(spec: str) -> list[int]:
    if ":" in spec:
        a, b, c = (int(x) for x in spec.split(":"))
        return list(range(a, b + 1, c))
    return [int(x) for x in spec.split(",") if x]


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--out", required=True)
    ap.add_argument("--tokenizer", action="append", required=True, metavar="NAME=PATH", help="`bytes` as the path for the byte tokenizer")
    ap.add_argument("--docs", action="append", default=[])
    ap.add_argument("--probes", default=",".join(T.PROBES))
    ap.add_argument("--lengths", default=",".join(map(str, T.LENGTHS)))
    ap.add_argument("--per-cell", type=int, default=20)
    ap.add_argument("--seed", type=int, default=T.SEED)
    ap.add_argument("--needle-distances", default="")
    ap.add_argument("--distance-per-cell", type=int, default=40)
    ap.add_argument("--distance-keys", type=int, default=4)
    ap.add_argument("--distance-tol", type=int, default=64)
    ap.add_argument("--allow-misses", action="store_true")
    ap.add_argument("--preset", choices=["pcr"])
    ap.add_argument("--copy-lengths", default="64,256,1024")
    ap.add_argument("--copy-per-length", type=int, default=32)
    a = ap.parse_args(argv)
    if a.preset == "pcr":
        a.probes, a.lengths = "uuid_needle,multikey,vt", "2048,4096,8192"
    toks = {}
    for spec in a.tokenizer:
        name, _, path = spec.partition("=")
        toks[name] = open_tokenizer(path or name)
    probes = a.probes.split(",")
    bad = [p for p in probes if p not in T.PROBES]
    if bad:
        ap.error(f"unknown probes {bad}: of {T.PROBES}")
    lengths = tuple(int(x) for x in a.lengths.split(","))
    needs_docs = [p for p in probes if p not in ("path_copy", "depth")]
    pool = T.DocPool(read_docs(a.docs)) if needs_docs else None
    if needs_docs and not a.docs:
        ap.error(f"--docs is needed for {needs_docs}")
    count = lambda text: max(len(t.encode(text)) for t in toks.values())
    out = Path(a.out)
    (out / "text").mkdir(parents=True, exist_ok=True)
    files, summary, misses = {}, {}, 0
    for probe in probes:
        items = T.build_cells(probe, a.per_cell, pool, count, lengths, a.seed)
        if a.needle_distances and probe in ("uuid_needle", "multikey"):
            keys = 1 if probe == "uuid_needle" else a.distance_keys
            for length in lengths:
                for i in range(a.distance_per_cell):
                    for dist in parse_distances(a.needle_distances):
                        if dist + 512 <= (1 - T.LENGTH_SLACK) * length:
                            items.append(T.needle_at_distance(pool, count, length, dist, i, keys, a.distance_tol, a.seed))
        text_path = out / "text" / f"{probe}.jsonl.gz"
        with gz_text_writer(text_path) as f:
            for it in items:
                f.write(json.dumps(it.to_json(), ensure_ascii=False) + "\n")
        files[str(text_path.relative_to(out))] = sha256(text_path)
        summary[probe] = {"items": len(items)}
        for name, tok in toks.items():
            recs = [T.encode_item(it, tok.encode) for it in items]
            (out / name).mkdir(exist_ok=True)
            path = out / name / f"{probe}.pt"
            torch.save({"probes": recs, "vocab": tok.vocab_size, "seed": a.seed, "tokenizer": getattr(tok, "name", name)}, path)
            files[str(path.relative_to(out))] = sha256(path)
            per_cell, failed = defaultdict(list), defaultdict(int)
            for r in recs:
                per_cell[r["cell"]].append(r["length"])
                for check, ok in r["checks"].items():
                    failed[check] += 0 if ok else 1
            misses += sum(failed.values())
            summary[probe][name] = {"cells": {c: {"items": len(v), "min_tokens": min(v), "max_tokens": max(v)} for c, v in sorted(per_cell.items())},
                                    "failed_checks": dict(failed)}
    if a.preset == "pcr":
        from gdn_hybrid_architecture_ideas_b200.eval import report_pcr as PCR

        for name, tok in toks.items():
            allowed = PCR.allowed_ids(tok.vocab_size, [tok.eos_id] if getattr(tok, "eos_id", None) is not None else [])
            for variant in PCR.COPY_VARIANTS:
                recs = []
                for n in (int(x) for x in a.copy_lengths.split(",")):
                    for i in range(a.copy_per_length):
                        ids, first = PCR.copy_item(allowed, variant, n, i)
                        recs.append({"id": PCR.copy_item_id(variant, n, i), "kind": variant, "cell": f"n={n}", "group": "", "ids": ids.tolist(),
                                     "answer_start": int(first), "answer_len": len(ids) - int(first), "length": len(ids), "pieces": (), "checks": {}})
                (out / name).mkdir(exist_ok=True)
                path = out / name / f"{variant}.pt"
                torch.save({"probes": recs, "vocab": tok.vocab_size, "seed": PCR.COPY_SEED, "tokenizer": getattr(tok, "name", name)}, path)
                files[str(path.relative_to(out))] = sha256(path)
                summary.setdefault(variant, {"items": len(recs)})[name] = {"cells": {}, "failed_checks": {}}
        probes = probes + list(PCR.COPY_VARIANTS)
    for name in toks:
        (out / name / "manifest.json").write_text(json.dumps({p: summary[p][name] for p in probes} | {"sha256": {k: v for k, v in files.items() if k.startswith(name + "/")}}, indent=1))
    (out / "manifest.json").write_text(json.dumps({"seed": a.seed, "probes": {p: summary[p]["items"] for p in probes}, "lengths": lengths,
                                                   "length_measure": f"max over tokenizers {sorted(toks)}", "pool": pool.describe() if pool else None,
                                                   "failed_checks": misses, "sha256": files}, indent=1))
    print(json.dumps({"items": {p: summary[p]["items"] for p in probes}, "failed_checks": misses}))
    return 1 if misses and not a.allow_misses else 0


if __name__ == "__main__":
    sys.exit(main())
