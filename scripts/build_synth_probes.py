#!/usr/bin/env python
"""Build the probes on synthetic code-like material (`eval/probe_synth.py`: copy, line_edit, line_edit_foil, copy_span,
edit_old, transcode) and tokenize them.

    python scripts/build_synth_probes.py --out probes/ --tokenizer t64k=tokenizer.json [--tokenizer bytes=bytes] \\
        [--probes copy,line_edit,line_edit_foil,copy_span,edit_old,transcode] [--per-cell 20] [--distances 1024,4096,8192] \\
        [--file-lines 40,160,480] [--first-control ID] [--max-attempts 8]

Writes, in the layout of `scripts/build_text_probes.py`,
    <out>/text/<probe>.jsonl.gz      the items, one JSON per line (tokenizer-independent)
    <out>/<tok>/<probe>.pt           {"probes": [...]} in the stored form `scripts/eval_probes.py --set` scores
    <out>/<tok>/synth_manifest.json  counts, token lengths per cell, failed per-item checks, sha256 of the files
    <out>/synth_manifest.json        seed, probes, length measure, attempts used, sha256 of everything written

No documents are read: every file, log and record is synthetic. An item's length measure is the largest of its token
counts under the tokenizers given. Chat items are encoded piece by piece, control tokens at ids of their own from
--first-control upward (default: right after each tokenizer's vocabulary, the training shards' convention). An item whose
checks fail under some tokenizer (a token straddling the lead-in's end, an answer that occurs twice, a distance outside
[0.9 D, D]) is rebuilt with the next attempt, up to --max-attempts; what still fails is counted in the manifest and fails
the build unless --allow-misses. Reference: tools/build_probes_ext.py, tools/build_probes_copy.py, tools/build_probes_transcode.py.
"""

from __future__ import annotations

import argparse
import json
import os
import sys
from collections import defaultdict
from pathlib import Path

import torch

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from build_text_probes import gz_text_writer, sha256  # noqa: E402
from gdn_hybrid_architecture_ideas_b200.data.tokenizers import open_tokenizer  # noqa: E402
from gdn_hybrid_architecture_ideas_b200.eval import probe_synth as PS  # noqa: E402
from gdn_hybrid_architecture_ideas_b200.eval import probe_text as T  # noqa: E402


def encode(item, tok, first_control: int) -> dict:
    if isinstance(item, PS.ChatItem):
        return PS.encode_chat_item(item, tok.encode, PS.control_ids(first_control or tok.vocab_size))
    rec = T.encode_item(item, tok.encode)
    if item.probe == "copy":
        d, want = item.meta["distance"], item.cell["dist"]
        rec["checks"]["distance"] = PS.DIST_LO * want <= d <= want
        rec["checks"]["answer_once"] = item.context.count(item.answer) == 1
        rec["floor"] = item.meta["floor"]
        if item.meta["diff_chars"]:
            rec["diff_index"] = [len(tok.encode(item.answer[:c])) for c in item.meta["diff_chars"]]
    if item.probe in ("line_edit", "line_edit_foil"):
        rec.update(floor=item.meta["floor"], question=item.meta["question"], line=item.meta["line"], gold_line=item.meta["gold_line"])
    return rec


def rebuild(item, attempt: int, count, seed: int):
    """The same cell and index at another attempt."""
    c, i = item.cell, int(item.id.split("/")[-1]) if item.probe != "line_edit_foil" else None
    if item.probe == "copy":
        return PS.copy(c["len"], c["dist"], c["variant"], item.group["form"], i, count, attempt, seed)
    if item.probe == "copy_span":
        return PS.copy_span(c["type"], c["len"], c["dist"], c["src"], c["variant"], i, count, attempt, seed=seed)
    if item.probe == "edit_old":
        return PS.edit_old(c["lines"], c["file"], c["render"], i, attempt, seed)
    if item.probe == "transcode":
        return PS.transcode(c["dir"], c["lines"], item.group["kind"], i, attempt, seed=seed)
    return None      # line_edit rows have no per-tokenizer rule beyond the clean boundary of " <N>"


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--out", required=True)
    ap.add_argument("--tokenizer", action="append", required=True, metavar="NAME=PATH", help="`bytes` as the path for the byte tokenizer")
    ap.add_argument("--probes", default=",".join(PS.PROBES))
    ap.add_argument("--per-cell", type=int, default=20)
    ap.add_argument("--distances", default=",".join(map(str, PS.COPY_DISTANCES)))
    ap.add_argument("--file-lines", default=",".join(map(str, PS.FILE_LINES)), help="file lengths of the line_edit cells")
    ap.add_argument("--seed", type=int, default=T.SEED)
    ap.add_argument("--first-control", type=int, default=0)
    ap.add_argument("--max-attempts", type=int, default=8)
    ap.add_argument("--allow-misses", action="store_true")
    a = ap.parse_args(argv)
    toks = {}
    for spec in a.tokenizer:
        name, _, path = spec.partition("=")
        toks[name] = open_tokenizer(path or name)
    probes = a.probes.split(",")
    bad = [p for p in probes if p not in PS.PROBES]
    if bad:
        ap.error(f"unknown probes {bad}: of {PS.PROBES}")
    distances = tuple(int(x) for x in a.distances.split(","))
    count = lambda text: max(len(t.encode(text)) for t in toks.values())
    out = Path(a.out)
    (out / "text").mkdir(parents=True, exist_ok=True)
    files, summary, misses, retried = {}, {}, 0, 0
    for probe in probes:
        items = PS.build_cells(probe, a.per_cell, count, distances, a.seed, tuple(int(x) for x in a.file_lines.split(",")))
        recs = {name: [] for name in toks}
        for n, item in enumerate(items):
            for attempt in range(a.max_attempts):
                enc = {name: encode(item, tok, a.first_control) for name, tok in toks.items()}
                if all(all(r["checks"].values()) for r in enc.values()) or attempt + 1 == a.max_attempts:
                    break
                again = rebuild(item, attempt + 1, count, a.seed)
                if again is None:
                    break
                item, retried = again, retried + 1
            items[n] = item
            for name in toks:
                recs[name].append(enc[name])
        text_path = out / "text" / f"{probe}.jsonl.gz"
        with gz_text_writer(text_path) as f:
            for it in items:
                f.write(json.dumps(it.to_json(), ensure_ascii=False) + "\n")
        files[str(text_path.relative_to(out))] = sha256(text_path)
        summary[probe] = {"items": len(items)}
        for name, tok in toks.items():
            (out / name).mkdir(exist_ok=True)
            path = out / name / f"{probe}.pt"
            vocab = max(tok.vocab_size, (a.first_control or tok.vocab_size) + len(PS.CF.CONTROL_TOKENS))
            torch.save({"probes": recs[name], "vocab": vocab, "seed": a.seed, "tokenizer": getattr(tok, "name", name)}, path)
            files[str(path.relative_to(out))] = sha256(path)
            per_cell, failed = defaultdict(list), defaultdict(int)
            for r in recs[name]:
                per_cell[r["cell"]].append(r["length"])
                for check, ok in r["checks"].items():
                    failed[check] += 0 if ok else 1
            misses += sum(failed.values())
            summary[probe][name] = {"cells": {c: {"items": len(v), "min_tokens": min(v), "max_tokens": max(v)} for c, v in sorted(per_cell.items())},
                                    "failed_checks": dict(failed)}
    for name in toks:
        (out / name / "synth_manifest.json").write_text(json.dumps({p: summary[p][name] for p in probes} | {"sha256": {k: v for k, v in files.items() if k.startswith(name + "/")}}, indent=1))
    (out / "synth_manifest.json").write_text(json.dumps({"seed": a.seed, "probes": {p: summary[p]["items"] for p in probes}, "distances": distances,
                                                         "length_measure": f"max over tokenizers {sorted(toks)}", "retried": retried,
                                                         "failed_checks": misses, "sha256": files}, indent=1))
    print(json.dumps({"items": {p: summary[p]["items"] for p in probes}, "retried": retried, "failed_checks": misses}))
    return 1 if misses and not a.allow_misses else 0


if __name__ == "__main__":
    sys.exit(main())
