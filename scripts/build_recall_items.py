#!/usr/bin/env python
"""Build the larger multi-key item sets of a retrieval rerun and cut them into the plan's scoring groups
(`eval/recall_items.py`; reference: tools/build_recall_items.py).

    python scripts/build_recall_items.py plan  --out plan.json --n 400 [--n-old 100] [--n-keys 4,16] [--lengths 8192,16384] [--budget-s 3000]
    python scripts/build_recall_items.py build --plan plan.json --out items/ --tokenizer t64k=tokenizer.json --docs web.docs.jsonl.gz [--docs ...]
    python scripts/build_recall_items.py split --plan plan.json --out items/
    python scripts/build_recall_items.py check-first-block --old OLD.pt --new NEW.pt

plan   every cell (multikey, n keys, length) gets --n items, of which the first --n-old are the ones already scored; the work is
       cut into groups of at most --budget-s modelled seconds (the dearest cells first). Deterministic.
build  one raw build with the text-probe builder (`scripts/build_text_probes.py --probes multikey`), per cell the plan's largest n:
       <out>/raw/<tok>/multikey.pt. An item is a pure function of (seed, cell, index) and the pool, so the old items are the first
       n_old of a cell; `check-first-block` verifies that against an older file instead of trusting it (same ids, same token ids;
       exit 4 on a difference).
split  <out>/groups/<group>/<tok>/multikey.pt for every group of the plan, each a stored set `scripts/eval_probes.py --set` scores.
"""

from __future__ import annotations

import argparse
import json
import os
import re
import sys
from pathlib import Path

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))

from gdn_hybrid_architecture_ideas_b200.eval import recall_items as RI  # noqa: E402

EX_CHECK = 4
_ID = re.compile(r"^multikey/len=(\d+)/n=(\d+)/(\d+)$")


def cell_key_of(item_id: str) -> tuple[str, int]:
    m = _ID.match(item_id)
    if not m:
        raise ValueError(f"not a multi-key item id: {item_id!r}")
    return RI.Cell("multikey", int(m.group(2)), int(m.group(1))).key, int(m.group(3))


def cmd_plan(a) -> int:
    cells = RI.cells_of("multikey", tuple(int(x) for x in a.n_keys.split(",")), tuple(int(x) for x in a.lengths.split(",")))
    plan = RI.make_plan({c.key: a.n for c in cells}, {c.key: a.n_old for c in cells} if a.n_old else None,
                        rule=f"{a.n} items per cell, the first {a.n_old} already scored", budget_s=a.budget_s)
    RI.validate_plan(plan)
    Path(a.out).write_text(json.dumps(plan, indent=1))
    print(json.dumps(plan["total"]))
    return 0


def cmd_build(a) -> int:
    import build_text_probes

    plan = RI.load_plan(a.plan)
    lengths = sorted({c["length"] for c in plan["cells"]})
    counts = sorted({c["n_keys"] for c in plan["cells"]})
    from gdn_hybrid_architecture_ideas_b200.eval import probe_text as T

    T.MULTIKEY_COUNTS = tuple(counts)          # the plan's key counts are the cells of this build
    argv = ["--out", str(Path(a.out) / "raw"), "--probes", "multikey", "--lengths", ",".join(map(str, lengths)),
            "--per-cell", str(max(c["n"] for c in plan["cells"]))]
    for t in a.tokenizer:
        argv += ["--tokenizer", t]
    for d in a.docs:
        argv += ["--docs", d]
    return build_text_probes.main(argv)


def cmd_split(a) -> int:
    plan = RI.load_plan(a.plan)
    raw = Path(a.out) / "raw"
    written = 0
    for tok_dir in sorted(p for p in raw.iterdir() if (p / "multikey.pt").is_file()):
        blob = torch.load(tok_dir / "multikey.pt", map_location="cpu", weights_only=False)
        by_cell: dict[str, dict[int, dict]] = {}
        for p in blob["probes"]:
            key, index = cell_key_of(p["id"])
            by_cell.setdefault(key, {})[index] = p
        for g in plan["groups"]:
            items = []
            for part in g["parts"]:
                have = by_cell.get(part["cell"], {})
                missing = [i for i in range(part["start"], part["stop"]) if i not in have]
                if missing:
                    raise SystemExit(f"group {g['name']}: cell {part['cell']} lacks items {missing[:5]}... in {tok_dir / 'multikey.pt'}")
                items += [have[i] for i in range(part["start"], part["stop"])]
            dest = Path(a.out) / "groups" / g["name"] / tok_dir.name
            dest.mkdir(parents=True, exist_ok=True)
            torch.save({**{k: v for k, v in blob.items() if k != "probes"}, "probes": items, "group": g["name"]}, dest / "multikey.pt")
            written += len(items)
    print(json.dumps({"groups": len(plan["groups"]), "items_written": written}))
    return 0


def cmd_check(a) -> int:
    old = {p["id"]: p for p in torch.load(a.old, map_location="cpu", weights_only=False)["probes"]}
    new = {p["id"]: p for p in torch.load(a.new, map_location="cpu", weights_only=False)["probes"]}
    missing = sorted(set(old) - set(new))
    changed = sorted(i for i in set(old) & set(new) if list(old[i]["ids"]) != list(new[i]["ids"]) or old[i]["answer_start"] != new[i]["answer_start"])
    print(json.dumps({"old_items": len(old), "missing_in_new": len(missing), "changed": len(changed), "first": (missing + changed)[:5]}))
    return EX_CHECK if missing or changed else 0


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    sub = ap.add_subparsers(dest="cmd", required=True)
    p = sub.add_parser("plan")
    p.add_argument("--out", required=True)
    p.add_argument("--n", type=int, required=True)
    p.add_argument("--n-old", type=int, default=0)
    p.add_argument("--n-keys", default="4,16")
    p.add_argument("--lengths", default="8192,16384,32768,65536")
    p.add_argument("--budget-s", type=float, default=RI.GROUP_BUDGET_S)
    p = sub.add_parser("build")
    p.add_argument("--plan", required=True)
    p.add_argument("--out", required=True)
    p.add_argument("--tokenizer", action="append", required=True)
    p.add_argument("--docs", action="append", default=[])
    p = sub.add_parser("split")
    p.add_argument("--plan", required=True)
    p.add_argument("--out", required=True)
    p = sub.add_parser("check-first-block")
    p.add_argument("--old", required=True)
    p.add_argument("--new", required=True)
    a = ap.parse_args(argv)
    return {"plan": cmd_plan, "build": cmd_build, "split": cmd_split, "check-first-block": cmd_check}[a.cmd](a)


if __name__ == "__main__":
    sys.exit(main())
