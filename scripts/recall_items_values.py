#!/usr/bin/env python
"""The values file of the larger multi-key item sets, in the common format of the recall builds (family "items"), from
the per-group outputs of `scripts/eval_probes.py --set <items>/groups/<group>/<tok>/multikey.pt --keep-items --out DIR/<group>.json`
(reference: tools/analysis/recall_items_values.py).

    python scripts/recall_items_values.py run   --plan plan.json --run NAME --probes-dir DIR --out NAME.values.json [--exclude-file FILE] [--allow-partial] [--first-block-only]
    python scripts/recall_items_values.py brief --values NAME.values.json

run    reads <group>.json for every group of the plan and writes {"run", "family": "items", "cells": {"items|multikey_n<k>|<length>|exact":
       accuracy}, "n_items", "excluded"} and beside it <out stem>.detail.json (per cell: the first block of old items and the
       new block apart with their binomial standard errors, items missing). --exclude-file: a JSON list of item ids left out of
       every cell (an id that names no item of the plan is an error). --first-block-only: the cells over the old items only.
brief  one line per cell: accuracy, items, binomial standard error.
Exit: 0 written; 2 bad input; 3 a group file missing, an item of the plan not scored (without --allow-partial), or an exclusion
that names no item of the plan.
"""

from __future__ import annotations

import argparse
import json
import os
import sys
from pathlib import Path

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from gdn_hybrid_architecture_ideas_b200.eval import recall_items as RI  # noqa: E402


def cmd_run(a) -> int:
    plan = RI.load_plan(a.plan)
    results = {}
    for g in plan["groups"]:
        path = Path(a.probes_dir) / f"{g['name']}.json"
        if not path.is_file():
            print(f"missing group file {path}", file=sys.stderr)
            if not a.allow_partial:
                return 3
            continue
        blob = json.loads(path.read_text())
        if "items" not in blob:
            print(f"{path} holds no per-item records (score with --keep-items)", file=sys.stderr)
            return 2
        for it in blob["items"]:
            results[it["id"]] = it
    plan_ids = {RI.item_id(RI.cell_of_key(c["key"]), i) for c in plan["cells"] for i in range(c["n"])}
    exclude = set(json.loads(Path(a.exclude_file).read_text())) if a.exclude_file else set()
    exclude = {x.split(":", 1)[-1] for x in exclude}                       # "<probe>:<id>" and the bare id name the same item
    stray = sorted(exclude - plan_ids)
    if stray:
        print(f"exclusions that name no item of the plan: {stray[:5]}", file=sys.stderr)
        return 3
    use = dict(plan)
    if a.first_block_only:
        use = dict(plan, cells=[dict(c, n=c["n_old"]) for c in plan["cells"] if c["n_old"]])
    if a.allow_partial:
        use = dict(use, cells=[dict(c, n=max((i + 1 for i in range(c["n"]) if RI.item_id(RI.cell_of_key(c["key"]), i) in results), default=0)) for c in use["cells"]])
    try:
        values = RI.values_for_run(a.run, use, list(results.values()), exclude)
    except ValueError as e:
        print(str(e), file=sys.stderr)
        return 3
    detail = {}
    for c in plan["cells"]:
        cell = RI.cell_of_key(c["key"])
        block = lambda lo, hi: [results[i]["exact"] for i in (RI.item_id(cell, k) for k in range(lo, hi)) if i in results and i not in exclude]
        old, new = block(0, c["n_old"]), block(c["n_old"], c["n"])
        part = lambda xs: {"n": len(xs), "exact": (sum(xs) / len(xs) if xs else None), "se": (RI.binomial_se(sum(xs) / len(xs), len(xs)) if xs else None)}
        missing = [i for i in (RI.item_id(cell, k) for k in range(c["n"])) if i not in results]
        detail[c["key"]] = {"first_block": part(old), "new_block": part(new), "missing": len(missing)}
    out = Path(a.out)
    out.write_text(json.dumps(values, indent=1))
    out.with_name(out.stem.replace(".values", "") + ".detail.json").write_text(json.dumps(detail, indent=1))
    return 0


def cmd_brief(a) -> int:
    v = json.loads(Path(a.values).read_text())
    for name in sorted(v["cells"]):
        p, n = v["cells"][name], v["n_items"][name]
        print(f"{name}: {'n/a' if p is None else f'{p:.4f}'}  n={n}  se={'n/a' if p is None or not n else f'{RI.binomial_se(p, n):.4f}'}")
    return 0


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    sub = ap.add_subparsers(dest="cmd", required=True)
    p = sub.add_parser("run")
    p.add_argument("--plan", required=True)
    p.add_argument("--run", required=True)
    p.add_argument("--probes-dir", required=True)
    p.add_argument("--out", required=True)
    p.add_argument("--exclude-file")
    p.add_argument("--allow-partial", action="store_true")
    p.add_argument("--first-block-only", action="store_true")
    p = sub.add_parser("brief")
    p.add_argument("--values", required=True)
    a = ap.parse_args(argv)
    return {"run": cmd_run, "brief": cmd_brief}[a.cmd](a)


if __name__ == "__main__":
    sys.exit(main())
