#!/usr/bin/env python
"""Synthetic recall probes (needle, multikey, copy, two-hop, path copy, multi-fact chain / concat, transcode) on a
checkpoint, teacher-forced
(reference: scripts/eval_probes.py).

    python scripts/eval_probes.py --checkpoint RUN --lengths 512,2048,8192 --per-kind 32 [--out probes.json]
"""

from __future__ import annotations

import argparse
import json
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from gdn_hybrid_architecture_ideas_b200.eval import probes  # noqa: E402
from gdn_hybrid_architecture_ideas_b200.train import checkpoint as ckpt  # noqa: E402


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__)
    ap.add_argument("--checkpoint", required=True)
    ap.add_argument("--lengths", default="512,2048")
    ap.add_argument("--per-kind", type=int, default=16)
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--batch-size", type=int, default=4)
    ap.add_argument("--device", default="cuda" if torch.cuda.is_available() else "cpu")
    ap.add_argument("--set", help="a stored probe set (scripts/build_probes.py) in place of probes built on the fly")
    ap.add_argument("--keep-items", action="store_true", help="with --set: the output also lists every item's id and exact-match score")
    ap.add_argument("--out")
    a = ap.parse_args(argv)
    model, cfg, step = ckpt.load_model(a.checkpoint, a.device)
    ac = torch.bfloat16 if a.device.startswith("cuda") else None
    table, item_records = {}, []
    stored = stored_ids = stored_recs = None
    if a.set:
        blob = torch.load(a.set, map_location="cpu", weights_only=False)
        if blob["vocab"] > cfg.model.vocab_size:
            ap.error(f"the set was built for a vocabulary of {blob['vocab']}, the model has {cfg.model.vocab_size}")
        stored, stored_ids, stored_recs = {}, {}, {}
        for p in blob["probes"]:
            stored_ids.setdefault((p.get("cell", p["length"]), p["kind"]), []).append(p.get("id"))
            stored_recs.setdefault((p.get("cell", p["length"]), p["kind"]), []).append(p)
            # token-id sets are keyed by their nominal length; text-level sets (scripts/build_text_probes.py) by their cell
            stored.setdefault((p.get("cell", p["length"]), p["kind"]), []).append(
                probes.Probe(p["kind"], p["ids"], p["answer_start"], p["answer_len"], tuple(map(tuple, p.get("pieces", ()))), p.get("group", ""),
                             tuple(map(tuple, p.get("candidates", ()))), p.get("gold", -1)))
    cells = sorted(stored, key=lambda c: (str(type(c[0])), c)) if stored is not None else [(int(x), k) for x in a.lengths.split(",") for k in probes.PROBE_KINDS]
    for length, kind in cells:
        ps = stored[(length, kind)] if stored is not None else [
            probes.build_probe(kind, cfg.model.vocab_size, length, a.seed, i) for i in range(a.per_kind)]
        synth = stored_recs is not None and any("floor" in p or "question" in p for p in stored_recs[(length, kind)])
        r = probes.score_probes(model, ps, a.batch_size, ac, keep_tokens=synth)
        cell = {"exact": r["exact"], "ce": r["ce"], "n": r["n"]}
        if synth:        # the probes on synthetic material (scripts/build_synth_probes.py): floors, near-duplicate tokens, line choices
            from gdn_hybrid_architecture_ideas_b200.eval.probe_synth import cell_extras

            cell.update(cell_extras(stored_recs[(length, kind)], r["items"]))
        if stored_ids is not None and a.keep_items:
            item_records += [{"id": i, "kind": kind, "exact": bool(it["exact"]), "ce": it["ce"]} for i, it in zip(stored_ids[(length, kind)], r["items"])]
        groups = sorted({it["group"] for it in r["items"] if "group" in it})
        for gname in groups:        # multi-fact layouts, transcode directions
            own = [it for it in r["items"] if it.get("group") == gname]
            cell[gname] = {"exact": sum(it["exact"] for it in own) / len(own), "n": len(own)}
        if kind.startswith("mf_"):
            for key in ("fact_acc", "first_ok", "nats", "exact_all"):
                cell[key] = sum(float(it[key]) for it in r["items"]) / len(r["items"])
        if any("choice_ok" in it for it in r["items"]):
            cell["choice_acc"] = sum(float(it.get("choice_ok", 0.0)) for it in r["items"]) / len(r["items"])
        if kind == "transcode" and not synth:       # the token-id transcode probe; the synthetic-material one stores its floor per item
            floors = [probes.copy_floor(q) for q in ps]
            cell["copy_floor"] = {k: sum(float(f[k]) for f in floors) / len(floors) for k in ("token_acc", "lcs_share")}
        table[f"{kind}@{length}"] = cell
        print(f"{kind:11s} {('length ' + str(length)) if isinstance(length, int) else length}: exact {r['exact']:.3f}  ce {r['ce']:.3f}")
    if a.out:
        with open(a.out, "w") as f:
            json.dump({"step": step, "probes": table, **({"items": item_records} if a.keep_items else {})}, f, indent=1)
    return 0


if __name__ == "__main__":
    sys.exit(main())
