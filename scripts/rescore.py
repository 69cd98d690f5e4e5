#!/usr/bin/env python
"""Bits per byte of a checkpoint on eval sets (reference: scripts/rescore.py).

    python scripts/rescore.py --checkpoint RUN_DIR_OR_FILE --set name=path.pt [--set ...] [--seq-len 4096] [--out scores.json]

An eval set file holds {"docs": [{"ids": [...], "byte_lens": [...], "scored": [...] or None}, ...]}.
"""

from __future__ import annotations

import argparse
import json
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from gdn_hybrid_architecture_ideas_b200.eval import span_bpb  # noqa: E402
from gdn_hybrid_architecture_ideas_b200.train import checkpoint as ckpt  # noqa: E402


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__)
    ap.add_argument("--checkpoint", required=True)
    ap.add_argument("--set", action="append", default=[], metavar="NAME=PATH")
    ap.add_argument("--seq-len", type=int, default=0)
    ap.add_argument("--batch-size", type=int, default=4)
    ap.add_argument("--device", default="cuda" if torch.cuda.is_available() else "cpu")
    ap.add_argument("--packing", choices=["documents", "stream"], default="documents",
                    help="documents: whole documents per row, longer ones skipped; stream: documents end to end, cut at the row length, nothing skipped")
    ap.add_argument("--out")
    a = ap.parse_args(argv)
    model, cfg, step = ckpt.load_model(a.checkpoint, a.device)
    seq_len = a.seq_len or cfg.data.seq_len
    ac = torch.bfloat16 if a.device.startswith("cuda") else None
    scores = {}
    for item in a.set:
        name, path = item.split("=", 1)
        blob = torch.load(path, map_location="cpu", weights_only=False)
        if blob["docs"] and "assistant" in blob["docs"][0]:     # chat documents: the assistant's tokens are scored, token classes kept apart
            docs = [span_bpb.RoleDoc(list(d["ids"]), list(d["byte_lens"]), None, d.get("name", ""), assistant=list(d["assistant"]),
                                     token_class=(list(d["token_class"]) if d.get("token_class") is not None else None)) for d in blob["docs"]]
            rows = span_bpb.build_role_rows(docs, seq_len, whole=a.packing == "documents")
        else:
            docs = [span_bpb.TokenizedDoc(d["ids"], d["byte_lens"], d.get("scored")) for d in blob["docs"]]
            rows = span_bpb.build_eval_rows(docs, seq_len) if a.packing == "documents" else span_bpb.build_stream_rows(docs, seq_len)
        if blob.get("special_ids") is not None:
            rows.special_ids = torch.as_tensor(blob["special_ids"], dtype=torch.long)
        if blob.get("doc_group") is not None:
            rows.doc_group = torch.as_tensor(blob["doc_group"], dtype=torch.long)
        ev = span_bpb.evaluate(model, rows, a.batch_size, autocast_dtype=ac)
        scores[name] = {"bpb": ev.bpb, "bpb_se": span_bpb.bpb_se(ev, "doc" if a.packing == "documents" else "cluster"), "ce": ev.ce, "docs": len(docs),
                        "skipped": len(rows.skipped), "rows": len(rows), "packing": a.packing, "rows_fingerprint": rows.fingerprint()}
        if ev.row_special_bytes is not None:
            scores[name]["bpb_without_special_bytes"] = ev.bpb_without_special_bytes()
        if ev.class_nats is not None:
            scores[name]["classes"] = ev.class_bpb()
        print(f"{name}: bpb {ev.bpb:.4f} +- {scores[name]['bpb_se']:.4f} ({len(docs)} documents)")
    if a.out:
        with open(a.out, "w") as f:
            json.dump({"step": step, "scores": scores}, f, indent=1)
    return 0


if __name__ == "__main__":
    sys.exit(main())
