#!/usr/bin/env python
"""Loss by token position inside the training length and copy loss on repeated random sequences, for a checkpoint
(reference: ced/eval/report_pcr.py, tools/build_report_pcr.py).

    python scripts/report_pcr.py --checkpoint RUN --set name=path.pt [--set ...] [--seq-len 4096] [--copy-lengths 64,256,1024]
                                 [--copy-items 16] [--out report.json]
"""

from __future__ import annotations

import argparse
import json
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from gdn_hybrid_architecture_ideas_b200.eval import report_pcr as rp, span_bpb  # noqa: E402
from gdn_hybrid_architecture_ideas_b200.train import checkpoint as ckpt  # noqa: E402


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__)
    ap.add_argument("--checkpoint", required=True)
    ap.add_argument("--set", action="append", default=[], metavar="NAME=PATH")
    ap.add_argument("--seq-len", type=int, default=0)
    ap.add_argument("--edges", default=",".join(map(str, rp.POS_EDGES)))
    ap.add_argument("--copy-lengths", default="64,256,1024")
    ap.add_argument("--copy-items", type=int, default=16)
    ap.add_argument("--batch-size", type=int, default=4)
    ap.add_argument("--device", default="cuda" if torch.cuda.is_available() else "cpu")
    ap.add_argument("--out")
    a = ap.parse_args(argv)
    model, cfg, step = ckpt.load_model(a.checkpoint, a.device)
    seq_len = a.seq_len or cfg.data.seq_len
    edges = tuple(e for e in (int(x) for x in a.edges.split(",")) if e < seq_len)
    ac = torch.bfloat16 if a.device.startswith("cuda") else None
    records = {}
    for item in a.set:
        name, path = item.split("=", 1)
        blob = torch.load(path, map_location="cpu", weights_only=False)
        docs = [span_bpb.TokenizedDoc(list(d["ids"]), list(d["byte_lens"]), d.get("scored")) for d in blob["docs"]]
        rows = span_bpb.build_eval_rows(docs, seq_len)
        sums = rp.bucket_sums(rp.position_ce(model, rows, a.batch_size, ac), rows, edges)
        records[name] = rp.set_record(sums)
        records[name]["doc"]["scored"]["bpb_se"] = rp.row_clustered_se(sums)
        print(f"{name}: bpb by context in document " + "  ".join(
            f"{b} {v:.3f}" for b, v in zip(rp.bucket_names(edges), records[name]["doc"]["scored"]["bpb"])))
    out = {"step": step, "edges": list(edges), "buckets": rp.bucket_names(edges), "sets": records}
    if len(records) > 1:
        out["all_sets"] = rp.all_sets(records)
    lengths = [n for n in (int(x) for x in a.copy_lengths.split(",") if x) if 3 * n <= seq_len]
    if lengths and a.copy_items:
        table = rp.copy_table(rp.score_copy_items(model, cfg.model.vocab_size, lengths, a.copy_items, batch_size=a.batch_size, autocast_dtype=ac))
        out["copy"], out["copy_gain"] = table, rp.copy_gain(table)
        for n, gain in out["copy_gain"].items():
            print(f"copy n={n}: {table['pcr_copy2'][n]['nats_after_first']:.3f} nats per token, {gain:.3f} below a fresh draw")
    if a.out:
        with open(a.out, "w") as f:
            json.dump(out, f, indent=1)
    return 0


if __name__ == "__main__":
    sys.exit(main())
