#!/usr/bin/env python
"""Score a checkpoint on the Based recall suite (SWDE, FDA, SQuAD completion) by greedy generation
(reference: scripts/recall_based_score.py).

    python scripts/recall_based_score.py --checkpoint RUN_DIR_OR_FILE --items DIR --tokenizer tokenizer.json|bytes --out OUT --run NAME \\
        [--tasks squad swde fda] [--max-length 8192] [--limit N] [--batch 8]

DIR holds `<task>.items.jsonl.gz` and `manifest.json` (eval.recall_based.write_set). Outputs OUT/NAME.values.json (cells
"based|<task>|all|acc") and OUT/NAME/<task>.items.jsonl.gz with one record per item.
"""

from __future__ import annotations

import argparse
import gzip
import json
import os
import sys
from pathlib import Path

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from gdn_hybrid_architecture_ideas_b200.data.tokenizers import open_tokenizer  # noqa: E402
from gdn_hybrid_architecture_ideas_b200.eval import recall_based as RB  # noqa: E402
from gdn_hybrid_architecture_ideas_b200.train import checkpoint as ckpt  # noqa: E402


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__)
    ap.add_argument("--checkpoint", required=True)
    ap.add_argument("--items", required=True)
    ap.add_argument("--tokenizer", required=True)
    ap.add_argument("--eos-token")
    ap.add_argument("--out", required=True)
    ap.add_argument("--run", required=True)
    ap.add_argument("--tasks", nargs="*", default=None)
    ap.add_argument("--max-length", type=int, default=0)
    ap.add_argument("--limit", type=int, default=0)
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--device", default="cuda" if torch.cuda.is_available() else "cpu")
    a = ap.parse_args(argv)
    tok = open_tokenizer(a.tokenizer, a.eos_token)
    model, cfg, step = ckpt.load_model(a.checkpoint, a.device)
    max_length = a.max_length or cfg.data.seq_len
    manifest = json.loads((Path(a.items) / RB.MANIFEST_NAME).read_text())
    tasks = a.tasks or [t for t in RB.TASKS if t in manifest]
    out = Path(a.out)
    (out / a.run).mkdir(parents=True, exist_ok=True)
    ac = torch.bfloat16 if a.device.startswith("cuda") else None
    by_task = {}
    for task in tasks:
        items = RB.load_set(a.items, task)
        if a.limit:
            items = items[:a.limit]
        recs = RB.score_items(model, items, tok.encode, tok.decode, max_length, tok.eos_id, a.batch, ac)
        by_task[task] = recs
        with gzip.open(out / a.run / f"{task}.items.jsonl.gz", "wt", encoding="utf-8") as f:
            for r in recs:
                f.write(json.dumps(r, ensure_ascii=False) + "\n")
        print(f"{task}: acc {sum(r['hit'] for r in recs) / max(len(recs), 1):.4f} over {len(recs)} items "
              f"({sum(r['truncated'] for r in recs)} truncated, {sum(r['hit_no_eos_cut'] for r in recs)} hits without the end-of-document cut)")
    (out / f"{a.run}.values.json").write_text(json.dumps(RB.values_json(a.run, by_task), indent=1))
    return 0


if __name__ == "__main__":
    sys.exit(main())
