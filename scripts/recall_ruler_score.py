#!/usr/bin/env python
"""Score a checkpoint on the RULER subset by greedy generation (reference: scripts/recall_ruler_score.py).

    python scripts/recall_ruler_score.py --checkpoint RUN_DIR_OR_FILE --tokenizer tokenizer.json|bytes --out OUT --run NAME \\
        [--pool docs.jsonl | --items BUILD_DIR] [--tasks ...] [--lengths 2048 4096 8192] [--n-per-cell 100] [--batch 8]

--pool: held-out documents for the open-haystack tasks, one JSON object with a "text" field per line; without it only the
needle- and noise-haystack tasks run. Items are generated on the fly (a pure function of task, length, index and pool).
A row stops at the end-of-document token or once all its references are in its text. Outputs: OUT/NAME.items.jsonl (one
record per item; a rerun skips the ids it already holds) and OUT/NAME.values.json (cells "ruler|task|length|metric").
"""

from __future__ import annotations

import argparse
import json
import os
import sys
from pathlib import Path

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from gdn_hybrid_architecture_ideas_b200.data.tokenizers import open_tokenizer  # noqa: E402
from gdn_hybrid_architecture_ideas_b200.eval import recall_ruler as RR  # noqa: E402
from gdn_hybrid_architecture_ideas_b200.eval.generate import generate_greedy_batched  # noqa: E402
from gdn_hybrid_architecture_ideas_b200.train import checkpoint as ckpt  # noqa: E402


def stored_items(directory: Path, task: str) -> dict:
    """{(length, index): RulerItem} of a task from a build of scripts/build_recall_ruler.py."""
    import gzip

    path = Path(directory) / "items" / f"{task}.jsonl.gz"
    if not path.is_file():
        raise FileNotFoundError(f"--items: no {path}")
    out = {}
    with gzip.open(path, "rt", encoding="utf-8") as f:
        for line in f:
            d = json.loads(line)
            d.pop("id", None)
            it = RR.RulerItem(**d)
            out[(it.length, it.index)] = it
    return out


def score(model, tok, tasks, lengths, n_per_cell, batch, pool, out_dir: Path, run: str, autocast=None, log=print, items_dir=None) -> dict:
    out_dir.mkdir(parents=True, exist_ok=True)
    items_path = out_dir / f"{run}.items.jsonl"
    have = {}
    if items_path.exists():
        for line in items_path.read_text().splitlines():
            r = json.loads(line)
            have[r["id"]] = r
    count = lambda text: len(tok.encode(text))
    with items_path.open("a") as sink:
        for task in tasks:
            stored = stored_items(items_dir, task) if items_dir else None
            for length in lengths:
                todo = []
                for i in range(n_per_cell):
                    if stored is not None:
                        it = stored.get((length, i))
                        if it is None:
                            continue
                    else:
                        try:
                            it = RR.make_item(task, length, i, count, pool)
                        except RR.NoFitError as e:
                            log(f"{task} len={length} #{i}: {e}")
                            continue
                    if it.id not in have:
                        todo.append(it)
                for lo in range(0, len(todo), batch):
                    group = todo[lo:lo + batch]
                    refs = [[tok.encode(" " + r) for r in it.refs] for it in group]
                    def done(b, seq, group=group):
                        return RR.recall(tok.decode(seq), group[b].refs) == 1.0
                    gens = generate_greedy_batched(model, [tok.encode(it.prompt) for it in group], group[0].gen_tokens, is_done=done,
                                                   eos_id=tok.eos_id, autocast_dtype=autocast)
                    for it, g in zip(group, gens):
                        pred = tok.decode(g)
                        rec = {"id": it.id, "task": it.task, "length": it.length, "tokens": it.tokens, "pred": pred, "ids": g,
                               "recall": RR.recall(pred, it.refs), "all_found": RR.all_found(pred, it.refs)}
                        have[it.id] = rec
                        sink.write(json.dumps(rec) + "\n")
                    sink.flush()
                    del refs
                log(f"{task} len={length}: {sum(1 for r in have.values() if r['task'] == task and r['length'] == length)} items")
    values = RR.values_file(run, list(have.values()))
    (out_dir / f"{run}.values.json").write_text(json.dumps(values, indent=1))
    return values


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__)
    ap.add_argument("--checkpoint", required=True)
    ap.add_argument("--tokenizer", required=True)
    ap.add_argument("--eos-token")
    ap.add_argument("--out", required=True)
    ap.add_argument("--run", required=True)
    ap.add_argument("--pool")
    ap.add_argument("--items", help="a build of scripts/build_recall_ruler.py: its stored items are scored instead of items generated on the fly")
    ap.add_argument("--tasks", nargs="*", default=None)
    ap.add_argument("--lengths", nargs="*", type=int, default=list(RR.LENGTHS))
    ap.add_argument("--n-per-cell", type=int, default=100)
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--device", default="cuda" if torch.cuda.is_available() else "cpu")
    a = ap.parse_args(argv)
    tok = open_tokenizer(a.tokenizer, a.eos_token)
    model, cfg, step = ckpt.load_model(a.checkpoint, a.device)
    if tok.vocab_size > cfg.model.vocab_size:
        print(f"tokenizer {tok.name} has {tok.vocab_size} ids, the model {cfg.model.vocab_size}", file=sys.stderr)
        return 2
    pool = None
    if a.pool:
        pool = [json.loads(line)["text"] for line in Path(a.pool).read_text().splitlines() if line.strip()]
    tasks = a.tasks or [t for t in RR.TASKS if pool or RR.SPEC[t]["haystack"] != "open" or (a.items and (Path(a.items) / "items" / f"{t}.jsonl.gz").is_file())]
    ac = torch.bfloat16 if a.device.startswith("cuda") else None
    values = score(model, tok, tasks, a.lengths, a.n_per_cell, a.batch, pool, Path(a.out), a.run, ac, items_dir=a.items)
    for k in sorted(values["cells"]):
        if k.endswith("|recall"):
            print(f"{k}: {values['cells'][k]:.4f}")
    return 0


if __name__ == "__main__":
    sys.exit(main())
