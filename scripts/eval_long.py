#!/usr/bin/env python
"""Long-context bits per byte by position bucket, and GDN state diagnostics along the row
(reference: scripts/eval_long.py).

    python scripts/eval_long.py --checkpoint RUN --docs long.pt --max-len 65536 [--gdn-diag] [--window 8192] [--out long.json] [--summary long.md]

--window W adds, per position bucket beyond W, the bpb of the bucket's targets with the full context minus the same targets
scored with only the last W tokens of context, and the degradation rule over it (eval/long_report.py).

`long.pt` holds {"docs": [{"ids": LongTensor, "byte_lens": LongTensor}, ...]}.
"""

from __future__ import annotations

import argparse
import json
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from gdn_hybrid_architecture_ideas_b200.eval import gdn_diag, long_context, long_report  # noqa: E402
from gdn_hybrid_architecture_ideas_b200.train import checkpoint as ckpt  # noqa: E402


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__)
    ap.add_argument("--checkpoint", required=True)
    ap.add_argument("--docs", required=True)
    ap.add_argument("--max-len", type=int, default=0)
    ap.add_argument("--base", type=int, default=long_context.BASE_LEN)
    ap.add_argument("--chunk", type=int, default=8192)
    ap.add_argument("--gdn-diag", action="store_true")
    ap.add_argument("--window", type=int, default=0)
    ap.add_argument("--train-len", type=int, default=0, help="degradations are listed beyond this length (default: the run's seq_len)")
    ap.add_argument("--agent-windows", default="", help="comma-separated context windows: the documents carry `assistant` flags (whole agent trajectories) and "
                    "their assistant bpb is scored with the context cut to each window (and to --base, the reference window)")
    ap.add_argument("--agent-tail", type=int, default=0, help="targets of the tail every window holds (default base / 2)")
    ap.add_argument("--summary")
    ap.add_argument("--device", default="cuda" if torch.cuda.is_available() else "cpu")
    ap.add_argument("--out")
    a = ap.parse_args(argv)
    model, cfg, step = ckpt.load_model(a.checkpoint, a.device)
    ac = torch.bfloat16 if a.device.startswith("cuda") else None
    docs = torch.load(a.docs, map_location="cpu", weights_only=False)["docs"]
    if a.agent_windows:
        missing = [i for i, d in enumerate(docs) if "assistant" not in d]
        if missing:
            ap.error(f"--agent-windows: documents {missing[:5]} carry no `assistant` flags")
        res = long_context.score_agent_windows(model, docs, windows=[int(x) for x in a.agent_windows.split(",")], ref_window=a.base,
                                               tail=a.agent_tail or None, base=a.base, chunk=a.chunk, autocast_dtype=ac)
        for W, row in res["window"].items():
            print(f"window {W:>7d}: assistant bpb {row['bpb']:.4f} ({row['trajectories']} trajectories, {row['filled']} filled)")
        if a.out:
            with open(a.out, "w") as f:
                json.dump({"step": step, "agent_windows": res}, f, indent=1, default=lambda o: o.tolist() if hasattr(o, "tolist") else str(o))
        return 0
    docs = [{"ids": torch.as_tensor(d["ids"]), "byte_lens": torch.as_tensor(d["byte_lens"])} for d in docs]
    res = long_context.score_position_bpb(model, docs, base=a.base, max_len=a.max_len or None, chunk=a.chunk, autocast_dtype=ac)
    for line in res["table"]:
        if line["bpb"] is not None:
            print(f"{line['bucket']:>12s}: bpb {line['bpb']:.4f} ({line['docs']} documents)")
    out = {"step": step, "edges": res["edges"], "table": res["table"]}
    if a.gdn_diag:
        ids = docs[0]["ids"][: a.max_len or None][None]
        out["gdn_diag"] = gdn_diag.encoder_gdn_diag(model, ids, torch.zeros_like(ids), block=a.chunk, autocast_dtype=ac)
        # state statistics by position bucket with their drift against the last bucket inside the training length
        out["gdn_positions"] = gdn_diag.gdn_position_diag(model, ids, torch.zeros_like(ids), train_len=a.train_len or cfg.data.seq_len, block=a.chunk,
                                                          autocast_dtype=ac)
    if a.window:
        rows = long_report.context_gain(model, docs if not a.max_len else [{k: v[:a.max_len] for k, v in d.items()} for d in docs], res["edges"], a.window,
                                        a.chunk, ac, full_records=res["records"])
        summary = {"bpb": {"docs": rows}}
        entries = long_report.degradations(summary, train_len=a.train_len or cfg.data.seq_len)
        out["context_gain"], out["degradations"], out["breaks_first"] = rows, entries, long_report.breaks_first(entries)
        text = long_report.render(summary, entries)
        print(text)
        if a.summary:
            with open(a.summary, "w") as f:
                f.write(text)
    if a.out:
        with open(a.out, "w") as f:
            json.dump(out, f, indent=1)
    return 0


if __name__ == "__main__":
    sys.exit(main())
