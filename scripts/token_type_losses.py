#!/usr/bin/env python
"""Loss of a checkpoint on agent trajectories, split by what kind of token is predicted (reasoning, call head,
arguments, copied spans, code, final answer, other) (reference: ced/eval/token_types.py; its analysis reads the same
labels against stored per-token losses).

    python scripts/token_type_losses.py --checkpoint RUN --set agent.pt [--chunk 8192] [--out types.json]

The set is one built by `scripts/build_eval_set.py --agent`: it carries the byte table and the control-token ids the
labels are computed from. Each conversation is scored whole, read in chunks through the cache.
"""

from __future__ import annotations

import argparse
import json
import os
import sys

import numpy as np
import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from gdn_hybrid_architecture_ideas_b200.eval import long_context, token_types  # noqa: E402
from gdn_hybrid_architecture_ideas_b200.train import checkpoint as ckpt  # noqa: E402


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__)
    ap.add_argument("--checkpoint", required=True)
    ap.add_argument("--set", required=True)
    ap.add_argument("--chunk", type=int, default=8192)
    ap.add_argument("--copy-min", type=int, default=token_types.COPY_MIN_TOKENS)
    ap.add_argument("--device", default="cuda" if torch.cuda.is_available() else "cpu")
    ap.add_argument("--out")
    a = ap.parse_args(argv)
    blob = torch.load(a.set, map_location="cpu", weights_only=False)
    if "token_bytes" not in blob:
        ap.error("the set carries no byte table: build it with scripts/build_eval_set.py --agent")
    model, cfg, step = ckpt.load_model(a.checkpoint, a.device)
    if cfg.model.vocab_size < len(blob["token_bytes"]):
        ap.error(f"the model's vocabulary ({cfg.model.vocab_size}) is smaller than the set's ({len(blob['token_bytes'])})")
    ac = torch.bfloat16 if a.device.startswith("cuda") else None
    labels, losses, lens, stats = [], [], [], {}
    for d in blob["docs"]:
        ids = torch.tensor(d["ids"])
        lab = token_types.label_document(d["ids"], d["scored"], blob["token_bytes"], blob["control"], a.copy_min, stats)
        ce = long_context.position_ce(model, ids, a.chunk, ac).numpy()
        labels.append(lab[1:])                      # the loss at i - 1 predicts token i
        losses.append(ce)
        lens.append(np.asarray(d["byte_lens"])[1:])
    out = {"step": step, "loss": token_types.loss_by_type(labels, losses), "shares": token_types.summarize(labels, lens), **stats}
    for name, v in out["loss"].items():
        print(f"{name:10s} {v['tokens']:8d} tokens  loss {v['loss'] if v['loss'] is None else round(v['loss'], 4)}")
    if a.out:
        with open(a.out, "w") as f:
            json.dump(out, f, indent=1)
    return 0


if __name__ == "__main__":
    sys.exit(main())
