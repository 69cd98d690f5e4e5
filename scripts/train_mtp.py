#!/usr/bin/env python
"""Train the multi-token-prediction drafter head on a frozen trunk (reference: ced/model/mtp.py:30-40 names this script).

    python scripts/train_mtp.py --checkpoint RUN_DIR_OR_FILE --steps 2000 [--lr 3e-4] [--out head.pt]

Loads a trained trunk, attaches a fresh head when the checkpoint has none, freezes every trunk tensor and runs AdamW on
the head alone over the run's own data stream (the batches after the trunk's last step). Prints the CE of t_{i+2} and
the draft's top-1 accuracy; --out saves the head's tensors (keys under `mtp.`).
"""

from __future__ import annotations

import argparse
import json
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from gdn_hybrid_architecture_ideas_b200.data.synthetic import make_data  # noqa: E402
from gdn_hybrid_architecture_ideas_b200.models import mtp  # noqa: E402
from gdn_hybrid_architecture_ideas_b200.train import checkpoint as ckpt  # noqa: E402


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__)
    ap.add_argument("--checkpoint", required=True)
    ap.add_argument("--steps", type=int, default=1000)
    ap.add_argument("--lr", type=float, default=3e-4)
    ap.add_argument("--weight-decay", type=float, default=0.0)
    ap.add_argument("--rows", type=int, default=0, help="rows per step (default: the run's batch size)")
    ap.add_argument("--log-every", type=int, default=50)
    ap.add_argument("--device", default="cuda" if torch.cuda.is_available() else "cpu")
    ap.add_argument("--out")
    a = ap.parse_args(argv)
    model, cfg, step = ckpt.load_model(a.checkpoint, a.device)
    if getattr(model, "mtp", None) is None:
        cfg.model.mtp.enabled = True
        mtp.check_mtp(cfg.model)
        torch.manual_seed(cfg.seed + 1)
        mtp.attach_mtp(model)
        model.mtp.to(a.device)
    head = mtp.freeze_trunk(model)
    # the frozen trunk is guarded: no gradient, no optimizer state, and its bytes are checked against the digest taken here
    from gdn_hybrid_architecture_ideas_b200.train.freeze_trunk import TrunkGuard

    guard = TrunkGuard(model, (mtp.PREFIX,))
    model.eval()
    model.mtp.train()
    opt = torch.optim.AdamW(head, lr=a.lr, weight_decay=a.weight_decay)
    guard.check_optimizer(opt)
    data = make_data(cfg.data, cfg.model.vocab_size)
    rows = a.rows or cfg.data.batch_size
    ac = torch.autocast("cuda", dtype=torch.bfloat16) if a.device.startswith("cuda") else torch.autocast("cpu", enabled=False)
    last = {}
    for i in range(a.steps):
        b = data.batch(step + i, 0, rows)
        dev = lambda t: t.to(a.device, non_blocking=True)
        with ac:
            last = mtp.train_step(model, opt, dev(b.tokens), dev(b.doc_ids), dev(b.targets), dev(b.target_valid))
        guard.check_grads()
        if a.log_every and (i % a.log_every == 0 or i == a.steps - 1):
            guard.check_values()
            print(json.dumps({"step": i, **last}))
    guard.check_values()
    if a.out:
        torch.save({"trunk_step": step, "head": {k: v.cpu() for k, v in model.state_dict().items() if k.startswith(mtp.PREFIX)}}, a.out)
    return 0


if __name__ == "__main__":
    sys.exit(main())
