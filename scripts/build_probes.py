#!/usr/bin/env python
"""Build a stored probe set: the synthetic recall probes of `eval/probes.py` written once, so every checkpoint of a
comparison is scored on the same file (reference: tools/build_probes.py, tools/build_probes_multifact.py).

    python scripts/build_probes.py --vocab 65536 --lengths 8192,16384,32768 --per-kind 100 --out probes.pt
                                   [--kinds needle,multikey,mf_chain,...] [--seed 0] [--n-keys 8] [--extend old.pt]

The file holds {"probes": [{"id", "kind", "length", "ids", "answer_start", "answer_len", "pieces", "group"}], "vocab", "seed"}.
An item is a pure function of (seed, kind, length, index): --extend keeps an older set's items as the first block of every
cell, checks them token for token against what this build generates, and appends the new ones. Score the file with
`scripts/eval_probes.py --set probes.pt`.
"""

from __future__ import annotations

import argparse
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from gdn_hybrid_architecture_ideas_b200.eval import probes  # noqa: E402


def probe_id(kind: str, length: int, index: int) -> str:
    return f"{kind}/len={length}/{index:04d}"


def build(vocab: int, lengths, kinds, per_kind: int, seed: int, n_keys: int) -> list[dict]:
    out = []
    for length in lengths:
        for kind in kinds:
            for i in range(per_kind):
                p = probes.build_probe(kind, vocab, length, seed, i, n_keys=n_keys)
                out.append({"id": probe_id(kind, length, i), "kind": kind, "length": length, "ids": p.ids, "answer_start": p.answer_start,
                            "answer_len": p.answer_len, "pieces": p.pieces, "group": p.group})
    return out


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--vocab", type=int, required=True)
    ap.add_argument("--lengths", default="512,2048")
    ap.add_argument("--kinds", default=",".join(probes.PROBE_KINDS))
    ap.add_argument("--per-kind", type=int, default=16)
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--n-keys", type=int, default=8)
    ap.add_argument("--extend")
    ap.add_argument("--out", required=True)
    a = ap.parse_args(argv)
    kinds = a.kinds.split(",")
    bad = [k for k in kinds if k not in probes.PROBE_KINDS]
    if bad:
        ap.error(f"unknown probe kinds {bad}: one of {probes.PROBE_KINDS}")
    items = build(a.vocab, [int(x) for x in a.lengths.split(",")], kinds, a.per_kind, a.seed, a.n_keys)
    if a.extend:
        old = torch.load(a.extend, map_location="cpu", weights_only=False)
        if (old["vocab"], old["seed"]) != (a.vocab, a.seed):
            ap.error(f"--extend: the old set was built with vocab {old['vocab']} seed {old['seed']}")
        new = {p["id"]: p for p in items}
        for p in old["probes"]:
            if p["id"] not in new:
                ap.error(f"--extend: the old set's item {p['id']} is not in this build (a cell got smaller or left)")
            if new[p["id"]]["ids"] != p["ids"]:
                ap.error(f"--extend: item {p['id']} differs from the old set's: the generator changed")
    torch.save({"probes": items, "vocab": a.vocab, "seed": a.seed, "n_keys": a.n_keys}, a.out)
    print(f"{len(items)} probes, {sum(len(p['ids']) for p in items)} tokens -> {a.out}")
    return 0


if __name__ == "__main__":
    sys.exit(main())
