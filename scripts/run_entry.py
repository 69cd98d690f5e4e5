#!/usr/bin/env python
"""Launch one named entry of a runs file: base config + `set` overrides, `${DATA_ROOT}` / `${RUN_ROOT}` expanded;
`--nproc N` > 1 launches through torchrun on this node (reference: scripts/run_entry.py:41-137).

    python scripts/run_entry.py runs/bench-200m.yaml --list
    python scripts/run_entry.py runs/bench-200m.yaml --name full200-dp --nproc 8 --run-root /tmp/runs [--dry-run]
"""

from __future__ import annotations

import argparse
import os
import shlex
import subprocess
import sys
from pathlib import Path

import yaml

ROOT = Path(__file__).resolve().parent.parent


def load_runs(path: str | Path, data_root: str, run_root: str) -> dict:
    text = Path(path).read_text().replace("${DATA_ROOT}", data_root).replace("${RUN_ROOT}", run_root)
    return yaml.safe_load(text)


def find_entry(runs: dict, name: str) -> dict:
    for entry in runs.get("runs", []):
        if entry["name"] == name:
            return entry
    raise KeyError(f"no entry {name!r}; entries: {[e['name'] for e in runs.get('runs', [])]}")


def build_command(runs: dict, entry: dict, run_root: str, nproc: int = 1, port: int = 29511) -> list[str]:
    sets = list(entry.get("set", []))
    if "seed" in entry:
        sets.append(f"seed={entry['seed']}")
    shards = entry.get("shards", runs.get("shards"))
    if shards and not any(s.startswith("data.kind=") for s in sets):
        sets.append(f"data.shard_dir={shards}")
    train = [str(ROOT / "scripts" / "train.py"), "--config", str(ROOT / entry["config"]),
             "--run-dir", str(Path(run_root) / entry["name"])]
    for s in sets:
        train += ["--set", s]
    if nproc > 1:
        return [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={nproc}",
                "--master-addr", "127.0.0.1", "--master-port", str(port)] + train
    return [sys.executable] + train


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__)
    ap.add_argument("runs")
    ap.add_argument("--list", action="store_true")
    ap.add_argument("--name")
    ap.add_argument("--nproc", type=int, default=1)
    ap.add_argument("--data-root", default=os.environ.get("DATA_ROOT", "/data"))
    ap.add_argument("--run-root", default=os.environ.get("RUN_ROOT", "/tmp/runs"))
    ap.add_argument("--dry-run", action="store_true")
    args = ap.parse_args(argv)
    runs = load_runs(args.runs, args.data_root, args.run_root)
    if args.list:
        for e in runs.get("runs", []):
            print(e["name"])
        return 0
    cmd = build_command(runs, find_entry(runs, args.name), args.run_root, args.nproc)
    print(" ".join(shlex.quote(c) for c in cmd))
    return 0 if args.dry_run else subprocess.call(cmd)


if __name__ == "__main__":
    sys.exit(main())
