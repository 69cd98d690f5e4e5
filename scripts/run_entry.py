#!/usr/bin/env python
"""Launch one named entry of a runs file: base config + overrides, `${DATA_ROOT}` / `${RUN_ROOT}` expanded;
`--nproc N` > 1 launches through torchrun on this node (reference: scripts/run_entry.py:41-137).

A runs file: `shards` (a shard directory, or a list read as one stream), `eval_dir`, optionally `common` (a nested patch every
entry starts from) and `runs`, each entry with `name`, `base` (or `config`), `seed` and its overrides as a nested `patch`
mirroring the config's sections and / or a flat `set` list of KEY=VALUE strings. The published runs files of the reference
(flat `set` lists) load as they are. An entry that continues another names it under `continues` (or `after` /
`after_step`): informational, the continuation itself is the entry's `resume_from` override.

    python scripts/run_entry.py runs/bench-200m.yaml --list
    python scripts/run_entry.py runs/bench-200m.yaml --name full200-dp --nproc 8 --run-root /tmp/runs [--dry-run]
"""

from __future__ import annotations

import argparse
import json
import os
import shlex
import subprocess
import sys
from pathlib import Path

import yaml

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT))

from gdn_hybrid_architecture_ideas_b200 import config as C  # noqa: E402


def load_runs(path: str | Path, data_root: str, run_root: str) -> dict:
    text = Path(path).read_text().replace("${DATA_ROOT}", data_root).replace("${RUN_ROOT}", run_root)
    return yaml.safe_load(text)


def flatten_patch(patch: dict, schema=None, prefix: str = "") -> list[str]:
    """A nested patch over the base config ({model: {encoder: {attn_res: block_entry}}, steps: 10}) as train.py overrides
    (`model.encoder.attn_res=block_entry`, `steps=10`). The config's own structure says where a mapping is a section to
    descend into and where it is a value (eval.sets, gdn_shape_by_layer): a key the config does not have raises KeyError."""
    import dataclasses

    schema = C.TrainConfig() if schema is None else schema
    out = []
    for key, value in patch.items():
        path = f"{prefix}{key}"
        if not hasattr(schema, key):
            raise KeyError(f"unknown config key {path!r}")
        node = getattr(schema, key)
        if dataclasses.is_dataclass(node):
            if not isinstance(value, dict):
                raise ValueError(f"{path} is a section of the config: give it a mapping, not {value!r}")
            out += flatten_patch(value, node, path + ".")
        elif value is None:
            out.append(f"{path}=null")
        elif isinstance(value, bool):
            out.append(f"{path}={'true' if value else 'false'}")
        elif isinstance(value, (list, tuple, dict)):
            out.append(f"{path}={json.dumps(value)}")
        else:
            out.append(f"{path}={value}")
    return out


def entry_overrides(runs: dict, entry: dict) -> list[str]:
    """The entry's own overrides, in order: the file's `common` patch, the entry's `patch` (nested form), then its `set`
    list (flat KEY=VALUE form; the published runs files use only this one)."""
    out = flatten_patch(runs.get("common") or {}) + flatten_patch(entry.get("patch") or {})
    return out + [str(x) for x in entry.get("set", [])]


def find_entry(runs: dict, name: str) -> dict:
    for entry in runs.get("runs", []):
        if entry["name"] == name:
            return entry
    raise KeyError(f"no entry {name!r}; entries: {[e['name'] for e in runs.get('runs', [])]}")


# Held-out text sets a run scores while it trains: name -> file inside the runs file's `eval_dir`; only files that exist are passed.
EVAL_SETS = {"web": "web.pt", "code": "code.pt", "agent": "agent.pt", "general_web": "general_web.pt"}


def build_command(runs: dict, entry: dict, run_root: str, nproc: int = 1, port: int = 29511, extra_sets=(), check_eval: bool = True) -> list[str]:
    """The training process's argv for one entry. Overrides, in order: the seed (and, for a shard-fed entry, the data seed
    1000 + seed, the first shard set and any further ones as one stream), the eval sets found in `eval_dir`, the entry's own
    `set` list, then `extra_sets` from the command line."""
    sets = []
    if "seed" in entry:
        sets.append(f"seed={int(entry['seed'])}")
    shards = entry.get("shards", runs.get("shards"))
    own = entry_overrides(runs, entry)
    if shards and not any(x.startswith("data.kind=") for x in own):
        first, *more = shards if isinstance(shards, list) else [shards]
        if "seed" in entry:
            sets.append(f"data.seed={1000 + int(entry['seed'])}")
        sets += ["data.kind=shards", f"data.shard_dir={first}"]
        if more:
            sets.append("data.extra_shard_dirs=" + json.dumps(more))
    eval_dir = runs.get("eval_dir")
    if eval_dir:
        present = {k: f"{eval_dir}/{v}" for k, v in EVAL_SETS.items() if not check_eval or (Path(eval_dir) / v).is_file()}
        if present:
            sets.append("eval.sets=" + json.dumps(present))
    sets += own + [str(x) for x in extra_sets]
    train = [str(ROOT / "scripts" / "train.py"), "--config", str(ROOT / (entry.get("config") or entry["base"])),
             "--run-dir", str(Path(run_root) / entry["name"])]
    for x in sets:
        train += ["--set", x]
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
    ap.add_argument("--set", dest="extra", action="append", default=[], metavar="KEY=VALUE", help="a further train.py override, after the entry's own")
    ap.add_argument("--dry-run", action="store_true")
    args = ap.parse_args(argv)
    runs = load_runs(args.runs, args.data_root, args.run_root)
    if args.list:
        for e in runs.get("runs", []):       # an entry that continues another names it: run that one first
            src = e.get("continues") or ({"run": e["after"], "step": e.get("after_step", "end")} if e.get("after") else None)
            print(e["name"] + (f"  (after {src['run']} step {src.get('step', 'end')})" if src else ""))
        return 0
    cmd = build_command(runs, find_entry(runs, args.name), args.run_root, args.nproc, extra_sets=args.extra, check_eval=not args.dry_run)
    print(" ".join(shlex.quote(c) for c in cmd))
    return 0 if args.dry_run else subprocess.call(cmd)


if __name__ == "__main__":
    sys.exit(main())
