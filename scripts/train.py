#!/usr/bin/env python
"""Train from a YAML config: `python scripts/train.py --config C.yaml --run-dir DIR [--steps N] [--until-step K]
[--set a.b=value ...]`. Under torchrun (WORLD_SIZE > 1) every rank runs this file and joins the data-parallel group.
A run directory with a `latest` checkpoint is resumed; a changed config is refused unless --allow-config-change.
Exit status 86: the run stopped on a non-finite loss (reference: scripts/train.py:64-213)."""

from __future__ import annotations

import argparse
import sys
from pathlib import Path

sys.path.insert(0, str(Path(__file__).resolve().parent.parent))

import torch  # noqa: E402

from gdn_hybrid_architecture_ideas_b200 import config as C  # noqa: E402
from gdn_hybrid_architecture_ideas_b200.parallel import data_parallel  # noqa: E402
from gdn_hybrid_architecture_ideas_b200.train import checkpoint as ckpt  # noqa: E402
from gdn_hybrid_architecture_ideas_b200.train.trainer import EXIT_DIVERGED, Diverged, Trainer  # noqa: E402


def parse(argv=None):
    ap = argparse.ArgumentParser(description=__doc__)
    ap.add_argument("--config", required=True)
    ap.add_argument("--run-dir", required=True)
    ap.add_argument("--steps", type=int, default=None)
    ap.add_argument("--until-step", type=int, default=None)
    ap.add_argument("--wandb", default=None)
    ap.add_argument("--threads", type=int, default=None)
    ap.add_argument("--allow-config-change", action="store_true")
    ap.add_argument("--set", action="append", default=[], metavar="KEY=VALUE")
    return ap.parse_args(argv)


def prepare(args, dp=None) -> Trainer:
    cfg = C.load_yaml(args.config)
    for item in args.set:
        C.apply_override(cfg, item)
    if args.steps is not None:
        cfg.steps = args.steps
    if args.wandb:
        cfg.wandb.mode = args.wandb
    trainer = Trainer(cfg, args.run_dir, dp)
    latest = ckpt.latest_path(Path(args.run_dir))
    if latest is not None:
        state = ckpt.load(latest)
        trainer.load_state_dict(state, check_config=not args.allow_config_change)
        trainer.resume_info = {"path": str(latest), "step": trainer.step}
    elif cfg.resume_from:       # a new run that continues another run's checkpoint (a branch, or a stage on other data)
        trainer.continue_from(cfg.resume_from)
    return trainer


def main(argv=None) -> int:
    args = parse(argv)
    if args.threads:
        torch.set_num_threads(args.threads)
    dp = data_parallel.from_environment()
    try:
        trainer = prepare(args, dp)
        info = getattr(trainer, "resume_info", None)
        if info and trainer.lead:
            print(f"resumed from {info['path']} at step {info['step']}", flush=True)
        trainer.fit(args.until_step)
    except Diverged as e:
        print(f"stopped: {e}", file=sys.stderr)
        return EXIT_DIVERGED
    finally:
        if dp is not None:
            dp.close()
    return 0


if __name__ == "__main__":
    sys.exit(main())
