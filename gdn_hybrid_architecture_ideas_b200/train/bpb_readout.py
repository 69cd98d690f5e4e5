"""Cheap in-loop readout: bits per byte on a FIXED sample of eval rows, every `eval.bpb_readout_every` steps from step
`eval.bpb_readout_from`. The sample (at most `eval.bpb_readout_rows` rows per set) is drawn once from
`eval.bpb_readout_seed`, so the curve over training compares like with like; results go to the metrics stream as
`readout/<set>/bpb`. Like every evaluation it restores the RNG streams and the model's mode
(reference: ced/train/bpb_readout.py:79-371, FixedRows in ced/train/periodic_eval.py:276)."""

from __future__ import annotations

import torch

from ..eval import span_bpb
from . import periodic_eval
from .sharded_eval import evaluate_sharded


class FixedRows:
    """The packed rows of one eval set with a seeded, fixed choice of rows."""

    def __init__(self, docs, seq_len: int, max_rows: int, seed: int):
        self.rows = span_bpb.build_eval_rows(docs, seq_len)
        n = self.rows.tokens.shape[0]
        g = torch.Generator().manual_seed(seed)
        self.chosen = sorted(torch.randperm(n, generator=g)[:max_rows].tolist()) if n > max_rows else list(range(n))


def due(cfg, step: int) -> bool:
    e = cfg.eval
    return e.bpb_readout_every > 0 and bool(e.bpb_readout_sets) and step >= e.bpb_readout_from and step % e.bpb_readout_every == 0


class BpbReadout:
    def __init__(self, trainer):
        self.trainer = trainer
        self.sets: dict[str, FixedRows] = {}

    def _load(self):
        cfg = self.trainer.cfg
        for name, spec in cfg.eval.bpb_readout_sets.items():
            if name not in self.sets:
                docs = periodic_eval.load_set(spec, self.trainer)
                self.sets[name] = FixedRows(docs, cfg.data.seq_len + 1, cfg.eval.bpb_readout_rows, cfg.eval.bpb_readout_seed)

    def run(self) -> dict:
        t = self.trainer
        self._load()
        saved = periodic_eval.rng_states(t.device)
        was_training = t.model.training
        out = {}
        try:
            ac = torch.bfloat16 if t.cfg.autocast == "bfloat16" else None
            for name, fixed in self.sets.items():
                rows = fixed.rows
                sub = span_bpb.EvalRows(*(getattr(rows, f)[fixed.chosen] for f in ("tokens", "targets", "doc_ids", "scored", "target_bytes", "doc_index")),
                                        n_docs=rows.n_docs, skipped=rows.skipped)
                ev = evaluate_sharded(t.model, sub, t.dp, max(t.cfg.eval.batch_size, 1), autocast_dtype=ac)
                if ev is not None:
                    out[f"readout/{name}/bpb"] = ev.bpb
        finally:
            t.model.train(was_training)
            periodic_eval.rng_restore(saved, t.device)
        return out
