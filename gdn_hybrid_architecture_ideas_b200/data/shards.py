"""Packs the documents of a shard set into fixed-length training rows.

Each epoch is one permutation of the documents (seeded by (seed, epoch)); documents are laid end to end and cut
into rows of seq_len + 1 tokens; a document cut by a row boundary continues in the next row under a new document
id. Row r of the global stream is a pure function of (seed, r), so `rows(first, count)` serves data-parallel slices
and a resume needs only the step (reference: ced/train/shards.py:92-342 — same contract, own algorithm). Under a
per-token loss mask (`data.loss_mask`: "assistant", or a loss-span mode) every row also carries which of its targets
keep their loss, read from the shard set's side arrays; the invariants a mask relies on are checked when the packer is
built and their identity goes into the checkpoint's data state.
"""

from __future__ import annotations

import numpy as np
import torch

from ..config import DataConfig
from .synthetic import Batch


class ShardPacker:
    def __init__(self, shards, cfg: DataConfig):
        self.shards, self.cfg = shards, cfg
        self.n_docs = len(shards)
        lens = shards.doc_len(np.arange(self.n_docs))
        self.tokens_per_epoch = int(lens.sum())
        self.row_tokens = cfg.seq_len + 1
        self.rows_per_epoch = self.tokens_per_epoch // self.row_tokens
        if self.rows_per_epoch < 1:
            raise ValueError("the shard set holds less than one row of tokens")
        self._epoch = None
        # per-token loss mask (data.loss_mask): which TARGETS keep their loss, from the set's side arrays
        from .shard_format import LOSS_MASK_MODES, LOSS_SPAN_KEEP, check_loss_spans, loss_keep_table

        self.loss_mask = getattr(cfg, "loss_mask", "all")
        if self.loss_mask not in LOSS_MASK_MODES:
            raise ValueError(f"data.loss_mask {self.loss_mask!r}: one of {LOSS_MASK_MODES}")
        self.loss_spans_state, self._keep, self._flags = None, None, None
        if self.loss_mask != "all":
            self.loss_spans_state = check_loss_spans(shards, self.loss_mask)
            if self.loss_mask in LOSS_SPAN_KEEP:
                self._keep, self._flags = loss_keep_table(self.loss_mask), shards.side("loss_spans")
            else:
                self._flags = shards.side("generated")
            self._doc_starts = np.asarray(shards.starts)

    def _load_epoch(self, epoch: int) -> None:
        if self._epoch == epoch:
            return
        rng = np.random.default_rng([self.cfg.seed, epoch])
        self._perm = rng.permutation(self.n_docs)
        self._cum = np.concatenate([[0], np.cumsum(self.shards.doc_len(self._perm))])
        self._epoch = epoch

    def row(self, index: int):
        """(tokens (L+1,), doc ids (L+1,)) of global row `index`."""
        epoch, r = divmod(index, self.rows_per_epoch)
        self._load_epoch(epoch)
        lo, hi = r * self.row_tokens, (r + 1) * self.row_tokens
        d = int(np.searchsorted(self._cum, lo, side="right") - 1)
        toks, docs, keeps, at, k = [], [], [], lo, 0
        while at < hi:
            which = int(self._perm[d])
            doc = self.shards.doc(which)
            a = at - int(self._cum[d])
            take = min(len(doc) - a, hi - at)
            toks.append(doc[a:a + take])
            docs.append(np.full(take, k, dtype=np.int64))
            if self._flags is not None:      # the mask value of every token of the piece, as a TARGET
                t0 = int(self._doc_starts[which]) + a
                f = np.asarray(self._flags[t0:t0 + take])
                keeps.append(self._keep[f] if self._keep is not None else f > 0)
            at, d, k = at + take, d + 1, k + 1
        keep = np.concatenate(keeps) if keeps else None
        return np.concatenate(toks).astype(np.int64), np.concatenate(docs), keep

    def rows(self, first: int, count: int) -> Batch:
        rows = [self.row(i) for i in range(first, first + count)]
        seq = torch.from_numpy(np.stack([r[0] for r in rows]))
        docs = torch.from_numpy(np.stack([r[1] for r in rows]))
        mask = None if rows[0][2] is None else torch.from_numpy(np.stack([r[2] for r in rows]))[:, 1:].contiguous()
        return Batch(tokens=seq[:, :-1].contiguous(), targets=seq[:, 1:].contiguous(),
                     target_valid=(docs[:, 1:] == docs[:, :-1]).contiguous(), doc_ids=docs[:, :-1].contiguous(), loss_mask=mask)

    def batch(self, step: int, first: int = 0, count: int | None = None) -> Batch:
        B = self.cfg.batch_size
        return self.rows(step * B + first, B - first if count is None else count)

    def fingerprint(self) -> str:
        return self.shards.fingerprint()
