"""Packs the documents of a shard set into fixed-length training rows.

Each epoch is one permutation of the documents (seeded by (seed, epoch)); documents are laid end to end and cut
into rows of seq_len + 1 tokens; a document cut by a row boundary continues in the next row under a new document
id. Row r of the global stream is a pure function of (seed, r), so `rows(first, count)` serves data-parallel slices
and a resume needs only the step (reference: ced/train/shards.py:92-342 — same contract, own algorithm). Under a
per-token loss mask (`data.loss_mask`: "assistant", or a loss-span mode) every row also carries which of its targets
keep their loss, read from the shard set's side arrays; the invariants a mask relies on are checked when the packer is
built and their identity goes into the checkpoint's data state.

`data.chat_whole`: a chat document of at most one row is never cut by a row boundary. When it does not fit the rest of
the current row, that space is filled with the head of the next non-chat document(s) of the permutation, the chat
document opens the next row, and the tail of a partly used filler follows it: every token is still used once per epoch,
only the order of the pieces changes. A chat document longer than a row, or one near the end of an epoch with no
non-chat document left to fill with, is placed as it comes (counted in `chat_cut`). An epoch is then a list of segments
(document, offset, length) instead of whole documents, computed once per epoch in one pass over the permutation.
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
        perm = rng.permutation(self.n_docs)
        lens = np.asarray(self.shards.doc_len(perm), dtype=np.int64)
        if getattr(self.cfg, "chat_whole", False) and bool(np.asarray(self.shards.doc_chat).any()):
            self._seg_doc, self._seg_off, self._seg_len, self.chat_cut = self._whole_chat_segments(perm, lens)
        else:
            self._seg_doc, self._seg_off, self._seg_len, self.chat_cut = perm, np.zeros(self.n_docs, dtype=np.int64), lens, 0
        self._cum = np.concatenate([[0], np.cumsum(self._seg_len)])
        self._epoch = epoch

    def _whole_chat_segments(self, perm: np.ndarray, lens: np.ndarray):
        """(document, offset, length) per segment of the epoch so that no chat document of at most a row crosses a row boundary."""
        W = self.row_tokens
        chat = np.asarray(self.shards.doc_chat).astype(bool)[perm]
        taken = np.zeros(len(perm), dtype=bool)
        fillers = [j for j in range(len(perm)) if not chat[j]]
        nxt = 0                       # next filler candidate
        doc, off, ln = [], [], []
        pos = cut = 0
        for j in range(len(perm)):
            if taken[j]:
                continue
            taken[j] = True
            n, tail = int(lens[j]), None
            if chat[j] and n <= W:
                room = W - pos % W
                if n > room:          # does not fit: fill the rest of the row with non-chat text, then start the next row
                    need = room
                    while need > 0:
                        while nxt < len(fillers) and (fillers[nxt] <= j or taken[fillers[nxt]]):
                            nxt += 1
                        if nxt == len(fillers):
                            cut += 1
                            break
                        k = fillers[nxt]
                        taken[k] = True
                        take = min(need, int(lens[k]))
                        doc.append(int(perm[k])), off.append(0), ln.append(take)
                        pos, need = pos + take, need - take
                        if take < int(lens[k]):
                            tail = (int(perm[k]), take, int(lens[k]) - take)
            elif chat[j]:
                cut += 1
            doc.append(int(perm[j])), off.append(0), ln.append(n)
            pos += n
            if tail is not None:
                doc.append(tail[0]), off.append(tail[1]), ln.append(tail[2])
                pos += tail[2]
        return np.asarray(doc, dtype=np.int64), np.asarray(off, dtype=np.int64), np.asarray(ln, dtype=np.int64), cut

    def row(self, index: int):
        """(tokens (L+1,), doc ids (L+1,)) of global row `index`."""
        epoch, r = divmod(index, self.rows_per_epoch)
        self._load_epoch(epoch)
        lo, hi = r * self.row_tokens, (r + 1) * self.row_tokens
        d = int(np.searchsorted(self._cum, lo, side="right") - 1)
        toks, docs, keeps, at, k = [], [], [], lo, 0
        while at < hi:
            which = int(self._seg_doc[d])
            doc = self.shards.doc(which)
            a = int(self._seg_off[d]) + at - int(self._cum[d])           # offset inside the document
            take = min(int(self._seg_off[d]) + int(self._seg_len[d]) - a, hi - at)
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
