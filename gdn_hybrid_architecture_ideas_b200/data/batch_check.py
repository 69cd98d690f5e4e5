"""Host-side validation of a batch before any kernel sees it: id ranges, shapes, document-id monotonicity and
cumulative-length metadata. A bad batch raises BatchError naming the rows, so every data-parallel rank can halt at
the same update (reference: ced/train/batch_check.py:47-194)."""

from __future__ import annotations

import hashlib

import numpy as np
import torch


class BatchError(ValueError):
    def __init__(self, message: str, rows=()):
        super().__init__(message)
        self.rows = list(rows)


def check_doc_ids(doc_ids: torch.Tensor) -> None:
    d = doc_ids.cpu().numpy()
    bad = np.nonzero((np.diff(d, axis=1) < 0).any(axis=1))[0]
    if bad.size:
        raise BatchError(f"document ids decrease along rows {bad.tolist()}", bad.tolist())


def check_cu_seqlens(cu: np.ndarray, total: int) -> None:
    cu = np.asarray(cu)
    if cu.ndim != 1 or cu.size < 2 or cu[0] != 0 or cu[-1] != total or (np.diff(cu) < 0).any():
        raise BatchError(f"cu_seqlens must rise from 0 to {total}, got {cu[:4].tolist()} .. {cu[-2:].tolist()}")


def check_batch(batch, vocab_size: int) -> None:
    t = batch.tokens
    if t.dtype != torch.long:
        raise BatchError(f"token ids must be int64, got {t.dtype}")
    lo, hi = int(t.min()), int(t.max())
    if lo < 0 or hi >= vocab_size:
        rows = ((t < 0) | (t >= vocab_size)).flatten(1).any(1).nonzero().flatten().tolist()
        raise BatchError(f"token id outside [0, {vocab_size}) in rows {rows}", rows)
    if batch.targets.shape != t.shape[:2] or batch.doc_ids.shape != t.shape[:2] or batch.target_valid.shape != t.shape[:2]:
        raise BatchError("targets, doc_ids and target_valid must have the tokens' (B, L) shape")
    valid_targets = batch.targets[batch.target_valid]
    if valid_targets.numel() and (int(valid_targets.min()) < 0 or int(valid_targets.max()) >= vocab_size):
        raise BatchError(f"target id outside [0, {vocab_size})")
    check_doc_ids(batch.doc_ids)


def row_hashes(tokens: torch.Tensor) -> list[int]:
    """63-bit digest of every row (ranks exchange them to prove they read disjoint, expected rows)."""
    return [int.from_bytes(hashlib.blake2b(r.cpu().numpy().tobytes(), digest_size=8).digest(), "little") & (2 ** 63 - 1)
            for r in tokens]
