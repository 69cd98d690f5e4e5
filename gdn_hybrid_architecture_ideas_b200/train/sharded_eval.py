"""Evaluation rows shared out over the data-parallel ranks: each rank scores a contiguous block of batches, the
partial per-row sums go to rank 0 through the host group and are added (reference: ced/train/sharded_eval.py:36-73)."""

from __future__ import annotations

from ..eval import span_bpb


def batch_block(n_rows: int, batch_size: int, rank: int, world: int) -> list[int]:
    """Row indices of this rank: a contiguous block of whole batches (earlier ranks take the remainder)."""
    n_batches = -(-n_rows // batch_size)
    per, extra = divmod(n_batches, world)
    first = rank * per + min(rank, extra)
    count = per + (1 if rank < extra else 0)
    return list(range(first * batch_size, min((first + count) * batch_size, n_rows)))


def evaluate_sharded(model, rows, dp, batch_size: int = 8, **kwargs):
    """SpanEval on rank 0, None on the other ranks. dp None: plain evaluate."""
    if dp is None or dp.world == 1:
        return span_bpb.evaluate(model, rows, batch_size, **kwargs)
    mine = batch_block(rows.tokens.shape[0], batch_size, dp.rank, dp.world)
    part = span_bpb.evaluate(model, rows, batch_size, row_indices=mine, **kwargs)
    parts = dp.gather_to_lead(part)
    return span_bpb.join_batches(parts) if dp.lead else None
