"""Token-superposition training plan: phases `[[start_step, s], ...]` in which a position is a bag of s consecutive
tokens (input = mean of their embeddings; loss = weighted CE against every token of the next bag), followed by plain
training at s = 1. The data stream position is the running sum of rows * seq_len * s, the optimizer moments are reset
at a switch unless `keep_optimizer_state` (reference: ced/train/tst.py:171-260, 452-935).
"""

from __future__ import annotations

import torch

from ..data.synthetic import Batch


def bag_weights(s: int) -> torch.Tensor:
    """Uniform 1/s for s < 8, proportional to 1/i (i = 1..s, normalised) from 8 on."""
    if s < 8:
        return torch.full((s,), 1.0 / s)
    w = 1.0 / torch.arange(1, s + 1, dtype=torch.float64)
    return (w / w.sum()).float()


class TSTSchedule:
    def __init__(self, schedule: list):
        if not schedule:
            raise ValueError("tst.schedule is empty")
        self.phases = sorted((int(a), int(s)) for a, s in schedule)
        if self.phases[0][0] != 0:
            raise ValueError("tst.schedule must start at step 0")
        if any(s < 1 for _, s in self.phases):
            raise ValueError("tst.schedule bag sizes must be >= 1")

    def s_at(self, step: int) -> int:
        s = self.phases[0][1]
        for start, size in self.phases:
            if step >= start:
                s = size
        return s

    def is_switch(self, step: int) -> bool:
        return step > 0 and any(step == start for start, _ in self.phases) and self.s_at(step) != self.s_at(step - 1)

    def tokens_before(self, step: int, rows: int, seq_len: int) -> int:
        """Stream position (in tokens) at the start of `step`."""
        total, bounds = 0, self.phases + [(step, 0)]
        for (a, s), (b, _) in zip(self.phases, bounds[1:]):
            lo, hi = min(a, step), min(b, step)
            total += max(0, hi - lo) * rows * seq_len * s
        if step > self.phases[-1][0] and len(self.phases) > 0:
            pass
        return total


class TSTPlan:
    """Turns the base data source's rows into bag batches during bag phases."""

    def __init__(self, cfg_tst, data, vocab_size: int):
        self.cfg, self.data, self.vocab = cfg_tst, data, vocab_size
        self.schedule = TSTSchedule(cfg_tst.schedule)

    def s_at(self, step: int) -> int:
        return self.schedule.s_at(step)

    def batch_at(self, step: int, first: int, count: int) -> Batch:
        s = self.s_at(step)
        if s == 1:
            return self.data.batch(step, first, count)
        # s plain rows of the same step, drawn from disjoint counter streams, concatenated into one row of L*s tokens
        parts = [self.data.batch(step * 131 + k + 7_000_000, first, count) for k in range(s)]
        seq = torch.cat([torch.cat([p.tokens, p.targets[:, -1:]], dim=1) for p in parts], dim=1)
        L = parts[0].tokens.shape[1]
        seq = seq[:, : (L + 1) * s].reshape(seq.shape[0], L + 1, s)
        tokens, nxt = seq[:, :-1], seq[:, 1:]
        B = tokens.shape[0]
        return Batch(tokens=tokens.contiguous(), targets=nxt[..., 0].contiguous(),
                     target_valid=torch.ones(B, L, dtype=torch.bool), doc_ids=torch.zeros(B, L, dtype=torch.long),
                     multi_targets=nxt.contiguous(), multi_valid=torch.ones(B, L, s, dtype=torch.bool), single_doc=True)

    def data_state(self) -> dict:
        return {"tst_schedule": [list(p) for p in self.schedule.phases]}
