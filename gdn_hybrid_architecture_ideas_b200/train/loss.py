"""Reference language-model loss: token cross-entropy plus z-loss on fp32 logits
(reference: ced/train/loss.py:20-58)."""

from __future__ import annotations

import torch
import torch.nn.functional as F


def lm_loss(logits: torch.Tensor, targets: torch.Tensor, valid: torch.Tensor | None = None, z_loss: float = 0.0,
            weights: torch.Tensor | None = None):
    """logits (..., V), targets (...). Returns (loss, ce_sum, z_sum, count): loss = (ce_sum + z_loss * z_sum) / count with
    sums over valid positions (optionally weighted), z = logsumexp(logits)^2."""
    lg = logits.float().reshape(-1, logits.shape[-1])
    tg = targets.reshape(-1)
    w = torch.ones_like(tg, dtype=torch.float32) if weights is None else weights.reshape(-1).float()
    if valid is not None:
        w = w * valid.reshape(-1).float()
    lse = torch.logsumexp(lg, dim=-1)
    ce = lse - lg.gather(1, tg.clamp_min(0)[:, None])[:, 0]
    ce_sum, z_sum, count = (ce * w).sum(), (lse * lse * w).sum(), w.sum()
    return (ce_sum + z_loss * z_sum) / count.clamp_min(1.0), ce_sum, z_sum, count
