"""Unfused LM head: logits and cross-entropy over chunks of positions under activation checkpointing, so that only one
chunk's (positions x vocabulary) logits are alive at a time. Valid targets are gathered first and padded to a whole
number of chunks, which keeps shapes static (reference: ced/train/chunked_loss.py:33-297)."""

from __future__ import annotations

import torch
import torch.utils.checkpoint as ckpt

HEAD_CHUNK = 1024


def head_positions(valid: torch.Tensor, chunk: int = HEAD_CHUNK):
    """(index, weight): flat indices of the valid targets first, padded with index 0 / weight 0 to a multiple of `chunk`
    (a fixed-shape stand-in for boolean indexing)."""
    flat = valid.reshape(-1)
    order = torch.argsort((~flat).to(torch.uint8), stable=True)
    n = flat.numel()
    padded = -(-n // chunk) * chunk
    idx = torch.zeros(padded, dtype=torch.long, device=valid.device)
    idx[:n] = order
    w = torch.zeros(padded, dtype=torch.float32, device=valid.device)
    w[:n] = flat[order].float()
    return idx, w


def _chunk_sums(h, weight, targets, w, z_loss):
    logits = h.float() @ weight.float().t()
    lse = torch.logsumexp(logits, dim=-1)
    ce = lse - logits.gather(1, targets[:, None])[:, 0]
    return (ce * w).sum(), (lse * lse * w).sum()


def token_ce(hidden: torch.Tensor, weight: torch.Tensor, targets: torch.Tensor, valid: torch.Tensor, z_loss: float = 0.0,
             chunk: int = HEAD_CHUNK):
    """hidden (B, L, d), weight (V, d), targets/valid (B, L). Returns (ce_sum, z_sum, count) like the fused head."""
    idx, w = head_positions(valid, chunk)
    h = hidden.reshape(-1, hidden.shape[-1])[idx]
    t = targets.reshape(-1)[idx].clamp_min(0)
    ce_sum = hidden.new_zeros((), dtype=torch.float32)
    z_sum = hidden.new_zeros((), dtype=torch.float32)
    for s in range(0, idx.numel(), chunk):
        args = (h[s:s + chunk], weight, t[s:s + chunk], w[s:s + chunk], z_loss)
        if torch.is_grad_enabled() and (hidden.requires_grad or weight.requires_grad):
            c, z = ckpt.checkpoint(_chunk_sums, *args, use_reentrant=False)
        else:
            c, z = _chunk_sums(*args)
        ce_sum, z_sum = ce_sum + c, z_sum + z
    return ce_sum, z_sum, w.sum()
