"""Monitor of exact-zero weight-gradient entries per linear layer: under low-precision recipes an underflowing
gradient shows up as entries that are exactly zero (reference: ced/train/zero_wgrad.py:33-86)."""

from __future__ import annotations

import torch


class ZeroWgradMonitor:
    def __init__(self, model: torch.nn.Module):
        self.params = [(n, p) for n, p in model.named_parameters() if p.dim() == 2 and p.requires_grad]

    @torch.no_grad()
    def counts(self) -> dict[str, tuple[int, int]]:
        """name -> (exact zeros, entries) for every 2-D weight that has a gradient."""
        out = {}
        for n, p in self.params:
            if p.grad is not None:
                out[n] = (int((p.grad == 0).sum()), p.grad.numel())
        return out

    def summary(self) -> dict[str, float]:
        c = self.counts()
        zeros, total = sum(z for z, _ in c.values()), sum(t for _, t in c.values())
        worst = max(c.items(), key=lambda kv: kv[1][0] / max(kv[1][1], 1), default=(None, (0, 1)))
        return {"zero_wgrad_fraction": zeros / max(total, 1), "zero_wgrad_worst": worst[1][0] / max(worst[1][1], 1),
                "zero_wgrad_worst_name": worst[0]}
