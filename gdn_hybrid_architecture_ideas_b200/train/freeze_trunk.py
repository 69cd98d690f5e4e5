"""Guard for training a small part of a model on a frozen trunk: the frozen parameters take no gradient, own no
optimizer state, and their bytes are checked against a digest taken at start
(reference: ced/train/freeze_trunk.py:57-219, where the part that trains is the copy-paste head; here it guards the
drafter head's training on a finished trunk, scripts/train_mtp.py)."""

from __future__ import annotations

import hashlib

import torch


def _digest(t: torch.Tensor) -> str:
    return hashlib.sha256(t.detach().contiguous().cpu().view(torch.uint8).numpy().tobytes()).hexdigest()


class TrunkGuard:
    def __init__(self, model: torch.nn.Module, trainable_prefixes: tuple[str, ...]):
        self.frozen, self.trainable = {}, []
        for name, p in model.named_parameters():
            if any(name.startswith(pre) for pre in trainable_prefixes):
                self.trainable.append(name)
            else:
                p.requires_grad_(False)
                self.frozen[name] = p
        if not self.trainable:
            raise ValueError(f"freeze_trunk: no parameter matches the trainable prefixes {trainable_prefixes}")
        self.digests = {n: _digest(p) for n, p in self.frozen.items()}

    def check_grads(self) -> None:
        bad = [n for n, p in self.frozen.items() if p.grad is not None]
        if bad:
            raise RuntimeError(f"freeze_trunk: frozen parameters received gradients: {bad[:4]}")

    def check_optimizer(self, optimizer) -> None:
        ids = {id(p) for p in self.frozen.values()}
        for group in getattr(optimizer, "param_groups", []):
            held = [p for p in group["params"] if id(p) in ids]
            if held:
                raise RuntimeError(f"freeze_trunk: the optimizer holds {len(held)} frozen parameters")

    def check_values(self) -> None:
        changed = [n for n, p in self.frozen.items() if _digest(p) != self.digests[n]]
        if changed:
            raise RuntimeError(f"freeze_trunk: frozen parameters changed: {changed[:4]}")
