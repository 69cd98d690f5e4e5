"""Guard for training a small part of a model on a frozen trunk: the frozen parameters take no gradient, own no
optimizer state (or, in the trainer's flat buffers, an update of learning-rate scale 0), and their bytes are checked
against a digest. Two users: the drafter head's training on a finished trunk (scripts/train_mtp.py) and
`TrainConfig.freeze_trunk`, the Copy-Paste head trained alone on the trunk that `init_from` loads (train/trainer.py):
the digests are then taken when the trunk has been loaded (`take_digests`), a step before that is refused
(`check_loaded`), every step checks that no frozen tensor has a gradient entry other than zero, and every save that the
trunk's bytes are the start's (reference: ced/train/freeze_trunk.py:1-56, 100-219; there the head is the add-on form,
whose sources are detached; here it is the base form, whose loss reaches the trunk's activations but, frozen, none of its
tensors)."""

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
        self.loaded = False

    def take_digests(self) -> None:
        """The trunk has been loaded: its bytes from now on."""
        self.digests = {n: _digest(p) for n, p in self.frozen.items()}
        self.loaded = True

    def summary(self) -> str:
        """One sha256 over the frozen tensors' names and digests, in name order."""
        h = hashlib.sha256()
        for n in sorted(self.digests):
            h.update(f"{n}|{self.digests[n]}|".encode())
        return h.hexdigest()

    def check_loaded(self) -> None:
        if not self.loaded:
            raise RuntimeError("freeze_trunk: a step before the trunk was loaded (init_from): a frozen random trunk would train a head on nothing")

    def check_grads(self) -> None:
        """No frozen tensor has a gradient (a view of a flat gradient buffer counts when it holds anything but zeros)."""
        bad = [n for n, p in self.frozen.items() if p.requires_grad or (p.grad is not None and bool(p.grad.ne(0).any()))]
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
