"""Static buffers with guard bands: every buffer of a decode engine is a view into the middle of its own allocation,
with a band of a fixed byte pattern before and after it. A kernel (or an index computed on the host) that writes past
either end of a buffer lands in a band instead of in a neighbouring allocation, and `check()` finds it after the run and
names the buffer and the side. The views' addresses never change after allocation, which is what a captured CUDA graph
needs. The bands cost 2 x GUARD bytes per buffer and nothing at run time; checking reads them back (a device
synchronisation), so it is done between runs, not per step.

This is the host-checked stand-in for a memory checker on the device side: it sees writes, not reads, and only within
GUARD bytes of a buffer's ends.
"""

from __future__ import annotations

import math

import torch

GUARD = 512                 # bytes on each side; a multiple of every element size and of the 256-byte alignment kernels assume
PATTERN = 0xA5


class GuardOverrun(RuntimeError):
    """A guard band no longer holds its pattern."""


class GuardedBuffers:
    def __init__(self, device, guard: int = GUARD):
        if guard % 256:
            raise ValueError("the guard width is a multiple of 256 bytes")
        self.device, self.guard = torch.device(device), guard
        self.raw: dict[str, torch.Tensor] = {}
        self.size: dict[str, int] = {}

    def zeros(self, name: str, shape, dtype) -> torch.Tensor:
        return self._make(name, shape, dtype, 0)

    def full(self, name: str, shape, value, dtype) -> torch.Tensor:
        return self._make(name, shape, dtype, value)

    def _make(self, name, shape, dtype, value) -> torch.Tensor:
        if name in self.raw:
            raise ValueError(f"buffer {name!r} exists")
        shape = tuple(int(s) for s in (shape if isinstance(shape, (tuple, list, torch.Size)) else (shape,)))
        item = torch.empty(0, dtype=dtype).element_size()
        n = math.prod(shape) * item
        padded = -(-max(n, 1) // 256) * 256                      # the trailing band starts on a 256-byte boundary
        raw = torch.full((self.guard + padded + self.guard,), PATTERN, dtype=torch.uint8, device=self.device)
        body = raw[self.guard:self.guard + n].view(dtype).view(shape)
        body.fill_(value)
        self.raw[name], self.size[name] = raw, n
        return body

    def bytes(self) -> int:
        return sum(self.size.values())

    def check(self) -> None:
        """Raises GuardOverrun naming every buffer whose leading or trailing band changed (the slack between a buffer's end
        and the next 256-byte boundary belongs to the trailing band)."""
        bad = []
        for name, raw in self.raw.items():
            n = self.size[name]
            lead, trail = raw[:self.guard], raw[self.guard + n:]
            if bool((lead != PATTERN).any()):
                at = int((lead != PATTERN).nonzero()[-1]) - self.guard
                bad.append(f"{name}: written {-at} bytes before its start")
            if bool((trail != PATTERN).any()):
                at = int((trail != PATTERN).nonzero()[0])
                bad.append(f"{name}: written {at} bytes past its end")
        if bad:
            raise GuardOverrun("; ".join(bad))
