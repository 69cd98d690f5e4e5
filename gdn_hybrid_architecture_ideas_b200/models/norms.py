"""Zero-centred RMSNorm and the gated output norm of a GDN layer.

y = x * rsqrt(mean(x^2) + eps) * (1 + w), w initialised to 0, computed in at least float32 and returned in the
input dtype (reference: ced/model/norms.py:51-94). On a CUDA tensor the work is one fused kernel
(`ops.rmsnorm` / `ops.gated_rmsnorm`); elsewhere the PyTorch statement of the same formula.
"""

from __future__ import annotations

import torch
import torch.nn as nn

from .. import ops


class RMSNorm(nn.Module):
    GAINS = ("channel", "scalar")

    def __init__(self, dim: int, eps: float = 1e-6, gain: str = "channel"):
        super().__init__()
        if gain not in self.GAINS:
            raise ValueError(f"RMSNorm gain {gain!r}: one of {self.GAINS}")
        self.eps = eps
        self.dim = dim
        self.weight = nn.Parameter(torch.zeros(dim if gain == "channel" else 1))

    def forward(self, x: torch.Tensor, out_dtype: torch.dtype | None = None) -> torch.Tensor:
        return ops.rmsnorm(x, self.weight, self.eps, out_dtype=out_dtype)


class GatedRMSNorm(RMSNorm):
    """RMSNorm over the value-head dimension times act(z), act = SiLU or sigmoid."""

    def __init__(self, dim: int, eps: float = 1e-6, gate: str = "silu", gain: str = "channel"):
        super().__init__(dim, eps, gain=gain)
        if gate not in ("silu", "sigmoid"):
            raise ValueError(f"unknown GDN output gate {gate!r}")
        self.gate = gate

    def forward(self, x: torch.Tensor, z: torch.Tensor, out_dtype: torch.dtype | None = None) -> torch.Tensor:
        return ops.gated_rmsnorm(x, z, self.weight, self.eps, self.gate, out_dtype=out_dtype)


def round_stream(x: torch.Tensor) -> torch.Tensor:
    """x held at bfloat16 precision in its own dtype, value and gradient alike (residual_dtype "bf16";
    reference: ced/model/norms.py:15-48)."""
    return _RoundBf16.apply(x)


class _RoundBf16(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x):
        return x.to(torch.bfloat16).to(x.dtype)

    @staticmethod
    def backward(ctx, g):
        return g.to(torch.bfloat16).to(g.dtype)
