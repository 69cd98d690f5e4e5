"""Dense feed-forward blocks: SwiGLU `w_down(silu(w_gate x) * w_up x)` and ReLU-squared, bias-free
(reference: ced/model/mlp.py:12-60). On CUDA the gate and up projections run as one tcgen05 GEMM whose epilogue
applies the activation (`ops.swiglu_mlp`)."""

from __future__ import annotations

import torch
import torch.nn as nn
import torch.nn.functional as F

from .. import ops
from .linear import Linear


class SwiGLU(nn.Module):
    def __init__(self, d_model: int, hidden: int):
        super().__init__()
        self.w_gate = Linear(d_model, hidden)
        self.w_up = Linear(d_model, hidden)
        self.w_down = Linear(hidden, d_model)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return ops.swiglu_mlp(x, self.w_gate, self.w_up, self.w_down)


class ReLU2(nn.Module):
    def __init__(self, d_model: int, hidden: int):
        super().__init__()
        self.w_up = Linear(d_model, hidden)
        self.w_down = Linear(hidden, d_model)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return self.w_down(F.relu(self.w_up(x)).square())


def dense_ffn(d_model: int, hidden: int, activation: str) -> nn.Module:
    if activation == "swiglu":
        return SwiGLU(d_model, hidden)
    if activation == "relu2":
        return ReLU2(d_model, hidden)
    raise ValueError(f"ffn_activation {activation!r}: 'swiglu' or 'relu2'")
