"""Bias-free linear layer whose GPU path is the framework's own tcgen05 GEMM.

The parameter is a plain `weight` (out, in), as nn.Linear's, so state dicts match the reference's
(every projection there is `nn.Linear(..., bias=False)`). `weight_lp` is an optional bfloat16 shadow of the weight
kept by the optimizer's fused update (a view into the flat low-precision parameter buffer): when present the GEMM
reads it instead of casting the master weight every step. `precision` names a block-scaled low-precision recipe
("mxfp8" / "nvfp4") applied in training mode only, as the reference's FP8Linear / NVFP4Linear do
(ced/model/fp8.py:347-367, ced/model/nvfp4.py:555).
"""

from __future__ import annotations

import torch
import torch.nn as nn

from .. import ops


class Linear(nn.Linear):
    def __init__(self, in_features: int, out_features: int):
        super().__init__(in_features, out_features, bias=False)
        self.weight_lp: torch.Tensor | None = None
        self.precision: str = "bf16"
        self.lowp = None  # recipe state (ops.lowp.Recipe) when precision != "bf16"
        self.tp = None           # parallel.tensor_parallel.TensorParallel when this projection is sharded over ranks
        self.tp_mode = None      # "column" (output features sharded, token-sharded input) or "row" (input features sharded)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return ops.linear(x, self)

    def rows(self, lo: int, hi: int) -> "RowView":
        return RowView(self, lo, hi)


class RowView:
    """Rows [lo, hi) of a Linear's weight as a projection of their own (the write/query mixes project different
    inputs through different row ranges of in_proj_qkv)."""

    def __init__(self, base: Linear, lo: int, hi: int):
        self.base, self.lo, self.hi = base, lo, hi

    @property
    def weight(self):
        return self.base.weight[self.lo:self.hi]

    @property
    def weight_lp(self):
        lp = self.base.weight_lp
        return None if lp is None else lp[self.lo:self.hi]

    @property
    def precision(self):
        return self.base.precision

    @property
    def tp(self):
        return self.base.tp

    @property
    def tp_mode(self):
        return self.base.tp_mode

    @property
    def lowp(self):
        return self.base.lowp

    @property
    def training(self):
        return self.base.training

    def __call__(self, x):
        return ops.linear(x, self)
