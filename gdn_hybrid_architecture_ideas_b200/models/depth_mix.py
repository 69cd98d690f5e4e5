"""Depth mixing over finished blocks (block-entry attention residuals).

A reader holds a (d,) pseudo-query w and an RMSNorm gain g, both zeros at init, and mixes a list of sources v_i per
position with weights softmax_i(w . RMSNorm(v_i)) (reference: ced/model/attn_res.py:406-482). With "block_entry" the
stack is cut into blocks of `full_attn_interval` layers; b_0 is the embedding output and b_n the sum of what block n's
sublayers added; block n >= 2 starts from the mix over [b_0 .. b_{n-1}] and the model output is the mix over all of
them (reference: ced/model/attn_res.py:670-797). On CUDA the mix is one kernel that reads every source once.
"""

from __future__ import annotations

import torch
import torch.nn as nn

from .. import ops
from .norms import RMSNorm


class DepthQuery(nn.Module):
    """heads: the number of softmaxes over the sources, one per contiguous slice of d / heads channels
    (`attn_res_heads`; a plain attribute, never in the state dict). 1 is the one-kernel read."""

    def __init__(self, d: int, eps: float, heads: int = 1):
        super().__init__()
        if heads < 1 or d % heads:
            raise ValueError(f"model.encoder.attn_res_heads {heads}: a divisor of d_model {d}")
        self.query = nn.Parameter(torch.zeros(d))
        self.key_norm = RMSNorm(d, eps)
        self.heads = heads

    def forward(self, sources: list) -> torch.Tensor:
        if len(sources) == 1:
            return sources[0]
        if self.heads > 1:
            return ops.ref.depth_mix_heads(sources, self.query, self.key_norm.weight, self.key_norm.eps, self.heads)
        return ops.depth_mix(sources, self.query, self.key_norm.weight, self.key_norm.eps)


class EntryLayer(nn.Module):
    """What a layer that opens or closes a block holds: `entry` (reader of the block's input; first layer of blocks
    2..N) and `out` (reader of the model output; last layer of the stack)."""

    def __init__(self, d: int, eps: float, entry: bool, closes: bool, last: bool, heads: int = 1):
        super().__init__()
        self.entry = DepthQuery(d, eps, heads) if entry else None
        self.closes = closes
        self.out = DepthQuery(d, eps, heads) if last else None


class LayerQueries(nn.Module):
    """Depth attention of both sublayers of one encoder layer ("block": every sublayer reads the finished blocks and the
    current block's partial sum): `pre_mixer` (None in layer 0, whose mixer reads the embedding alone) and `pre_mlp`;
    `first`: the layer opens a block; `out`: only in the last layer, the read of the model output
    (reference: ced/model/attn_res.py:439-452)."""

    def __init__(self, d: int, eps: float, first: bool, has_mixer_query: bool, last: bool):
        super().__init__()
        self.first = first
        self.pre_mixer = DepthQuery(d, eps) if has_mixer_query else None
        self.pre_mlp = DepthQuery(d, eps)
        self.out = DepthQuery(d, eps) if last else None
