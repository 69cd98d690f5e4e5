"""Depth mixing over finished blocks (block-entry attention residuals).

A reader holds a (d,) pseudo-query w and an RMSNorm gain g, both zeros at init, and mixes a list of sources v_i per
position with weights softmax_i(w . RMSNorm(v_i)) (reference: ced/model/attn_res.py:406-482). With "block_entry" the
stack is cut into blocks of `full_attn_interval` layers; b_0 is the embedding output and b_n the sum of what block n's
sublayers added; block n >= 2 starts from the mix over [b_0 .. b_{n-1}] and the model output is the mix over all of
them (reference: ced/model/attn_res.py:670-797). On CUDA the mix is one kernel that reads every source once.
"""

from __future__ import annotations

from typing import Callable

import torch
import torch.nn as nn
import torch.nn.functional as F

from .. import ops
from .norms import RMSNorm

OWN_SEED_OFFSET = 0x1D3_2610_18809      # added to the run's seed for the address networks' generator (shared with the reference: equal starts)


class _Reader(nn.Module):
    """What every reader has: the key norm's gain and the number of softmaxes over the sources, one per contiguous slice
    of d / heads channels (`attn_res_heads`; a plain attribute, never in the state dict)."""

    def __init__(self, width: int, norm_eps: float, n_heads: int):
        super().__init__()
        if n_heads < 1 or width % n_heads:
            raise ValueError(f"model.encoder.attn_res_heads {n_heads}: a divisor of d_model {width}")
        self.heads = n_heads
        self.key_norm = RMSNorm(width, norm_eps)

    def mix(self, sources: list, query: torch.Tensor) -> torch.Tensor:
        gain, eps = self.key_norm.weight, self.key_norm.eps
        if self.heads == 1 and query.dim() == 1:
            return ops.depth_mix(sources, query, gain, eps)                  # the one-kernel read
        return ops.ref.depth_mix_heads(sources, query, gain, eps, self.heads)


class DepthQuery(_Reader):
    """The static reader: a (d,) pseudo-query, zeros at the start (a uniform read)."""

    def __init__(self, width: int, norm_eps: float, n_heads: int = 1):
        super().__init__(width, norm_eps, n_heads)
        self.register_parameter("query", nn.Parameter(torch.zeros(width)))

    def forward(self, sources: list) -> torch.Tensor:
        return self.mix(sources, self.query) if len(sources) > 1 else sources[0]


class OwnLinear(nn.Linear):
    """A biased Linear that takes no part in the model's general initialisation: it is zero when built (so building it
    draws nothing from the global generator) and marked `own_init`, which the model's N(0, init_std) pass skips. Its start
    comes later from `init_own_parameters`, out of a generator reserved for these layers; a model with such layers
    therefore starts with exactly the base weights of the model without them (reference: ced/model/ldm.py:88-101)."""

    own_init = True

    @torch.no_grad()
    def reset_parameters(self) -> None:
        self.weight.zero_()
        if self.bias is not None:
            self.bias.zero_()

    def at(self, x: torch.Tensor) -> torch.Tensor:
        """The layer applied with its tensors cast to x's dtype (the networks run in the stream's dtype under autocast too)."""
        return F.linear(x, self.weight.to(x.dtype), self.bias.to(x.dtype))


class AddressNet(nn.Module):
    """A small per-position network that turns the stream into an address: RMSNorm -> `inp` (d -> hidden) -> SiLU ->
    `head` (hidden -> out), plus, when `gates` > 0, a second head `gate` (hidden -> gates) of gate logits.

    Start (`reset_own`): `inp` ~ N(0, std); `head` ~ N(0, std), or zero with `zero_head` (a token-dependent depth query
    must start as the zero pseudo-query, i.e. a uniform read); every bias and the whole gate head zero (gates start
    open at sigmoid(0)). Draw order: inp.weight, then head.weight (reference: ced/model/ldm.py:103-137)."""

    def __init__(self, width: int, hidden: int, out: int, norm_eps: float, gates: int = 0, zero_head: bool = True):
        super().__init__()
        self.zero_head = zero_head
        self.norm = RMSNorm(width, norm_eps)
        self.inp, self.head = OwnLinear(width, hidden), OwnLinear(hidden, out)
        self.gate = OwnLinear(hidden, gates) if gates > 0 else None

    @torch.no_grad()
    def reset_own(self, g: torch.Generator, std: float) -> None:
        for name, drawn in (("inp", True), ("head", not self.zero_head), ("gate", False)):
            layer = getattr(self, name)
            if layer is None:
                continue
            layer.reset_parameters()
            if drawn:
                layer.weight.copy_(torch.randn(layer.weight.shape, generator=g, dtype=torch.float32, device="cpu") * std)

    def hidden(self, x: torch.Tensor) -> torch.Tensor:
        return F.silu(self.inp.at(self.norm(x, out_dtype=x.dtype)))

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return self.head.at(self.hidden(x))

    def both(self, x: torch.Tensor):
        """(address, gate logits) from one pass through the trunk."""
        h = self.hidden(x)
        return self.head.at(h), self.gate.at(h)


def init_own_parameters(model: nn.Module, std: float) -> int:
    """Starts every AddressNet of `model`, in module order, from ONE CPU generator seeded with the run's seed + a fixed
    offset; the global generator is neither read nor advanced (reference: ced/model/ldm.py:423-438)."""
    gen, count = None, 0
    for m in model.modules():
        if not isinstance(m, AddressNet):
            continue
        if gen is None:
            gen = torch.Generator().manual_seed((torch.initial_seed() + OWN_SEED_OFFSET) % (1 << 63))
        m.reset_own(gen, std)
        count += 1
    return count


class TokenQuery(_Reader):
    """A block-entry reader whose query is a function of the stream at the read (`attn_res_query: token`): the key norm
    of a DepthQuery, and in place of the (d,) pseudo-query an address network whose head starts at zero, so the read
    starts uniform as the static reader does (reference: ced/model/attn_res.py:422-437)."""

    def __init__(self, width: int, norm_eps: float, hidden: int, n_heads: int = 1):
        super().__init__(width, norm_eps, n_heads)
        self.net = AddressNet(width, hidden, width, norm_eps)

    def forward(self, sources: list, src: torch.Tensor) -> torch.Tensor:
        return self.mix(sources, self.net(src)) if len(sources) > 1 else sources[0]


def reader_factory(width: int, norm_eps: float, n_heads: int = 1, query_hidden: int = 0) -> Callable[[], _Reader]:
    """Builds block-entry readers of one kind: token-dependent when query_hidden > 0, static otherwise."""
    if query_hidden:
        return lambda: TokenQuery(width, norm_eps, query_hidden, n_heads)
    return lambda: DepthQuery(width, norm_eps, n_heads)


class EntryLayer(nn.Module):
    """What a layer that opens or closes a block holds: `entry` (reader of the block's input; first layer of blocks
    2..N) and `out` (reader of the model output; last layer of the stack). `token`: the readers take the stream at the read."""

    def __init__(self, make: Callable[[], _Reader], token: bool, opens: bool, closes: bool, last: bool):
        super().__init__()
        self.token, self.closes = token, closes
        for slot, wanted in (("entry", opens), ("out", last)):
            self.add_module(slot, make() if wanted else None)


class LayerQueries(nn.Module):
    """Depth attention of both sublayers of one encoder layer ("block": every sublayer reads the finished blocks and the
    current block's partial sum): `pre_mixer` (None in layer 0, whose mixer reads the embedding alone) and `pre_mlp`;
    `first`: the layer opens a block; `out`: only in the last layer, the read of the model output
    (reference: ced/model/attn_res.py:439-452)."""

    def __init__(self, width: int, norm_eps: float, first: bool, has_mixer_query: bool, last: bool):
        super().__init__()
        self.first = first
        for slot, wanted in (("pre_mixer", has_mixer_query), ("pre_mlp", True), ("out", last)):
            self.add_module(slot, DepthQuery(width, norm_eps) if wanted else None)
