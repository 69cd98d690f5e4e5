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


OWN_SEED_OFFSET = 0x1D3_2610_18809      # added to the run's seed for the address networks' generator (shared with the reference: equal starts)


class OwnLinear(nn.Linear):
    """A biased Linear that takes no part in the model's general initialisation: it is zero when built (so building it
    draws nothing from the global generator) and marked `own_init`, which the model's N(0, init_std) pass skips. Its start
    comes later from `init_own_parameters`, out of a generator reserved for these layers; a model with such layers
    therefore starts with exactly the base weights of the model without them (reference: ced/model/ldm.py:88-101)."""

    own_init = True

    def reset_parameters(self) -> None:
        for t in (self.weight, self.bias):
            if t is not None:
                nn.init.zeros_(t)


def _affine(layer: nn.Linear, x: torch.Tensor) -> torch.Tensor:
    """layer(x) with the layer's tensors cast to x's dtype (the networks run in the stream's dtype under autocast too)."""
    return torch.nn.functional.linear(x, layer.weight.to(x.dtype), layer.bias.to(x.dtype))


class AddressNet(nn.Module):
    """A small per-position network that turns the stream into an address: RMSNorm -> `inp` (d -> hidden) -> SiLU ->
    `head` (hidden -> out), plus, when `gates` > 0, a second head `gate` (hidden -> gates) of gate logits.

    Start (`reset_own`): `inp` ~ N(0, std); `head` ~ N(0, std), or zero with `zero_head` (a token-dependent depth query
    must start as the zero pseudo-query, i.e. a uniform read); every bias and the whole gate head zero (gates start
    open at sigmoid(0)). Draw order: inp.weight, then head.weight (reference: ced/model/ldm.py:103-137)."""

    def __init__(self, d: int, hidden: int, out: int, eps: float, gates: int = 0, zero_head: bool = True):
        super().__init__()
        self.norm = RMSNorm(d, eps)
        self.inp = OwnLinear(d, hidden)
        self.head = OwnLinear(hidden, out)
        self.gate = OwnLinear(hidden, gates) if gates else None
        self.zero_head = zero_head

    @torch.no_grad()
    def reset_own(self, g: torch.Generator, std: float) -> None:
        for layer in (self.inp, self.head, self.gate):
            if layer is not None:
                layer.reset_parameters()
        drawn = [self.inp.weight] + ([] if self.zero_head else [self.head.weight])
        for w in drawn:
            w.copy_(torch.randn(w.shape, generator=g, dtype=torch.float32, device="cpu") * std)

    def hidden(self, x: torch.Tensor) -> torch.Tensor:
        return torch.nn.functional.silu(_affine(self.inp, self.norm(x, out_dtype=x.dtype)))

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return _affine(self.head, self.hidden(x))

    def both(self, x: torch.Tensor):
        """(address, gate logits) from one pass through the trunk."""
        h = self.hidden(x)
        return _affine(self.head, h), _affine(self.gate, h)


def init_own_parameters(model: nn.Module, std: float) -> int:
    """Starts every AddressNet of `model`, in module order, from ONE CPU generator seeded with the run's seed + a fixed
    offset; the global generator is neither read nor advanced (reference: ced/model/ldm.py:423-438)."""
    found = [m for m in model.modules() if isinstance(m, AddressNet)]
    if found:
        gen = torch.Generator().manual_seed((torch.initial_seed() + OWN_SEED_OFFSET) % (1 << 63))
        for net in found:
            net.reset_own(gen, std)
    return len(found)


class TokenQuery(nn.Module):
    """A block-entry reader whose query is a function of the stream at the read (`attn_res_query: token`): the key norm
    of a DepthQuery, and in place of the (d,) pseudo-query an address network whose head starts at zero, so the read
    starts uniform as the static reader does (reference: ced/model/attn_res.py:422-437)."""

    def __init__(self, d: int, eps: float, hidden: int, heads: int = 1):
        super().__init__()
        self.key_norm = RMSNorm(d, eps)
        self.net = AddressNet(d, hidden, d, eps)
        self.heads = heads

    def forward(self, sources: list, src: torch.Tensor) -> torch.Tensor:
        if len(sources) == 1:
            return sources[0]
        return ops.ref.depth_mix_heads(sources, self.net(src), self.key_norm.weight, self.key_norm.eps, self.heads)


class EntryLayer(nn.Module):
    """What a layer that opens or closes a block holds: `entry` (reader of the block's input; first layer of blocks
    2..N) and `out` (reader of the model output; last layer of the stack)."""

    def __init__(self, d: int, eps: float, entry: bool, closes: bool, last: bool, heads: int = 1, query_hidden: int = 0):
        super().__init__()
        reader = (lambda: TokenQuery(d, eps, query_hidden, heads)) if query_hidden else (lambda: DepthQuery(d, eps, heads))
        self.entry = reader() if entry else None
        self.closes = closes
        self.out = reader() if last else None
        self.token = bool(query_hidden)      # the readers take the stream at the read


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
