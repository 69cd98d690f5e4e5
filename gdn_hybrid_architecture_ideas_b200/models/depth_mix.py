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


OWN_SEED_OFFSET = 0x1D3_2610_18809


class OwnLinear(nn.Linear):
    """A Linear (with bias) the model's N(0, init_std) pass leaves alone: zeros at construction (no draw from the global
    generator), then started by `init_own_parameters` from a generator of its own, so every other tensor starts as in
    the model without it (reference: ced/model/ldm.py:88-101)."""

    own_init = True

    def reset_parameters(self) -> None:
        with torch.no_grad():
            self.weight.zero_()
            if self.bias is not None:
                self.bias.zero_()


class AddressNet(nn.Module):
    """RMSNorm -> Linear(d, hidden) -> SiLU -> an address head Linear(hidden, out) and, with `gates`, a gate head
    Linear(hidden, gates). zero_head (a token-dependent query, which must start as the zero pseudo-query): the head
    starts at zero; otherwise it is drawn as the backbone's linears are. The gate head starts at zero
    (reference: ced/model/ldm.py:103-137)."""

    def __init__(self, d: int, hidden: int, out: int, eps: float, gates: int = 0, zero_head: bool = True):
        super().__init__()
        self.norm = RMSNorm(d, eps)
        self.inp = OwnLinear(d, hidden)
        self.head = OwnLinear(hidden, out)
        self.gate = OwnLinear(hidden, gates) if gates else None
        self.zero_head = zero_head

    @torch.no_grad()
    def reset_own(self, g: torch.Generator, std: float) -> None:
        draw = lambda t: t.copy_(torch.randn(t.shape, generator=g, dtype=torch.float32, device="cpu") * std)
        draw(self.inp.weight)
        self.inp.bias.zero_()
        if self.zero_head:
            self.head.weight.zero_()
        else:
            draw(self.head.weight)
        self.head.bias.zero_()
        if self.gate is not None:
            self.gate.weight.zero_()
            self.gate.bias.zero_()

    def hidden(self, x: torch.Tensor) -> torch.Tensor:
        lin = torch.nn.functional.linear
        return torch.nn.functional.silu(lin(self.norm(x, out_dtype=x.dtype), self.inp.weight.to(x.dtype), self.inp.bias.to(x.dtype)))

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return torch.nn.functional.linear(self.hidden(x), self.head.weight.to(x.dtype), self.head.bias.to(x.dtype))

    def both(self, x: torch.Tensor):
        """(address, gate logits)."""
        hid, lin = self.hidden(x), torch.nn.functional.linear
        return lin(hid, self.head.weight.to(x.dtype), self.head.bias.to(x.dtype)), lin(hid, self.gate.weight.to(x.dtype), self.gate.bias.to(x.dtype))


def init_own_parameters(model: nn.Module, std: float) -> int:
    """Start every address network, in module order, from a CPU generator seeded with torch.initial_seed() + a fixed
    offset; the global generator is not drawn (reference: ced/model/ldm.py:423-438)."""
    nets = [m for m in model.modules() if isinstance(m, AddressNet)]
    if nets:
        g = torch.Generator().manual_seed((torch.initial_seed() + OWN_SEED_OFFSET) % (1 << 63))
        for m in nets:
            m.reset_own(g, std)
    return len(nets)


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
