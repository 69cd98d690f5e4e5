"""Linear depth memory with a delta-rule write (`model.encoder.attn_res: ldm`).

Instead of mixing earlier blocks' outputs back into the stream, every POSITION carries a small associative memory along
the depth of the network: G groups, each a (K, D) matrix with K = ldm_key_dim and D = d_model / G. Sublayers write what
they added to the stream into it and read from it before they run. Nothing in the memory mixes positions, so cached
generation needs no memory state: a new token rebuilds its own memory on its way up the stack.

Along the depth (x is the stream, f a sublayer: each layer's mixer, then its MLP):

    M   = write_0(k(h0), v = h0)                       the embedding output is the first thing remembered
    r   = M^T (gain * gate * q)                         per group; q unit (G, K), gate = 2 sigmoid(.) from the READ net at x
    d   = f(x + r);   x <- x + d                        the read feeds the sublayer, it is not added to the stream
    M   = lam (I - w k k^T) M + w k d^T                 per group; k unit, w = 2 sigmoid(.) from the WRITE net at the new x
    ... after the last layer the final norm sees x + r_out (the output's own read).

lam = sigmoid(lam_logit) per group is the forgetting along depth (starts at 0.99); w and lam are floored at 1e-6. The
addresses come from `AddressNet`s (models/depth_mix.py); their gate heads start at zero, so every gate starts at 1.
Memory arithmetic runs in float32 or wider with autocast off. Reference: ced/model/ldm.py:1-62, 149-259, 413-452.
"""

from __future__ import annotations

import math

import torch
import torch.nn as nn
import torch.nn.functional as F

from .depth_mix import AddressNet

LAMBDA_INIT = 0.99
EPS = 1e-6


def address_hidden(d: int, value: int) -> int:
    """Width of the address networks' hidden layer: the configured value, else d / 32."""
    return value or max(1, d // 32)


def state_dtype(x: torch.Tensor) -> torch.dtype:
    return torch.promote_types(x.dtype, torch.float32)


# ---------------------------------------------------------------------------------------------------- memory arithmetic
# M: (B, L, G, K, D); keys / queries: (B, L, G, K); values: (B, L, G, D). All in the memory's dtype, autocast off.

def _unit_rows(addr: torch.Tensor, groups: int, key_dim: int) -> torch.Tensor:
    return F.normalize(addr.unflatten(-1, (groups, key_dim)), dim=-1, eps=EPS)


def memory_read(M: torch.Tensor, query: torch.Tensor) -> torch.Tensor:
    """M^T query per group -> (B, L, G, D)."""
    return torch.einsum("blgkd,blgk->blgd", M, query)


def delta_write(M: torch.Tensor | None, key: torch.Tensor, value: torch.Tensor, weight: torch.Tensor, keep: torch.Tensor | None) -> torch.Tensor:
    """keep (I - w k k^T) M + w k v^T per group; M None (with keep None): the write into an empty memory, w k v^T."""
    if M is None:
        return torch.einsum("blgk,blgd->blgkd", key * weight[..., None], value)
    kept = M * keep[:, None, None]
    seen = memory_read(kept, key)                                   # what the memory already answers for this key
    return kept + torch.einsum("blgk,blgd->blgkd", key * weight[..., None], value - seen)


class _Port(nn.Module):
    """An address network and the shape bookkeeping shared by reads and writes."""

    def __init__(self, d: int, groups: int, key_dim: int, hidden: int, eps: float):
        super().__init__()
        self.groups, self.key_dim = groups, key_dim
        self.net = AddressNet(d, hidden, groups * key_dim, eps, gates=groups, zero_head=False)

    def _address(self, x: torch.Tensor):
        """(unit keys (B, L, G, K), gate 2 sigmoid (B, L, G)) in the memory's dtype."""
        addr, gate = self.net.both(x)
        dt = state_dtype(x)
        with torch.autocast(x.device.type, enabled=False):
            return _unit_rows(addr.to(dt), self.groups, self.key_dim), 2.0 * torch.sigmoid(gate.to(dt))


class LdmRead(_Port):
    def __init__(self, d: int, groups: int, key_dim: int, hidden: int, eps: float):
        super().__init__(d, groups, key_dim, hidden, eps)
        self.read_gain = nn.Parameter(torch.ones(groups))

    def query(self, x: torch.Tensor) -> torch.Tensor:
        key, gate = self._address(x)
        with torch.autocast(x.device.type, enabled=False):
            return key * (gate * self.read_gain.to(key.dtype))[..., None]

    def read(self, M: torch.Tensor, x: torch.Tensor) -> torch.Tensor:
        """The read as a (B, L, d) tensor in the stream's dtype."""
        q = self.query(x)
        with torch.autocast(x.device.type, enabled=False):
            return memory_read(M, q).flatten(-2).to(x.dtype)


class LdmWrite(_Port):
    """`first`: the embedding's write into the still-empty memory; it has no forgetting (there is nothing to forget)."""

    def __init__(self, d: int, groups: int, key_dim: int, hidden: int, eps: float, first: bool = False):
        super().__init__(d, groups, key_dim, hidden, eps)
        self.lam_logit = None if first else nn.Parameter(torch.full((groups,), math.log(LAMBDA_INIT / (1.0 - LAMBDA_INIT))))

    def _observation(self, x: torch.Tensor, v: torch.Tensor):
        key, gate = self._address(x)
        with torch.autocast(x.device.type, enabled=False):
            return key, v.to(key.dtype).unflatten(-1, (self.groups, -1)), gate.clamp_min(EPS)

    def first(self, h: torch.Tensor) -> torch.Tensor:
        key, value, w = self._observation(h, h)
        with torch.autocast(h.device.type, enabled=False):
            return delta_write(None, key, value, w, None)

    def write(self, M: torch.Tensor, x: torch.Tensor, v: torch.Tensor) -> torch.Tensor:
        key, value, w = self._observation(x, v)
        with torch.autocast(x.device.type, enabled=False):
            keep = torch.sigmoid(self.lam_logit.to(key.dtype)).clamp_min(EPS)
            return delta_write(M, key, value, w, keep)


class LdmLayer(nn.Module):
    """One encoder layer's ports (its `attn_res`): a read and a write for each of its two sublayers; layer 0 also holds
    the embedding's write, the last layer the output's read. Attribute order is the state dict's order."""

    def __init__(self, d: int, groups: int, key_dim: int, hidden: int, eps: float, first: bool, last: bool):
        super().__init__()
        port = (d, groups, key_dim, hidden, eps)
        self.embed_write = LdmWrite(*port, first=True) if first else None
        self.mixer_read, self.mixer_write = LdmRead(*port), LdmWrite(*port)
        self.mlp_read, self.mlp_write = LdmRead(*port), LdmWrite(*port)
        self.out_read = LdmRead(*port) if last else None


def build(cfg, layers) -> None:
    enc, d = cfg.encoder, cfg.d_model
    if d % enc.ldm_groups:
        raise ValueError(f"model.encoder.ldm_groups {enc.ldm_groups} must divide d_model {d}")
    hidden = address_hidden(d, enc.ldm_hidden)
    for i, layer in enumerate(layers):
        layer.attn_res = LdmLayer(d, enc.ldm_groups, enc.ldm_key_dim, hidden, cfg.norm_eps, first=i == 0, last=i == len(layers) - 1)


def _sublayer(layer, which: str, h, ctx, cache, need_state):
    """(scaled, normed branch output in the stream's dtype, cache entry) of the mixer or the MLP on input h."""
    if which == "mlp":
        out, entry = layer.mlp(layer.mlp_in_norm(h)), None
        norm = layer.mlp_out_norm
    else:
        extra = {"need_state": need_state} if layer.kind == "gdn" else {}
        out, entry = layer.mixer(layer.mixer_in_norm(h), ctx, cache, **extra)
        norm = layer.mixer_out_norm
    return (layer.residual_scale * norm(out, out_dtype=h.dtype)).to(h.dtype), entry


def layer_forward(layer, x, M, ctx, cache, need_state: bool = True):
    """One layer with its memory traffic. M is None on entry to layer 0, which writes the embedding first. Returns
    (x, M, cache entry); from the last layer x comes back with the output's read added, ready for the final norm."""
    ports = layer.attn_res
    if ports.embed_write is not None:
        M = ports.embed_write.first(x)
    entry = None
    for which, reader, writer in (("mixer", ports.mixer_read, ports.mixer_write), ("mlp", ports.mlp_read, ports.mlp_write)):
        delta, got = _sublayer(layer, which, x + reader.read(M, x), ctx, cache, need_state)
        entry = got if which == "mixer" else entry
        x = x + delta
        M = writer.write(M, x, delta)
    if ports.out_read is not None:
        x = x + ports.out_read.read(M, x)
    return x, M, entry


def parameter_count(d: int, n_layers: int, groups: int, key_dim: int, hidden: int) -> int:
    """Parameters the memory adds to a model of n_layers: 2 n + 1 reads and as many writes (the embedding's included),
    each an address network; every read a gain per group, every write but the first a forgetting logit per group."""
    net = d + (d + 1) * hidden + (hidden + 1) * groups * (key_dim + 1)
    ports = 2 * n_layers + 1
    return ports * (2 * net + groups) + (ports - 1) * groups
