"""Linear Depth Memory with the delta-rule write (`model.encoder.attn_res: ldm`).

The residual stream stays as it is (x <- x + delta). Beside it each position carries a memory M of G groups, each a
(K, D) matrix (K = ldm_key_dim, D = d_model / G):

    the embedding output h0 is the first write: M_0 = write(0, k(h0), v = h0)
    before every sublayer f (the mixer, then the MLP, of every layer):
        r = per group M^T (gamma g q)        q (G, K) unit per group and g = 2 sigmoid(.) from the read's address network of x
        delta = f(x + r);  x = x + delta     the read is not added to the stream
        M = write(M, k, v = delta)           k (G, K) unit and w = 2 sigmoid(.) from the write's address network of the new x
    the final norm reads x + r_out, the output's own read.

    write: k_w = sqrt(w) k, v_w = sqrt(w) v (w floored at eps), A = lam M (lam = sigmoid(logit) floored at eps),
           M' = A + k_w (v_w - A^T k_w)^T, that is M' = lam (I - w k k^T) M + w k v^T.

Address networks: RMSNorm -> Linear(d, hidden) -> SiLU -> an address head (G K) and a gate head (G); hidden =
ldm_hidden or d_model // 32. Start: first Linear and address heads N(0, init_std) from a generator of their own, gate
heads zero (every gate 1), read gains 1, forgetting logits logit(0.99). The memory, its writes and reads, the norms
and gates run in >= float32 with autocast off. The memory is per position: nothing in it mixes positions, so a cached
chunk carries nothing of it (reference: ced/model/ldm.py:1-62, 149-259, 413-452).
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
    return value if value else max(1, d // 32)


def state_dtype(x: torch.Tensor) -> torch.dtype:
    return torch.promote_types(x.dtype, torch.float32)


def _no_autocast(x: torch.Tensor):
    return torch.autocast(x.device.type, enabled=False)


class LdmRead(nn.Module):
    def __init__(self, d: int, groups: int, key_dim: int, hidden: int, eps: float):
        super().__init__()
        self.groups, self.key_dim = groups, key_dim
        self.net = AddressNet(d, hidden, groups * key_dim, eps, gates=groups, zero_head=False)
        self.read_gain = nn.Parameter(torch.ones(groups))

    def query(self, x: torch.Tensor) -> torch.Tensor:
        """gamma g q (B, L, G, K) in the memory's dtype."""
        addr, gate = self.net.both(x)
        dt = state_dtype(x)
        with _no_autocast(x):
            q = F.normalize(addr.to(dt).unflatten(-1, (self.groups, self.key_dim)), dim=-1, eps=EPS)
            return q * (2.0 * torch.sigmoid(gate.to(dt)) * self.read_gain.to(dt))[..., None]

    def read(self, M: torch.Tensor, x: torch.Tensor) -> torch.Tensor:
        q = self.query(x)
        with _no_autocast(x):
            r = (M * q[..., None]).sum(-2)
        return r.flatten(-2).to(x.dtype)


class LdmWrite(nn.Module):
    """first: the embedding's write into the empty memory, which has no forgetting logit (it would multiply zeros)."""

    def __init__(self, d: int, groups: int, key_dim: int, hidden: int, eps: float, first: bool = False):
        super().__init__()
        self.groups, self.key_dim = groups, key_dim
        self.net = AddressNet(d, hidden, groups * key_dim, eps, gates=groups, zero_head=False)
        self.lam_logit = None if first else nn.Parameter(torch.full((groups,), math.log(LAMBDA_INIT / (1.0 - LAMBDA_INIT))))

    def observation(self, x: torch.Tensor, v: torch.Tensor):
        addr, gate = self.net.both(x)
        dt = state_dtype(x)
        with _no_autocast(x):
            k = F.normalize(addr.to(dt).unflatten(-1, (self.groups, self.key_dim)), dim=-1, eps=EPS)
            s = (2.0 * torch.sigmoid(gate.to(dt))).clamp_min(EPS).sqrt()
            lam = None if self.lam_logit is None else torch.sigmoid(self.lam_logit.to(dt)).clamp_min(EPS)
            return k * s[..., None], v.to(dt).unflatten(-1, (self.groups, -1)) * s[..., None], lam

    def first(self, h: torch.Tensor) -> torch.Tensor:
        kw, vw, _ = self.observation(h, h)
        with _no_autocast(h):
            return kw[..., None] * vw[..., None, :]

    def write(self, M: torch.Tensor, x: torch.Tensor, v: torch.Tensor) -> torch.Tensor:
        kw, vw, lam = self.observation(x, v)
        with _no_autocast(x):
            A = M * lam[:, None, None]
            return A + kw[..., None] * (vw - (A * kw[..., None]).sum(-2))[..., None, :]


class LdmLayer(nn.Module):
    """What one encoder layer holds of the memory (its `attn_res`): the read and write of its two sites; in layer 0
    also the embedding write, in the last layer also the output's read."""

    def __init__(self, d: int, groups: int, key_dim: int, hidden: int, eps: float, first: bool, last: bool):
        super().__init__()
        args = (d, groups, key_dim, hidden, eps)
        self.embed_write = LdmWrite(*args, first=True) if first else None
        self.mixer_read = LdmRead(*args)
        self.mixer_write = LdmWrite(*args)
        self.mlp_read = LdmRead(*args)
        self.mlp_write = LdmWrite(*args)
        self.out_read = LdmRead(*args) if last else None


def build(cfg, layers) -> None:
    e, d = cfg.encoder, cfg.d_model
    if d % e.ldm_groups:
        raise ValueError(f"model.encoder.ldm_groups {e.ldm_groups} must divide d_model {d}")
    hidden, n = address_hidden(d, e.ldm_hidden), len(layers)
    for i, layer in enumerate(layers):
        layer.attn_res = LdmLayer(d, e.ldm_groups, e.ldm_key_dim, hidden, cfg.norm_eps, first=i == 0, last=i == n - 1)


def layer_forward(layer, x, M, ctx, cache, need_state: bool = True):
    """One layer's two sites. M None in layer 0 (it writes the embedding first). Returns (x, M, cache entry); the last
    layer returns the stream plus the output's read as x."""
    res = layer.attn_res
    if res.embed_write is not None:
        M = res.embed_write.first(x)
    h = x + res.mixer_read.read(M, x)
    if layer.kind == "gdn":
        mixed, c = layer.mixer(layer.mixer_in_norm(h), ctx, cache, need_state=need_state)
    else:
        mixed, c = layer.mixer(layer.mixer_in_norm(h), ctx, cache)
    delta = (layer.residual_scale * layer.mixer_out_norm(mixed, out_dtype=x.dtype)).to(x.dtype)
    x = x + delta
    M = res.mixer_write.write(M, x, delta)
    h = x + res.mlp_read.read(M, x)
    delta = (layer.residual_scale * layer.mlp_out_norm(layer.mlp(layer.mlp_in_norm(h)), out_dtype=x.dtype)).to(x.dtype)
    x = x + delta
    M = res.mlp_write.write(M, x, delta)
    if res.out_read is not None:
        x = x + res.out_read.read(M, x)
    return x, M, c


def parameter_count(d: int, n_layers: int, groups: int, key_dim: int, hidden: int) -> int:
    net = d + (d + 1) * hidden + (hidden + 1) * groups * key_dim + (hidden + 1) * groups
    sites = 2 * n_layers + 1
    return sites * (net + groups) + sites * net + (sites - 1) * groups
