"""Gated DeltaProduct with a second step made from the first (`gdn.dprod.key` lowrank / prev / perm / rot, n_h 2).

The rule is Gated DeltaProduct's with two steps a token (models/gdn_dprod.py); the second step's value is the first's
(`dprod.value: v1`), its write strength 2 sigmoid of its own projection `dprod.in_proj_b` (d -> H_v), and its key is made
cheaply from the first step's unit key k1, with no conv channel of its own (`dprod.conv: false`):

    lowrank   k2 = L2norm(k1 + U_h W_h x)    W: d -> r per key head (`dprod.k_down`), U_h: r -> d_k (`dprod.k_up`, (H_k d_k, r)
                                             applied per head as one batched product), r = `dprod.rank`
    prev      k2_t = k1_{t-1}                zero at a document start and at a sequence's first token (then the second write
                                             is the identity); a cached forward carries the last key (`GDNState.k_prev`)
    perm      k2 = P k1                      a cyclic shift by d_k / 2 (`dprod.perm: roll`) or a seeded permutation (`random`,
                                             a persistent buffer)
    rot       k2 = Q k1                      a seeded Haar rotation (det +1), one per layer, a persistent buffer

Starts: in_proj_b and k_down ~ N(0, std), k_up ~ N(0, s) with s = 1 / (sqrt(d_k r) std sqrt(d)) so that the correction has
about k1's size from the first step on; all from the generator the extra steps of Gated DeltaProduct use, in module
order, so the base layer starts as in the base model of the same seed. Buffers are in the state dict: a resume never
redraws them. Every head of every GDN layer carries (no placement, no shape table). Tensor ops on every device
(reference: ced/model/gdn_dprod_c.py:1-365).
"""

from __future__ import annotations

import math

import torch
import torch.nn as nn
import torch.nn.functional as F

from .. import ops
from .linear import Linear

DERIVED = ("lowrank", "prev", "perm", "rot")
KEYS = ("proj",) + DERIVED
PERMS = ("roll", "random")
STANDALONE_SEED = 0xC2_0D


def is_derived(cfg) -> bool:
    return getattr(cfg.dprod, "key", "proj") in DERIVED


def check_second(cfg, where: str = "gdn.dprod") -> None:
    """The second step's keys of one GDN config (ValueError naming the key)."""
    d = cfg.dprod
    default = type(d)()
    if d.key not in KEYS:
        raise ValueError(f"{where}.key {d.key!r}: one of {KEYS}")
    if d.value not in ("proj", "v1"):
        raise ValueError(f"{where}.value {d.value!r}: 'proj' or 'v1'")
    if d.beta != "proj":
        raise ValueError(f"{where}.beta {d.beta!r}: 'proj' (its own projection; tied and constant forms are not built)")
    if d.perm not in PERMS:
        raise ValueError(f"{where}.perm {d.perm!r}: one of {PERMS}")
    if type(d.rank) is not int or d.rank < 1 or (d.key == "lowrank" and d.rank > cfg.k_head_dim):
        raise ValueError(f"{where}.rank {d.rank!r}: an integer >= 1 (with key 'lowrank' at most k_head_dim = {cfg.k_head_dim})")
    if type(d.conv) is not bool:
        raise ValueError(f"{where}.conv {d.conv!r}: true or false")
    off = [k for k in ("key", "value", "beta", "rank", "perm", "conv") if getattr(d, k) != getattr(default, k)]
    if d.n_h == 1:
        if off:
            raise ValueError(f"{where}.{', '.join(off)} set with n_h 1: the second step's keys are read only with n_h 2")
        return
    if d.key == "proj":
        wrong = [k for k in off if k != "key"]
        if wrong:
            raise ValueError(f"{where}.key 'proj' (full projections and the short conv) with {', '.join(wrong)} off their defaults: those belong "
                             "to a derived key (lowrank, prev, perm, rot); the strided and summarised second steps are not built")
        return
    if d.n_h != 2:
        raise ValueError(f"{where}.key {d.key!r} with n_h {d.n_h}: the derived second step is built for n_h 2")
    wrong = [f"{k} {getattr(d, k)!r} (wants {w!r})" for k, w in (("value", "v1"), ("beta", "proj"), ("conv", False)) if getattr(d, k) != w]
    if wrong:
        raise ValueError(f"{where}.key {d.key!r}: {'; '.join(wrong)}: the second step has no value or conv channels of its own")
    if d.key != "lowrank" and d.rank != default.rank:
        raise ValueError(f"{where}.rank {d.rank!r} is read with key 'lowrank'; this layer's key is {d.key!r}")
    if d.key != "perm" and d.perm != default.perm:
        raise ValueError(f"{where}.perm {d.perm!r} is read with key 'perm'; this layer's key is {d.key!r}")
    unread = [k for k in ("layers", "heads", "heads_by_layer", "beta_max", "beta_init", "stride", "summary", "first_beta", "route")
              if getattr(d, k) != getattr(default, k)]
    if unread:
        raise ValueError(f"{where}.{', '.join(unread)} with key {d.key!r}: the derived second step reads none of these keys; not built together")


def params_per_layer(d_model: int, cfg) -> int:
    n = d_model * cfg.n_v_heads
    if cfg.dprod.key == "lowrank":
        n += d_model * cfg.dprod.rank * cfg.n_k_heads + cfg.dprod.rank * cfg.n_k_heads * cfg.k_head_dim
    return n


def random_rotation(dk: int, g: torch.Generator) -> torch.Tensor:
    """A Haar rotation (det +1) from the CPU generator: Q of a Gaussian matrix's QR with R's diagonal made positive, the
    first column negated when the determinant is -1. float32."""
    q, r = torch.linalg.qr(torch.randn(dk, dk, generator=g, dtype=torch.float64))
    q = q * torch.sign(torch.diagonal(r))[None, :]
    if float(torch.linalg.det(q)) < 0:
        q[:, 0] = -q[:, 0]
    return q.to(torch.float32)


class DerivedSteps(nn.Module):
    n_extra = 1

    def __init__(self, d_model: int, cfg):
        super().__init__()
        check_second(cfg)
        d = cfg.dprod
        self.key, self.perm_kind, self.rank = d.key, d.perm, d.rank
        self.d_model, self.hk, self.hv, self.dk = d_model, cfg.n_k_heads, cfg.n_v_heads, cfg.k_head_dim
        with torch.random.fork_rng(devices=[]):           # building draws nothing from the global stream
            self.in_proj_b = Linear(d_model, self.hv)
            if self.key == "lowrank":
                self.k_down = Linear(d_model, self.rank * self.hk)
                self.k_up = Linear(self.rank, self.hk * self.dk)
        for m in self.children():
            m.own_init = True
        if self.key == "rot":
            self.register_buffer("rot", torch.empty(self.dk, self.dk, dtype=torch.float32))
        if self.key == "perm" and self.perm_kind == "random":
            self.register_buffer("perm", torch.empty(self.dk, dtype=torch.long))
        self.reset_own(torch.Generator().manual_seed(STANDALONE_SEED), 0.02)

    @torch.no_grad()
    def reset_own(self, g: torch.Generator, std: float) -> None:
        draws = [(self.in_proj_b.weight, std)]
        if self.key == "lowrank":
            draws += [(self.k_down.weight, std), (self.k_up.weight, 1.0 / (math.sqrt(self.dk * self.rank) * std * math.sqrt(self.d_model)))]
        for p, s in draws:
            if not p.is_meta:
                p.copy_((torch.randn(p.shape, generator=g, dtype=torch.float32) * s).to(device=p.device, dtype=p.dtype))
        if self.key == "rot" and not self.rot.is_meta:
            self.rot.copy_(random_rotation(self.dk, g).to(device=self.rot.device, dtype=self.rot.dtype))
        if self.key == "perm" and self.perm_kind == "random" and not self.perm.is_meta:
            self.perm.copy_(torch.randperm(self.dk, generator=g).to(self.perm.device))

    def second_key(self, x, k1, is_doc_start, k_prev):
        """k2 (B, L, H_k, d_k) in k1's dtype. Fixed shapes: a roll or an index buffer, one batched product, a shift and a 0 / 1 factor."""
        wide = torch.promote_types(k1.dtype, torch.float32)
        if self.key == "lowrank":
            z = self.k_down(x).unflatten(-1, (self.hk, self.rank))
            w = self.k_up.weight.to(z.dtype).view(self.hk, self.dk, self.rank)
            return ops.ref.l2_normalize(k1.to(wide) + torch.einsum("...hr,hdr->...hd", z, w).to(wide)).to(k1.dtype)
        if self.key == "prev":
            first = torch.zeros_like(k1[:, :1]) if k_prev is None else k_prev[:, None].to(k1.dtype)
            prev = torch.cat([first, k1[:, :-1]], dim=1)
            return prev * (~is_doc_start).to(prev.dtype)[..., None, None]
        if self.key == "perm":
            return torch.roll(k1, shifts=self.dk // 2, dims=-1) if self.perm_kind == "roll" else k1[..., self.perm]
        return torch.einsum("...hd,ed->...he", k1.to(wide), self.rot.to(wide)).to(k1.dtype)

    def extra_repr(self) -> str:
        return f"key={self.key!r}" + (f", rank={self.rank}" if self.key == "lowrank" else "")


def forward(layer, x, ctx, state):
    """(o, conv history, its document ids, S, k_prev): the plain layer's input preparation, the second key from the first,
    and the two-step rule on the stacks (the loop, or the 2T interleave into the chunked rule)."""
    from .gdn_dprod import dprod_recurrence, interleave, last_substep

    cfg, steps = layer.cfg, layer.dprod
    B, L = ctx.doc.shape
    hk, hv, dk, dv = cfg.n_k_heads, cfg.n_v_heads, cfg.k_head_dim, cfg.v_head_dim
    u = layer.in_proj_qkv(x)
    if state is not None and state.conv_input.shape[-1] != u.shape[-1]:
        raise ValueError(f"this GDN cache holds {state.conv_input.shape[-1]} conv channels; a layer with a derived second step carries {u.shape[-1]}")
    if steps.key == "prev" and state is not None and state.k_prev is None:
        raise ValueError("this GDN cache holds no previous key: it was not written by a layer with gdn.dprod.key 'prev'")
    hist, hist_doc = (None, None) if state is None else (state.conv_input, state.conv_doc)
    q, k1, v1, conv_input, conv_doc = ops.ref.gdn_prep(u, ctx.doc, layer.conv_weight, hk, hv, dk, dv, hist, hist_doc)
    k2 = steps.second_key(x, k1, ctx.is_doc_start, None if state is None else state.k_prev)
    g, beta1 = ops.ref.gdn_gates(layer.in_proj_a(x), layer.in_proj_b(x), layer.A_log, layer.dt_bias)
    beta2 = 2 * torch.sigmoid(steps.in_proj_b(x))
    rep = hv // hk
    dt = ops.ref.work_dtype(q)
    k = torch.stack([k1, k2], dim=2).repeat_interleave(rep, dim=3).to(dt)
    v = torch.stack([v1, v1], dim=2).to(dt)
    beta = torch.stack([2 * beta1, beta2], dim=2).to(dt)
    qr, g = q.repeat_interleave(rep, dim=2).to(dt), g.to(dt)
    S0 = x.new_zeros(B, hv, dk, dv, dtype=dt) if state is None else state.S.to(dt)
    if cfg.kernel != "recurrence" and L > 1:
        qi, ki, vi, gi, bi, si = interleave(qr, k, v, g, beta, ctx.is_doc_start)
        oi, S = ops.ref.chunked_delta_rule(qi, ki, vi, gi, bi, si, S0, cfg.chunk_size)
        o = last_substep(oi, 2)
    else:
        o, S = dprod_recurrence(qr, k, v, g, beta, ctx.is_doc_start, S0)
    return o, conv_input, conv_doc, S, (k1[:, -1].clone() if steps.key == "prev" else None)
