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

from .. import ops
from .linear import Linear

DERIVED = ("lowrank", "prev", "perm", "rot")
KEYS = ("proj",) + DERIVED
PERMS = ("roll", "random")
STANDALONE_SEED = 0xC2_0D
_SECOND = ("key", "value", "beta", "rank", "perm", "conv")           # the keys this module reads
_FOREIGN = ("layers", "heads", "heads_by_layer", "beta_max", "beta_init", "stride", "summary", "first_beta", "route")


def is_derived(cfg) -> bool:
    return getattr(cfg.dprod, "key", "proj") in DERIVED


def _off_default(d, names) -> list:
    plain = type(d)()
    return [n for n in names if getattr(d, n) != getattr(plain, n)]


def check_second(cfg, where: str = "gdn.dprod") -> None:
    """The second step's keys of one GDN config (ValueError naming the key)."""
    d = cfg.dprod
    plain = type(d)()
    domain = {"key": KEYS, "value": ("proj", "v1"), "beta": ("proj",), "perm": PERMS}
    for name, allowed in domain.items():
        if getattr(d, name) not in allowed:
            raise ValueError(f"{where}.{name} {getattr(d, name)!r}: one of {allowed}")
    limit = cfg.k_head_dim if d.key == "lowrank" else None
    if type(d.rank) is not int or d.rank < 1 or (limit is not None and d.rank > limit):
        raise ValueError(f"{where}.rank {d.rank!r}: an integer >= 1" + (f" and, with key 'lowrank', at most k_head_dim = {limit}" if limit else ""))
    if not isinstance(d.conv, bool):
        raise ValueError(f"{where}.conv {d.conv!r}: a bool")
    moved = _off_default(d, _SECOND)
    if d.n_h == 1:
        if moved:
            raise ValueError(f"{where}.{', '.join(moved)} set with n_h 1: the second step's keys are read only with n_h 2")
        return
    if not is_derived(cfg):
        extra = [n for n in moved if n != "key"]
        if extra:
            raise ValueError(f"{where}.key 'proj' (full projections and the short conv) with {', '.join(extra)} off their defaults: those belong "
                             "to a derived key (lowrank, prev, perm, rot); the strided and summarised second steps are not built")
        return
    if d.n_h != 2:
        raise ValueError(f"{where}.key {d.key!r} with n_h {d.n_h}: the derived second step is built for n_h 2")
    needs = {"value": "v1", "beta": "proj", "conv": False}
    wrong = [f"{n} {getattr(d, n)!r} (wants {w!r})" for n, w in needs.items() if getattr(d, n) != w]
    if wrong:
        raise ValueError(f"{where}.key {d.key!r}: {'; '.join(wrong)}: the second step has no value or conv channels of its own")
    for name, owner in (("rank", "lowrank"), ("perm", "perm")):
        if d.key != owner and getattr(d, name) != getattr(plain, name):
            raise ValueError(f"{where}.{name} {getattr(d, name)!r} belongs to key {owner!r}; this layer's key is {d.key!r}")
    unread = _off_default(d, _FOREIGN)
    if unread:
        raise ValueError(f"{where}.{', '.join(unread)} with key {d.key!r}: the derived second step reads none of these keys; not built together")


def params_per_layer(d_model: int, cfg) -> int:
    extra = cfg.dprod.rank * cfg.n_k_heads * (d_model + cfg.k_head_dim) if cfg.dprod.key == "lowrank" else 0
    return d_model * cfg.n_v_heads + extra


def random_rotation(dk: int, g: torch.Generator) -> torch.Tensor:
    """A Haar rotation (det +1) from the CPU generator: Q of a Gaussian matrix's QR with R's diagonal made positive, the
    first column negated when the determinant is -1. float32."""
    basis, upper = torch.linalg.qr(torch.randn(dk, dk, generator=g, dtype=torch.float64))
    basis = basis * upper.diagonal().sign().unsqueeze(0)
    if torch.linalg.det(basis).item() < 0:
        basis[:, 0].neg_()
    return basis.float()


class DerivedSteps(nn.Module):
    n_extra = 1

    def __init__(self, d_model: int, cfg):
        super().__init__()
        check_second(cfg)
        self.key, self.perm_kind, self.rank = cfg.dprod.key, cfg.dprod.perm, cfg.dprod.rank
        self.d_model, self.hk, self.hv, self.dk = d_model, cfg.n_k_heads, cfg.n_v_heads, cfg.k_head_dim
        widths = {"in_proj_b": (d_model, self.hv)}
        if self.key == "lowrank":
            widths.update(k_down=(d_model, self.rank * self.hk), k_up=(self.rank, self.hk * self.dk))
        with torch.random.fork_rng(devices=[]):           # building draws nothing from the global stream
            for name, (n_in, n_out) in widths.items():
                lin = Linear(n_in, n_out)
                lin.own_init = True
                setattr(self, name, lin)
        if self.key == "rot":
            self.register_buffer("rot", torch.empty(self.dk, self.dk, dtype=torch.float32))
        elif self.key == "perm" and self.perm_kind == "random":
            self.register_buffer("perm", torch.empty(self.dk, dtype=torch.long))
        self.reset_own(torch.Generator().manual_seed(STANDALONE_SEED), 0.02)

    def _normal_draws(self, std: float) -> list:
        """(tensor, its standard deviation) in draw order: in_proj_b, then the low-rank pair; k_up's so that the correction has about k1's size."""
        out = [(self.in_proj_b.weight, std)]
        if self.key == "lowrank":
            out += [(self.k_down.weight, std), (self.k_up.weight, (self.dk * self.rank * self.d_model) ** -0.5 / std)]
        return out

    @torch.no_grad()
    def reset_own(self, g: torch.Generator, std: float) -> None:
        for tensor, sigma in self._normal_draws(std):
            if tensor.is_meta:
                continue
            tensor.copy_(torch.randn(tensor.shape, generator=g, dtype=torch.float32).mul(sigma).to(tensor))
        seeded = getattr(self, "rot", None) if self.key == "rot" else getattr(self, "perm", None)
        if seeded is not None and not seeded.is_meta:
            seeded.copy_((random_rotation(self.dk, g) if self.key == "rot" else torch.randperm(self.dk, generator=g)).to(seeded))

    # one method per key: k2 (B, L, H_k, d_k) in k1's dtype (fixed shapes: a roll or an index buffer, one batched product, a shift and a 0 / 1 factor)

    def _key_lowrank(self, x, k1, is_doc_start, k_prev):
        wide = torch.promote_types(k1.dtype, torch.float32)
        coeff = self.k_down(x).unflatten(-1, (self.hk, self.rank))
        lift = self.k_up.weight.to(coeff.dtype).view(self.hk, self.dk, self.rank)
        return ops.ref.l2_normalize(k1.to(wide) + torch.einsum("...hr,hdr->...hd", coeff, lift).to(wide)).to(k1.dtype)

    def _key_prev(self, x, k1, is_doc_start, k_prev):
        lead = k1.new_zeros(k1[:, :1].shape) if k_prev is None else k_prev.unsqueeze(1).to(k1.dtype)
        shifted = torch.cat([lead, k1[:, :-1]], dim=1)
        return shifted * is_doc_start.logical_not().to(shifted.dtype)[..., None, None]      # a document's first token reads no earlier key

    def _key_perm(self, x, k1, is_doc_start, k_prev):
        return k1.roll(self.dk // 2, -1) if self.perm_kind == "roll" else k1.index_select(-1, self.perm)

    def _key_rot(self, x, k1, is_doc_start, k_prev):
        wide = torch.promote_types(k1.dtype, torch.float32)
        return torch.matmul(k1.to(wide), self.rot.to(wide).t()).to(k1.dtype)

    def second_key(self, x, k1, is_doc_start, k_prev):
        return getattr(self, "_key_" + self.key)(x, k1, is_doc_start, k_prev)

    def extra_repr(self) -> str:
        return f"key={self.key!r}" + (f", rank={self.rank}" if self.key == "lowrank" else "")


def forward(layer, x, ctx, state):
    """(o, conv history, its document ids, S, k_prev): the plain layer's input preparation, the second key from the first,
    and the two-step rule on the stacks (the loop, or the 2T interleave into the chunked rule)."""
    from .gdn_dprod import dprod_recurrence, interleave, last_substep

    g_cfg, steps = layer.cfg, layer.dprod
    rows, length = ctx.doc.shape
    n_k, n_v, d_k, d_v = g_cfg.n_k_heads, g_cfg.n_v_heads, g_cfg.k_head_dim, g_cfg.v_head_dim
    u = layer.in_proj_qkv(x)
    if state is not None:
        if state.conv_input.shape[-1] != u.shape[-1]:
            raise ValueError(f"this GDN cache holds {state.conv_input.shape[-1]} conv channels; a layer with a derived second step carries {u.shape[-1]}")
        if steps.key == "prev" and state.k_prev is None:
            raise ValueError("this GDN cache holds no previous key: it was not written by a layer with gdn.dprod.key 'prev'")
    past = (None, None) if state is None else (state.conv_input, state.conv_doc)
    q, k1, v1, conv_input, conv_doc = ops.ref.gdn_prep(u, ctx.doc, layer.conv_weight, n_k, n_v, d_k, d_v, *past)
    k2 = steps.second_key(x, k1, ctx.is_doc_start, state.k_prev if state is not None else None)
    g, beta1 = ops.ref.gdn_gates(layer.in_proj_a(x), layer.in_proj_b(x), layer.A_log, layer.dt_bias)
    work = ops.ref.work_dtype(q)
    group = n_v // n_k
    keys = torch.stack((k1, k2), dim=2).repeat_interleave(group, dim=3).to(work)
    values = torch.stack((v1, v1), dim=2).to(work)                                      # one value, two addresses
    betas = torch.stack((2 * beta1, 2 * torch.sigmoid(steps.in_proj_b(x))), dim=2).to(work)
    query, decay = q.repeat_interleave(group, dim=2).to(work), g.to(work)
    S0 = state.S.to(work) if state is not None else x.new_zeros(rows, n_v, d_k, d_v, dtype=work)
    if g_cfg.kernel == "recurrence" or length == 1:
        o, S = dprod_recurrence(query, keys, values, decay, betas, ctx.is_doc_start, S0)
    else:
        o_rows, S = ops.ref.chunked_delta_rule(*interleave(query, keys, values, decay, betas, ctx.is_doc_start), S0, g_cfg.chunk_size)
        o = last_substep(o_rows, 2)
    return o, conv_input, conv_doc, S, (k1[:, -1].clone() if steps.key == "prev" else None)
