"""Gated DeltaProduct in the GDN layers (`gdn.dprod.n_h` >= 2): n_h delta-rule steps a token.

    S <- a_t S                                                          the decay, once
    S <- S + k_{t,j} (beta_{t,j} (v_{t,j} - S^T k_{t,j}))^T,  j = 1..n_h  each with its own key, value and write strength
    o_t = S^T q_t                                                       the read, once, after the last step

beta = M sigmoid(b) on every step, M = `dprod.beta_max` (2, the default: every step's transition has an eigenvalue in
(-1, 1) along its key; 1: beta in (0, 1)); `dprod.beta_init` p (with beta_max 1) adds the fixed offset logit(p) to b on
every step, no tensor. Step 1 is the layer's own (in_proj_qkv's k and v, in_proj_b's beta); steps 2..n_h read
`dprod.in_proj_kv` (d -> (n_h - 1)(Hk dk + Hv dv), each step's [k_j | v_j] in turn), `dprod.conv_weight` (their short
conv) and `dprod.in_proj_b` (d -> (n_h - 1) Hv, step-major). One causal conv runs over [in_proj_qkv(x) | in_proj_kv(x)],
so the cache's conv history holds both. The extra tensors are drawn from a generator of their own after every other
tensor, so the base layer starts as in the base model of the same seed.

Paths: the token-and-step loop (`dprod_recurrence`), and the n_h T interleave into the chunked delta rule: sub-step
n_h t + j - 1 is an ordinary step with k_{t,j}, v_{t,j}, beta_{t,j}; the decay and a document start on sub-step 1
only, q_t on sub-step n_h only, where the output is read. Tensor ops on every device.

Placement (`dprod.layers`, `dprod.heads`, `dprod.heads_by_layer`; resolved per GDN layer by the config's `dprod_carry` /
`gdn_layer_configs`): a layer that does not carry is the plain layer (no module here); a layer that carries SOME value
heads (whole key groups) holds `PartialSteps`, the extra steps' tensors sized for the carrying heads alone, and the
same `forward` runs it: one projection and one conv over [q | k_1 | v_1 | the carrying heads' k_j, v_j], then the
carrying heads through the n_h-step rule (beta = 2 sigmoid(b) on every step) and the others through the plain rule
(beta = sigmoid(b), one write), the outputs and states joined along the head axis before the gated norm. The two groups
of heads are gathered through index tensors built once a device (`HeadSplit`) and joined through the inverse
permutation. The derived second step and the second step on a subset of the tokens live in modules of their own
(reference: ced/model/gdn_dprod.py:1-100, 155-210, 278-335, 389-476, 479-545; ced/model/gdn_dprod_place.py:36-327).
"""

from __future__ import annotations

import dataclasses
import math

import torch
import torch.nn as nn
import torch.nn.functional as F

from .. import ops
from .linear import Linear

SEED_OFFSET = 0xD9_0D_2026_1022
STANDALONE_SEED = 0xD9_0D
BETA_MAXES = (1, 2)
PLACEMENT_KEYS = ("layers", "heads", "heads_by_layer")


def _is_count(x) -> bool:
    return type(x) is int


def n_steps(cfg) -> int:
    if not _is_count(cfg.dprod.n_h) or cfg.dprod.n_h < 1:
        raise ValueError(f"gdn.dprod.n_h {cfg.dprod.n_h!r}: an integer >= 1 (1: Gated DeltaNet, the layer as it was)")
    return cfg.dprod.n_h


def is_on(cfg) -> bool:
    return n_steps(cfg) > 1


def _placed(d) -> list:
    plain = type(d)()
    return [k for k in PLACEMENT_KEYS if getattr(d, k) != getattr(plain, k)]


def _scalar_layer_only(cfg) -> None:
    if is_on(cfg) and (cfg.negeig.beta_max, cfg.kda.decay, cfg.erase.mode) != (1, "scalar", "none"):
        raise ValueError("gdn.dprod.n_h >= 2 is built on the scalar-decay layer alone: negeig.beta_max 1, kda.decay 'scalar', erase.mode 'none'")


def check_config(cfg) -> None:
    """The keys of one GDN layer's `dprod` section, the placement keys aside (they are the model's)."""
    from . import gdn_dprod_derived as derived, gdn_dprod_sparse as sparse

    d, steps = cfg.dprod, n_steps(cfg)
    if _placed(d):
        raise ValueError(f"gdn.dprod.{', '.join(_placed(d))} on a GDN layer built on its own: the placement keys are model.encoder.gdn.dprod's, "
                         "resolved per layer (the layer is given its heads)")
    sparse.check_keys(cfg)
    if not sparse.is_sparse(cfg):
        derived.check_second(cfg)
    if d.route != "interleave":
        raise ValueError(f"gdn.dprod.route {d.route!r}: the one-readout route is a kernel of the reference's fused path; the rule here runs as "
                         "tensor ops on the interleave (leave it 'interleave')")
    if not _is_count(d.beta_max) or d.beta_max not in BETA_MAXES:
        raise ValueError(f"gdn.dprod.beta_max {d.beta_max!r}: 1 (beta = sigmoid(b)) or 2 (beta = 2 sigmoid(b), the default)")
    _scalar_layer_only(cfg)
    if derived.is_derived(cfg) or sparse.is_sparse(cfg):
        return                                  # those forms check beta_init themselves
    start = d.beta_init
    if start is not None:
        if type(start) not in (int, float) or not 0.0 < start < 1.0:
            raise ValueError(f"gdn.dprod.beta_init {start!r}: None or a number in (0, 1)")
        if steps == 1 or d.beta_max != 1:
            raise ValueError(f"gdn.dprod.beta_init {start!r} is set for n_h >= 2 with beta_max 1")
    if steps == 1 and d.beta_max != 2:
        raise ValueError(f"gdn.dprod.beta_max {d.beta_max} with dprod.n_h 1: beta_max needs n_h >= 2")


def check_model(cfg) -> None:
    """What the whole model adds: placement against the other forms, and the parts the extra steps are not built with."""
    enc = cfg.encoder
    if not is_on(enc.gdn):
        return
    from . import gdn_dprod_derived as derived, gdn_dprod_sparse as sparse

    d = enc.gdn.dprod
    if derived.is_derived(enc.gdn):
        if enc.gdn_shape_by_layer:
            raise ValueError(f"model.encoder.gdn_shape_by_layer with model.encoder.gdn.dprod.key {d.key!r}: not built together")
        if _placed(d):
            raise ValueError(f"model.encoder.gdn.dprod.layers / heads / heads_by_layer with dprod.key {d.key!r}: the derived second step is built "
                             "for every head of every GDN layer")
    if sparse.is_sparse(enc.gdn) and (_placed(d) or enc.gdn_shape_by_layer):
        raise ValueError("model.encoder.gdn.dprod.layers / heads / heads_by_layer (or gdn_shape_by_layer) with dprod.stride / summary / conv: "
                         "the second step on a subset of the tokens is built for every head of every GDN layer")
    split_layers = [i for i, (_, carry) in enumerate(enc.gdn_layer_configs()) if carry is not None]
    if split_layers and (d.beta_max, d.beta_init) != (2, None):
        raise ValueError(f"model.encoder.gdn.dprod.beta_max / beta_init with GDN layer(s) {split_layers} that carry only some of their value heads: "
                         "the split layer writes 2 sigmoid(b) on the carrying heads and sigmoid(b) on the others and reads neither key")
    clashes = []
    if enc.gdn_write_mix != "none":
        clashes.append(f"model.encoder.gdn_write_mix {enc.gdn_write_mix!r}")
    if enc.gdn_shape_by_layer:
        clashes.append("model.encoder.gdn_shape_by_layer")
    if cfg.mtp.enabled:
        clashes.append("model.mtp.enabled")
    clashes += [f"model.{name}.mode {getattr(cfg, name).mode!r}" for name in ("fp8", "nvfp4") if getattr(cfg, name).mode != "none"]
    if clashes:
        raise ValueError(f"model.encoder.gdn.dprod.n_h {d.n_h} is not built with: {'; '.join(clashes)}")


def step_channels(cfg) -> int:
    """The conv channels one extra step adds: its key heads and its value heads."""
    return cfg.k_head_dim * cfg.n_k_heads + cfg.v_head_dim * cfg.n_v_heads


def params_per_layer(d_model: int, cfg) -> int:
    per_step = step_channels(cfg) * (d_model + cfg.conv_kernel) + cfg.n_v_heads * d_model
    return (n_steps(cfg) - 1) * per_step


def beta_offset(cfg) -> float:
    """logit(beta_init), added to every step's b; 0 without the key."""
    p = cfg.dprod.beta_init
    return 0.0 if p is None else math.log(p) - math.log1p(-p)


class DeltaProductSteps(nn.Module):
    """The tensors of steps 2..n_h when every head carries."""

    split = None

    def __init__(self, d_model: int, cfg):
        super().__init__()
        self.n_extra = n_steps(cfg) - 1
        self.channels = step_channels(cfg) * self.n_extra
        with torch.random.fork_rng(devices=[]):                     # building draws nothing from the global generator
            self.in_proj_kv = Linear(d_model, self.channels)
            self.in_proj_b = Linear(d_model, cfg.n_v_heads * self.n_extra)
        for lin in (self.in_proj_kv, self.in_proj_b):
            lin.own_init = True
        self.conv_weight = nn.Parameter(torch.empty(self.channels, cfg.conv_kernel))
        self.reset_own(torch.Generator().manual_seed(STANDALONE_SEED), 0.02)

    @torch.no_grad()
    def reset_own(self, g: torch.Generator, std: float) -> None:
        """in_proj_kv, in_proj_b ~ N(0, std), then the conv ~ U(+-1 / sqrt(kernel)), in that order from g."""
        width = 1.0 / math.sqrt(self.conv_weight.shape[1])
        for t, normal in ((self.in_proj_kv.weight, True), (self.in_proj_b.weight, True), (self.conv_weight, False)):
            if t.is_meta:
                continue
            if normal:
                fresh = torch.randn(t.shape, generator=g, dtype=torch.float32) * std
            else:
                fresh = (torch.rand(t.shape, generator=g, dtype=torch.float32) * 2 - 1) * width
            t.copy_(fresh.to(device=t.device, dtype=t.dtype))


class HeadSplit:
    """A partition of a layer's value heads into the carrying heads (whole key groups) and the others, with the matching
    partition of the key heads. `pick` gathers one side along a head axis; `join` puts two sides back in head order."""

    def __init__(self, n_k: int, n_v: int, carry: tuple):
        group = n_v // n_k
        self.v = {"carry": tuple(carry), "plain": tuple(h for h in range(n_v) if h not in carry)}
        k_carry = tuple(sorted({h // group for h in carry}))
        self.k = {"carry": k_carry, "plain": tuple(h for h in range(n_k) if h not in k_carry)}
        if not (0 < len(carry) < n_v and len(k_carry) * group == len(carry)):
            raise ValueError(f"the carrying value heads {carry!r}: some whole key groups of {group} value heads, not all of the layer's {n_v}")
        order = self.v["carry"] + self.v["plain"]
        self._back = tuple(order.index(h) for h in range(n_v))
        self._index: dict = {}

    def _idx(self, heads: tuple, device) -> torch.Tensor:
        key = (heads, str(device))
        if key not in self._index:
            self._index[key] = torch.tensor(heads, dtype=torch.long, device=device)
        return self._index[key]

    def pick(self, t: torch.Tensor, side: str, dim: int, keys: bool = False) -> torch.Tensor:
        return t.index_select(dim, self._idx((self.k if keys else self.v)[side], t.device))

    def join(self, carry_t: torch.Tensor, plain_t: torch.Tensor, dim: int) -> torch.Tensor:
        return torch.cat([carry_t, plain_t], dim).index_select(dim, self._idx(self._back, carry_t.device))


class PartialSteps(DeltaProductSteps):
    """The extra steps' tensors of a layer that carries only the value heads `carry` (whole key groups): DeltaProductSteps
    at the carrying heads' counts, so names, shapes' meaning and draws are its own."""

    def __init__(self, d_model: int, cfg, carry: tuple):
        split = HeadSplit(cfg.n_k_heads, cfg.n_v_heads, tuple(carry))
        super().__init__(d_model, dataclasses.replace(cfg, n_k_heads=len(split.k["carry"]), n_v_heads=len(split.v["carry"])))
        self.split = split


def build_steps(d_model: int, cfg, carry: tuple | None):
    """A GDN layer's extra steps: None at n_h 1, DeltaProductSteps when every head carries (carry None), else PartialSteps."""
    from . import gdn_dprod_derived as derived, gdn_dprod_sparse as sparse

    carry = None if carry is None else tuple(carry)
    if not is_on(cfg):
        if carry:
            raise ValueError(f"gdn.dprod.n_h 1 with carrying heads {carry!r}: a layer that does not carry has none")
        return None
    every_head = carry is None or carry == tuple(range(cfg.n_v_heads))
    if sparse.is_sparse(cfg):
        if not every_head:
            raise ValueError(f"gdn.dprod.stride / summary / conv with the carrying value heads {carry!r}: not built together with a placement")
        return sparse.SparseSteps(d_model, cfg)
    if derived.is_derived(cfg):
        if not every_head:
            raise ValueError(f"gdn.dprod.key {cfg.dprod.key!r} with the carrying value heads {carry!r}: the derived second step is built for every head of a layer")
        return derived.DerivedSteps(d_model, cfg)
    return DeltaProductSteps(d_model, cfg) if every_head else PartialSteps(d_model, cfg, carry)


def init_own_parameters(model: nn.Module, std: float) -> int:
    """Starts the extra steps' tensors of every layer, in module order, from one generator of their own."""
    from . import gdn_dprod_derived as derived, gdn_dprod_sparse as sparse

    kinds = (DeltaProductSteps, derived.DerivedSteps, sparse.SparseSteps)
    g, count = torch.Generator().manual_seed((torch.initial_seed() + SEED_OFFSET) % (1 << 63)), 0
    for m in model.modules():
        if isinstance(m, kinds):
            m.reset_own(g, std)
            count += 1
    return count


# ------------------------------------------------------------------------------------------------------------- the rule

def dprod_recurrence(q, k, v, g, beta, is_doc_start, S):
    """q (B, L, H, dk) at the value heads; k (B, L, n_h, H, dk); v (B, L, n_h, H, dv); g (B, L, H); beta (B, L, n_h, H)."""
    reads = []
    for t in range(q.shape[1]):
        carried = is_doc_start[:, t].logical_not().to(S.dtype)[:, None] * g[:, t].exp()
        S = S * carried[:, :, None, None]
        for j in range(k.shape[2]):
            miss = v[:, t, j] - torch.einsum("bhkv,bhk->bhv", S, k[:, t, j])
            S = S + torch.einsum("bhk,bhv->bhkv", k[:, t, j], beta[:, t, j].unsqueeze(-1) * miss)
        reads.append(torch.einsum("bhkv,bhk->bhv", S, q[:, t]))
    return torch.stack(reads, dim=1), S


def _only_substep(t: torch.Tensor, n_h: int, last: bool) -> torch.Tensor:
    """(B, L, ...) -> (B, L n_h, ...): t on the first (or last) sub-step of each token, zeros on the others."""
    lead, trail = (n_h - 1, 0) if last else (0, n_h - 1)
    return F.pad(t.unsqueeze(2), (0, 0) * (t.dim() - 2) + (lead, trail)).flatten(1, 2)


def interleave(q, k, v, g, beta, is_doc_start):
    """The n_h L sub-step sequence: (q, k, v, g, beta, is_doc_start) of the ordinary delta rule."""
    n_h = k.shape[2]
    return (_only_substep(q, n_h, True), k.flatten(1, 2), v.flatten(1, 2), _only_substep(g, n_h, False), beta.flatten(1, 2),
            _only_substep(is_doc_start, n_h, False))


def last_substep(o: torch.Tensor, n_h: int) -> torch.Tensor:
    return o.unflatten(1, (-1, n_h)).select(2, n_h - 1)


def _product_rule(cfg, L, q, k, v, g, beta, starts, S0):
    if cfg.kernel == "recurrence" or L == 1:
        return dprod_recurrence(q, k, v, g, beta, starts, S0)
    o, S = ops.ref.chunked_delta_rule(*interleave(q, k, v, g, beta, starts), S0, cfg.chunk_size)
    return last_substep(o, k.shape[2]), S


def _plain_rule(cfg, L, q, k, v, g, beta, starts, S0):
    if cfg.kernel == "recurrence" or L == 1:
        return ops.ref.delta_rule_recurrence(q, k, v, g, beta, starts, S0)
    return ops.ref.chunked_delta_rule(q, k, v, g, beta, starts, S0, cfg.chunk_size)


def forward(layer, x, ctx, state):
    """The GDN layer's forward with the extra steps: (y, conv history over all channels, its document ids, S). One routine
    for a layer whose heads all carry and for a split layer; the split layer's other heads take the plain rule."""
    cfg, steps = layer.cfg, layer.dprod
    split: HeadSplit | None = steps.split
    B, L = ctx.doc.shape
    n_k, n_v, d_k, d_v = cfg.n_k_heads, cfg.n_v_heads, cfg.k_head_dim, cfg.v_head_dim
    c_k, c_v = (n_k, n_v) if split is None else (len(split.k["carry"]), len(split.v["carry"]))
    extra, group = steps.n_extra, n_v // n_k
    pre = torch.cat([layer.in_proj_qkv(x), steps.in_proj_kv(x)], dim=-1)
    if state is not None and state.conv_input.shape[-1] != pre.shape[-1]:
        where = "" if split is None else f" on {c_v} of {n_v} value heads"
        raise ValueError(f"this GDN cache holds {state.conv_input.shape[-1]} conv channels; Gated DeltaProduct n_h {extra + 1}{where} carries {pre.shape[-1]}")
    past = (None, None) if state is None else (state.conv_input, state.conv_doc)
    post, conv_input, conv_doc = ops.ref.causal_doc_conv(pre, ctx.doc, torch.cat([layer.conv_weight, steps.conv_weight], dim=0), *past)
    widths = [n_k * d_k, n_k * d_k, n_v * d_v] + [c_k * d_k, c_v * d_v] * extra
    q, k1, v1, *later = F.silu(post).split(widths, dim=-1)
    heads = lambda t, n, d: t.unflatten(-1, (n, d))                                      # noqa: E731
    q = ops.ref.l2_normalize(heads(q, n_k, d_k)) * d_k ** -0.5
    k1, v1 = ops.ref.l2_normalize(heads(k1, n_k, d_k)), heads(v1, n_v, d_v)
    k_later = [ops.ref.l2_normalize(heads(t, c_k, d_k)) for t in later[0::2]]
    v_later = [heads(t, c_v, d_v) for t in later[1::2]]
    # a split layer reads neither beta_max nor beta_init: 2 sigmoid(b) on its carrying heads, sigmoid(b) on the others
    top, shift = (cfg.dprod.beta_max, beta_offset(cfg)) if split is None else (2, 0.0)
    b_first, b_later = layer.in_proj_b(x), steps.in_proj_b(x)
    if shift:
        b_first, b_later = b_first + shift, b_later + shift
    g, beta1 = ops.ref.gdn_gates(layer.in_proj_a(x), b_first, layer.A_log, layer.dt_bias)
    beta_later = list((top * b_later.sigmoid()).unflatten(-1, (extra, c_v)).unbind(2))
    work = ops.ref.work_dtype(q)
    at_values = lambda t, dim: t.repeat_interleave(group, dim=dim)                       # noqa: E731
    S0 = state.S.to(work) if state is not None else x.new_zeros(B, n_v, d_k, d_v, dtype=work)
    starts = ctx.is_doc_start
    if split is None:
        k_all = at_values(torch.stack([k1] + k_later, dim=2), 3).to(work)
        o, S = _product_rule(cfg, L, at_values(q, 2).to(work), k_all, torch.stack([v1] + v_later, dim=2).to(work), g.to(work),
                             torch.stack([top * beta1] + beta_later, dim=2).to(work), starts, S0)
        return o, conv_input, conv_doc, S
    sides = {}
    for side in ("carry", "plain"):
        sides[side] = dict(q=at_values(split.pick(q, side, 2, keys=True), 2).to(work), k=split.pick(k1, side, 2, keys=True),
                           v=split.pick(v1, side, 2), g=split.pick(g, side, 2).to(work), beta=split.pick(beta1, side, 2), S=split.pick(S0, side, 1))
    c, p = sides["carry"], sides["plain"]
    o_c, S_c = _product_rule(cfg, L, c["q"], at_values(torch.stack([c["k"]] + k_later, dim=2), 3).to(work), torch.stack([c["v"]] + v_later, dim=2).to(work),
                             c["g"], torch.stack([top * c["beta"]] + beta_later, dim=2).to(work), starts, c["S"])
    o_p, S_p = _plain_rule(cfg, L, p["q"], at_values(p["k"], 2).to(work), p["v"].to(work), p["g"], p["beta"].to(work), starts, p["S"])
    return split.join(o_c, o_p, 2), conv_input, conv_doc, split.join(S_c, S_p, 1)
