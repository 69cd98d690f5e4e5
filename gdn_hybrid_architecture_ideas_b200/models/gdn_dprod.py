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
heads (whole key groups) holds `PartialSteps`, the extra steps' tensors sized for the carrying heads alone, and runs
`forward_partial`: one projection and one conv over [q | k_1 | v_1 | the carrying heads' k_j, v_j], then the carrying
heads through the n_h-step rule (beta = 2 sigmoid(b) on every step) and the others through the plain rule
(beta = sigmoid(b), one write), the outputs and states joined along the head axis before the gated norm. Heads are cut
by static slices. The derived-key and sparse-step forms of the reference are refused by name
(reference: ced/model/gdn_dprod.py:1-100, 155-210, 278-335, 389-476, 479-545; ced/model/gdn_dprod_place.py:36-327).
"""

from __future__ import annotations

import math

import torch
import torch.nn as nn
import torch.nn.functional as F

from .. import ops
from .linear import Linear

SEED_OFFSET = 0xD9_0D_2026_1022
STANDALONE_SEED = 0xD9_0D
BETA_MAXES = (1, 2)


def n_steps(cfg) -> int:
    n = cfg.dprod.n_h
    if isinstance(n, bool) or not isinstance(n, int) or n < 1:
        raise ValueError(f"gdn.dprod.n_h {n!r}: an integer >= 1 (1: Gated DeltaNet, the layer as it was)")
    return n


def is_on(cfg) -> bool:
    return n_steps(cfg) > 1


def check_config(cfg) -> None:
    d, n = cfg.dprod, n_steps(cfg)
    default = type(d)()
    placed = [k for k in ("layers", "heads", "heads_by_layer") if getattr(d, k) != getattr(default, k)]
    if placed:
        raise ValueError(f"gdn.dprod.{', '.join(placed)} on a GDN layer built on its own: the placement keys are model.encoder.gdn.dprod's, "
                         "resolved per layer (the layer is given its heads)")
    from .gdn_dprod_derived import check_second, is_derived

    from . import gdn_dprod_sparse

    gdn_dprod_sparse.check_keys(cfg)
    if not gdn_dprod_sparse.is_sparse(cfg):
        check_second(cfg)
    if d.route != default.route:
        raise ValueError(f"gdn.dprod.route {d.route!r}: the one-readout route is a kernel of the reference's fused path; the rule here runs as "
                         "tensor ops on the interleave (leave it 'interleave')")
    if isinstance(d.beta_max, bool) or d.beta_max not in BETA_MAXES:
        raise ValueError(f"gdn.dprod.beta_max {d.beta_max!r}: 1 (beta = sigmoid(b)) or 2 (beta = 2 sigmoid(b), the default)")
    if is_derived(cfg) or gdn_dprod_sparse.is_sparse(cfg):
        if n > 1 and (cfg.negeig.beta_max != 1 or cfg.kda.decay != "scalar" or cfg.erase.mode != "none"):
            raise ValueError("gdn.dprod.n_h >= 2 is built on the scalar-decay layer alone: negeig.beta_max 1, kda.decay 'scalar', erase.mode 'none'")
        return
    m = d.beta_max
    if isinstance(m, bool) or not isinstance(m, int) or m not in BETA_MAXES:
        raise ValueError(f"gdn.dprod.beta_max {m!r}: 1 (beta = sigmoid(b)) or 2 (beta = 2 sigmoid(b), the default)")
    p = d.beta_init
    if p is not None and (isinstance(p, bool) or not isinstance(p, (int, float)) or not 0.0 < p < 1.0):
        raise ValueError(f"gdn.dprod.beta_init {p!r}: None or a number in (0, 1)")
    if n == 1 and m != 2:
        raise ValueError(f"gdn.dprod.beta_max {m} with dprod.n_h 1: beta_max needs n_h >= 2")
    if p is not None and (n == 1 or m != 1):
        raise ValueError(f"gdn.dprod.beta_init {p!r} is set for n_h >= 2 with beta_max 1")
    if n > 1 and (cfg.negeig.beta_max != 1 or cfg.kda.decay != "scalar" or cfg.erase.mode != "none"):
        raise ValueError("gdn.dprod.n_h >= 2 is built on the scalar-decay layer alone: negeig.beta_max 1, kda.decay 'scalar', erase.mode 'none'")


def check_model(cfg) -> None:
    if not is_on(cfg.encoder.gdn):
        return
    d = cfg.encoder.gdn.dprod
    from .gdn_dprod_derived import is_derived

    if is_derived(cfg.encoder.gdn) and cfg.encoder.gdn_shape_by_layer:
        raise ValueError(f"model.encoder.gdn_shape_by_layer with model.encoder.gdn.dprod.key {d.key!r}: not built together")
    if is_derived(cfg.encoder.gdn) and (d.layers != () or d.heads != 0 or d.heads_by_layer != {}):
        raise ValueError(f"model.encoder.gdn.dprod.layers / heads / heads_by_layer with dprod.key {d.key!r}: the derived second step is built "
                         "for every head of every GDN layer")
    from . import gdn_dprod_sparse

    if gdn_dprod_sparse.is_sparse(cfg.encoder.gdn) and (d.layers != () or d.heads != 0 or d.heads_by_layer != {} or cfg.encoder.gdn_shape_by_layer):
        raise ValueError("model.encoder.gdn.dprod.layers / heads / heads_by_layer (or gdn_shape_by_layer) with dprod.stride / summary / conv: "
                         "the second step on a subset of the tokens is built for every head of every GDN layer")
    partial = [i for i, (c, heads) in enumerate(cfg.encoder.gdn_layer_configs()) if heads is not None]
    if partial and (d.beta_max != 2 or d.beta_init is not None):
        raise ValueError(f"model.encoder.gdn.dprod.beta_max / beta_init with GDN layer(s) {partial} that carry only some of their value heads: "
                         "the split layer writes 2 sigmoid(b) on the carrying heads and sigmoid(b) on the others and reads neither key")
    refused = [(cfg.encoder.gdn_write_mix != "none", f"model.encoder.gdn_write_mix {cfg.encoder.gdn_write_mix!r}"),
               (bool(cfg.encoder.gdn_shape_by_layer), "model.encoder.gdn_shape_by_layer"), (bool(cfg.mtp.enabled), "model.mtp.enabled"),
               (cfg.fp8.mode != "none", f"model.fp8.mode {cfg.fp8.mode!r}"), (cfg.nvfp4.mode != "none", f"model.nvfp4.mode {cfg.nvfp4.mode!r}")]
    bad = [why for cond, why in refused if cond]
    if bad:
        raise ValueError(f"model.encoder.gdn.dprod.n_h {cfg.encoder.gdn.dprod.n_h} is not built with: {'; '.join(bad)}")


def step_channels(cfg) -> int:
    return cfg.n_k_heads * cfg.k_head_dim + cfg.n_v_heads * cfg.v_head_dim


def params_per_layer(d_model: int, cfg) -> int:
    n, c = n_steps(cfg) - 1, step_channels(cfg)
    return n * (d_model * c + d_model * cfg.n_v_heads + cfg.conv_kernel * c)


def beta_offset(cfg) -> float | None:
    p = cfg.dprod.beta_init
    return None if p is None else math.log(p) - math.log1p(-p)


class DeltaProductSteps(nn.Module):
    def __init__(self, d_model: int, cfg):
        super().__init__()
        self.n_extra = n_steps(cfg) - 1
        self.channels = self.n_extra * step_channels(cfg)
        with torch.random.fork_rng(devices=[]):
            self.in_proj_kv = Linear(d_model, self.channels)
            self.in_proj_b = Linear(d_model, self.n_extra * cfg.n_v_heads)
        self.in_proj_kv.own_init = self.in_proj_b.own_init = True
        self.conv_weight = nn.Parameter(torch.empty(self.channels, cfg.conv_kernel))
        self.reset_own(torch.Generator().manual_seed(STANDALONE_SEED), 0.02)

    @torch.no_grad()
    def reset_own(self, g: torch.Generator, std: float) -> None:
        bound = 1.0 / math.sqrt(self.conv_weight.shape[1])
        draws = ((self.in_proj_kv.weight, lambda s: torch.randn(s, generator=g, dtype=torch.float32) * std),
                 (self.in_proj_b.weight, lambda s: torch.randn(s, generator=g, dtype=torch.float32) * std),
                 (self.conv_weight, lambda s: (torch.rand(s, generator=g, dtype=torch.float32) * 2 - 1) * bound))
        for p, draw in draws:
            if not p.is_meta:
                p.copy_(draw(p.shape).to(device=p.device, dtype=p.dtype))


def runs_of(heads) -> tuple:
    """((start, length), ...): the maximal runs of consecutive indices in `heads` (sorted, distinct)."""
    out: list = []
    for h in heads:
        if out and out[-1][0] + out[-1][1] == h:
            out[-1] = (out[-1][0], out[-1][1] + 1)
        else:
            out.append((h, 1))
    return tuple(out)


def take(t: torch.Tensor, runs: tuple, dim: int) -> torch.Tensor:
    """The heads of `runs` along `dim`, in order: slices and at most one concatenation (no index tensor, no mask)."""
    pieces = [t.narrow(dim, s, n) for s, n in runs]
    return pieces[0] if len(pieces) == 1 else torch.cat(pieces, dim)


def merge(a: torch.Tensor, runs_a: tuple, b: torch.Tensor, runs_b: tuple, dim: int) -> torch.Tensor:
    """The inverse of `take` for a partition of the heads: a holds the heads of runs_a, b those of runs_b."""
    pieces, at = [], 0
    for s, n in runs_a:
        pieces.append((s, a.narrow(dim, at, n)))
        at += n
    at = 0
    for s, n in runs_b:
        pieces.append((s, b.narrow(dim, at, n)))
        at += n
    return torch.cat([p for _, p in sorted(pieces, key=lambda x: x[0])], dim)


class PartialSteps(DeltaProductSteps):
    """The extra steps' tensors of a layer that carries only the value heads `carry` (whole key groups): DeltaProductSteps
    at the carrying heads' counts, so names, shapes' meaning and draws are its own."""

    def __init__(self, d_model: int, cfg, carry: tuple):
        import dataclasses

        hk, hv = cfg.n_k_heads, cfg.n_v_heads
        g = hv // hk
        keys = tuple(sorted({h // g for h in carry}))
        if not (0 < len(carry) < hv and len(keys) * g == len(carry)):
            raise ValueError(f"the carrying value heads {carry!r}: some whole key groups of {g} value heads, not all of the layer's {hv}")
        self_hk, self_hv = len(keys), len(carry)
        super().__init__(d_model, dataclasses.replace(cfg, n_k_heads=self_hk, n_v_heads=self_hv))
        self.hk_c, self.hv_c, self.carry = self_hk, self_hv, tuple(carry)
        self.runs_v, self.runs_k = runs_of(self.carry), runs_of(keys)
        self.runs_v_plain = runs_of([h for h in range(hv) if h not in set(self.carry)])
        self.runs_k_plain = runs_of([h for h in range(hk) if h not in set(keys)])


def build_steps(d_model: int, cfg, carry: tuple | None):
    """A GDN layer's extra steps: None at n_h 1, DeltaProductSteps when every head carries (carry None), else PartialSteps."""
    if not is_on(cfg):
        if carry:
            raise ValueError(f"gdn.dprod.n_h 1 with carrying heads {tuple(carry)!r}: a layer that does not carry has none")
        return None
    from . import gdn_dprod_sparse
    from .gdn_dprod_derived import DerivedSteps, is_derived

    if gdn_dprod_sparse.is_sparse(cfg):
        if carry is not None and tuple(carry) != tuple(range(cfg.n_v_heads)):
            raise ValueError(f"gdn.dprod.stride / summary / conv with the carrying value heads {tuple(carry)!r}: not built together with a placement")
        return gdn_dprod_sparse.SparseSteps(d_model, cfg)
    if is_derived(cfg):
        if carry is not None and tuple(carry) != tuple(range(cfg.n_v_heads)):
            raise ValueError(f"gdn.dprod.key {cfg.dprod.key!r} with the carrying value heads {tuple(carry)!r}: the derived second step is built for every head of a layer")
        return DerivedSteps(d_model, cfg)
    if carry is None or len(carry) == cfg.n_v_heads:
        return DeltaProductSteps(d_model, cfg)
    return PartialSteps(d_model, cfg, tuple(carry))


def init_own_parameters(model: nn.Module, std: float) -> int:
    from .gdn_dprod_derived import DerivedSteps
    from .gdn_dprod_sparse import SparseSteps

    steps = [m for m in model.modules() if isinstance(m, (DeltaProductSteps, DerivedSteps, SparseSteps))]
    if steps:
        g = torch.Generator().manual_seed((torch.initial_seed() + SEED_OFFSET) % (1 << 63))
        for m in steps:
            m.reset_own(g, std)
    return len(steps)


def dprod_recurrence(q, k, v, g, beta, is_doc_start, S):
    """q (B, L, H, dk) at the value heads; k (B, L, n_h, H, dk); v (B, L, n_h, H, dv); g (B, L, H); beta (B, L, n_h, H)."""
    outs = []
    for q_t, k_t, v_t, g_t, b_t, s_t in zip(q.unbind(1), k.unbind(1), v.unbind(1), g.unbind(1), beta.unbind(1), is_doc_start.unbind(1)):
        S = S * (~s_t).to(S.dtype)[:, None, None, None]
        S = S * torch.exp(g_t)[:, :, None, None]
        for j in range(k.shape[2]):
            kj = k_t[:, j]
            S = S + torch.einsum("bhk,bhv->bhkv", kj, b_t[:, j, :, None] * (v_t[:, j] - torch.einsum("bhkv,bhk->bhv", S, kj)))
        outs.append(torch.einsum("bhkv,bhk->bhv", S, q_t))
    return torch.stack(outs, dim=1), S


def interleave(q, k, v, g, beta, is_doc_start):
    B, L, n_h = q.shape[0], q.shape[1], k.shape[2]
    flat = lambda t: t.reshape(B, n_h * L, *t.shape[3:])
    zq, zg, zs = torch.zeros_like(q), torch.zeros_like(g), torch.zeros_like(is_doc_start)
    return (flat(torch.stack([zq] * (n_h - 1) + [q], dim=2)), flat(k), flat(v), flat(torch.stack([g] + [zg] * (n_h - 1), dim=2)),
            flat(beta), flat(torch.stack([is_doc_start] + [zs] * (n_h - 1), dim=2)))


def last_substep(o: torch.Tensor, n_h: int) -> torch.Tensor:
    B, T = o.shape[:2]
    return o.reshape(B, T // n_h, n_h, *o.shape[2:])[:, :, n_h - 1]


def forward_partial(layer, x, ctx, state):
    """`forward` for a layer that carries some of its value heads (`PartialSteps`)."""
    cfg, steps = layer.cfg, layer.dprod
    B, L = ctx.doc.shape
    hk, hv, dk, dv = cfg.n_k_heads, cfg.n_v_heads, cfg.k_head_dim, cfg.v_head_dim
    hk_c, hv_c, n_x = steps.hk_c, steps.hv_c, steps.n_extra
    n_h = n_x + 1
    u_all = torch.cat([layer.in_proj_qkv(x), steps.in_proj_kv(x)], dim=-1)
    w_all = torch.cat([layer.conv_weight, steps.conv_weight], dim=0)
    if state is not None and state.conv_input.shape[-1] != u_all.shape[-1]:
        raise ValueError(f"this GDN cache holds {state.conv_input.shape[-1]} conv channels; Gated DeltaProduct n_h {n_h} on {hv_c} of "
                         f"{hv} value heads carries {u_all.shape[-1]}")
    hist, hist_doc = (None, None) if state is None else (state.conv_input, state.conv_doc)
    u, conv_input, conv_doc = ops.ref.causal_doc_conv(u_all, ctx.doc, w_all, hist, hist_doc)
    u = F.silu(u)
    q, k1, rest = torch.split(u, [hk * dk, hk * dk, u.shape[-1] - 2 * hk * dk], dim=-1)
    q = ops.ref.l2_normalize(q.reshape(B, L, hk, dk)) * dk ** -0.5
    k1 = ops.ref.l2_normalize(k1.reshape(B, L, hk, dk))
    parts = torch.split(rest, [hv * dv] + [hk_c * dk, hv_c * dv] * n_x, dim=-1)
    v1 = parts[0].reshape(B, L, hv, dv)
    xk = [ops.ref.l2_normalize(parts[1 + 2 * j].reshape(B, L, hk_c, dk)) for j in range(n_x)]
    xv = [parts[2 + 2 * j].reshape(B, L, hv_c, dv) for j in range(n_x)]
    g, beta1 = ops.ref.gdn_gates(layer.in_proj_a(x), layer.in_proj_b(x), layer.A_log, layer.dt_bias)
    xb = list((2 * torch.sigmoid(steps.in_proj_b(x))).reshape(B, L, n_x, hv_c).unbind(2))
    rv, rk, rvp, rkp = steps.runs_v, steps.runs_k, steps.runs_v_plain, steps.runs_k_plain
    dt = ops.ref.work_dtype(q)
    rep = hv // hk
    qc = take(q, rk, 2).repeat_interleave(rep, dim=2).to(dt)
    kc = torch.stack([take(k1, rk, 2)] + xk, dim=2).repeat_interleave(rep, dim=3).to(dt)
    vc = torch.stack([take(v1, rv, 2)] + xv, dim=2).to(dt)
    bc = torch.stack([2 * take(beta1, rv, 2)] + xb, dim=2).to(dt)        # step 1 of a carrying head writes with 2 sigmoid(b) too
    gc = take(g, rv, 2).to(dt)
    qp, kp = take(q, rkp, 2).repeat_interleave(rep, dim=2).to(dt), take(k1, rkp, 2).repeat_interleave(rep, dim=2).to(dt)
    vp, gp, bp = take(v1, rvp, 2).to(dt), take(g, rvp, 2).to(dt), take(beta1, rvp, 2).to(dt)
    S_all = x.new_zeros(B, hv, dk, dv, dtype=dt) if state is None else state.S.to(dt)
    S0c, S0p = take(S_all, rv, 1), take(S_all, rvp, 1)
    if cfg.kernel != "recurrence" and L > 1:
        qi, ki, vi, gi, bi, si = interleave(qc, kc, vc, gc, bc, ctx.is_doc_start)
        oi, S_c = ops.ref.chunked_delta_rule(qi, ki, vi, gi, bi, si, S0c, cfg.chunk_size)
        o_c = last_substep(oi, n_h)
        o_p, S_p = ops.ref.chunked_delta_rule(qp, kp, vp, gp, bp, ctx.is_doc_start, S0p, cfg.chunk_size)
    else:
        o_c, S_c = dprod_recurrence(qc, kc, vc, gc, bc, ctx.is_doc_start, S0c)
        o_p, S_p = ops.ref.delta_rule_recurrence(qp, kp, vp, gp, bp, ctx.is_doc_start, S0p)
    return merge(o_c, rv, o_p, rvp, 2), conv_input, conv_doc, merge(S_c, rv, S_p, rvp, 1)


def forward(layer, x, ctx, state):
    """The GDN layer's forward with the extra steps: (y, conv history over all channels, its document ids, S)."""
    if isinstance(layer.dprod, PartialSteps):
        return forward_partial(layer, x, ctx, state)
    cfg, steps = layer.cfg, layer.dprod
    B, L = ctx.doc.shape
    hk, hv, dk, dv = cfg.n_k_heads, cfg.n_v_heads, cfg.k_head_dim, cfg.v_head_dim
    n_x = steps.n_extra
    n_h = n_x + 1
    u_all = torch.cat([layer.in_proj_qkv(x), steps.in_proj_kv(x)], dim=-1)
    w_all = torch.cat([layer.conv_weight, steps.conv_weight], dim=0)
    if state is not None and state.conv_input.shape[-1] != u_all.shape[-1]:
        raise ValueError(f"this GDN cache holds {state.conv_input.shape[-1]} conv channels; Gated DeltaProduct n_h {n_h} carries {u_all.shape[-1]}")
    hist, hist_doc = (None, None) if state is None else (state.conv_input, state.conv_doc)
    u, conv_input, conv_doc = ops.ref.causal_doc_conv(u_all, ctx.doc, w_all, hist, hist_doc)
    u = F.silu(u)
    q, k1, rest = torch.split(u, [hk * dk, hk * dk, u.shape[-1] - 2 * hk * dk], dim=-1)
    q = ops.ref.l2_normalize(q.reshape(B, L, hk, dk)) * dk ** -0.5
    parts = torch.split(rest, [hv * dv] + [hk * dk, hv * dv] * n_x, dim=-1)
    ks = [ops.ref.l2_normalize(k1.reshape(B, L, hk, dk))] + [ops.ref.l2_normalize(parts[1 + 2 * j].reshape(B, L, hk, dk)) for j in range(n_x)]
    vs = [parts[2 * j].reshape(B, L, hv, dv) for j in range(n_x + 1)]
    boff, bmax = beta_offset(cfg), cfg.dprod.beta_max
    b1, bx = layer.in_proj_b(x), steps.in_proj_b(x)
    if boff is not None:
        b1, bx = b1 + boff, bx + boff
    g, beta1 = ops.ref.gdn_gates(layer.in_proj_a(x), b1, layer.A_log, layer.dt_bias)
    betas = [bmax * beta1] + list((bmax * torch.sigmoid(bx)).reshape(B, L, n_x, hv).unbind(2))
    rep = hv // hk
    dt = ops.ref.work_dtype(q)
    k = torch.stack(ks, dim=2).repeat_interleave(rep, dim=3).to(dt)
    v, beta = torch.stack(vs, dim=2).to(dt), torch.stack(betas, dim=2).to(dt)
    q, g = q.repeat_interleave(rep, dim=2).to(dt), g.to(dt)
    S0 = x.new_zeros(B, hv, dk, dv, dtype=dt) if state is None else state.S.to(dt)
    if cfg.kernel != "recurrence" and L > 1:
        qi, ki, vi, gi, bi, si = interleave(q, k, v, g, beta, ctx.is_doc_start)
        oi, S = ops.ref.chunked_delta_rule(qi, ki, vi, gi, bi, si, S0, cfg.chunk_size)
        o = last_substep(oi, n_h)
    else:
        o, S = dprod_recurrence(q, k, v, g, beta, ctx.is_doc_start, S0)
    return o, conv_input, conv_doc, S
