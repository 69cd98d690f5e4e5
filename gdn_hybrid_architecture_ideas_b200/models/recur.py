"""A looped middle of the stack (`loop.recur_layers: [first, end]`): the layers first .. end - 1 run T times with the same
weights, between a prelude (layers 0 .. first - 1, once) and a coda (layers end .. N - 1, once).

    p   = Prelude(x0)                      x0: the embedding's output
    z_k = Middle(u_k),  k = 1 .. T         every pass with its own GDN states and K/V over the whole chunk
    out = Coda(z_T)

What pass k reads (`loop.injection`):

  "none"       u_1 = p, u_k = z_{k-1}: the plain stack with its middle repeated (tied weights); no tensor is added.
  "mix"        u_1 = p, u_k = w p + (1 - w) z_{k-1} for k >= 2 with ONE learned scalar w (`encoder.recur_mix`, 0-dim, starts at
               `loop.recur_mix_init`). At T = 1 the model is the plain stack bit for bit; at w = 1 a later pass repeats the
               first.
  "parcae"     the diagonal injection: e = RMSNorm(p) (`loop.recur_prelude_norm`), z_0 = 0 or e (`loop.recur_state_init`),
               u_k = decay * z_{k-1} + dt * (B e) with dt = softplus(dt_bias), decay = exp(-dt exp(A_log)) per channel and B a
               d x d matrix ("dense") or a vector ("diag"); A = -exp(A_log) < 0 whatever the parameters, so the linear part of
               the recurrence contracts. Starts at decay = `loop.parcae_init_decay`, B the identity.
  "depth_mix"  every pass reads a softmax mix, per position, over its candidates V_1 = [x0, p], V_k = [x0, p, z_1 .. z_{k-1}]:
               one depth reader for all passes (a (d,) pseudo-query and the gain of its key norm, zeros at the start:
               `encoder.recur_depth`), so at its start every candidate has equal weight and the model is not the plain stack
               even at T = 1.

A pass takes from the one before only its output stream, position by position: causality and the cache of a chunk are the
layers' own. A cached sequence holds one entry per layer APPLICATION, first + T (end - first) + N - end of them in running
order, and keeps the T it was prefilled with. T is an argument of the forward (default `loop.t_eval`); training draws one T
per optimizer step from `loop.t_choices` / `loop.t_probs`. Full backpropagation through all passes.
Reference: ced/model/control.py:104-151, ced/model/encoder.py:143-175 and 1017-1134, ced/model/loop.py:58-121,
ced/model/recur_depth.py.
"""

from __future__ import annotations

import math

import torch
import torch.nn as nn
import torch.nn.functional as F

T_SAMPLINGS = ("step", "sequence")
INJECTIONS = ("none", "mix", "parcae", "depth_mix")
B_FORMS = ("dense", "diag")
STATE_INITS = ("zeros", "prelude")
MIN_RATE, MAX_RATE = 1e-7, 30.0          # dt exp(A_log) is clamped here before the exp: decay stays inside (0, 1) as a float too


def is_on(cfg) -> bool:
    return bool(cfg.loop.recur_layers)


def check_config(cfg) -> None:
    """Refuses, by key, a looped middle that cannot be built, and its keys set on a model without one."""
    lc, enc = cfg.loop, cfg.encoder
    fresh = type(lc)()
    r = tuple(lc.recur_layers)
    if not r:
        if lc.injection in ("mix", "depth_mix"):
            raise ValueError(f"model.loop.injection {lc.injection!r} belongs to a looped middle (model.loop.recur_layers): this model has none")
        if lc.recur_mix_init != fresh.recur_mix_init or lc.t_sampling != "step":
            raise ValueError("model.loop.recur_mix_init / t_sampling are read with model.loop.recur_layers: this model has no looped middle")
        return
    n = enc.n_layers
    if not (len(r) == 2 and all(type(i) is int for i in r) and 0 <= r[0] < r[1] <= n):
        raise ValueError(f"model.loop.recur_layers {list(r)!r}: [first, end] with 0 <= first < end <= {n} (the layers first .. end - 1 loop)")
    if lc.injection not in INJECTIONS:
        raise ValueError(f"model.loop.injection {lc.injection!r} with a looped middle: one of {INJECTIONS}")
    if lc.t_sampling not in T_SAMPLINGS:
        raise ValueError(f"model.loop.t_sampling {lc.t_sampling!r}: one of {T_SAMPLINGS} (one pass count per optimizer step, or one per row)")
    if lc.t_sampling == "sequence" and lc.injection == "depth_mix":
        raise ValueError("model.loop.t_sampling 'sequence' (a pass count per row) is not built together with model.loop.injection 'depth_mix'")
    clashes = {"model.encoder.attn_res": enc.attn_res != "none", "model.encoder.layer_scalars": enc.layer_scalars != "none",
               "model.encoder.canon_kernel": bool(enc.canon_kernel), "model.nvfp4.mode": cfg.nvfp4.mode != "none",
               "model.encoder.attention.normalizer 'asentmax'": enc.attention.normalizer != "softmax", "model.mtp.enabled": bool(cfg.mtp.enabled)}
    hit = [k for k, v in clashes.items() if v]
    if hit:
        raise ValueError(f"model.loop.recur_layers is not built together with: {', '.join(hit)}")
    if lc.injection == "depth_mix" and r[0] == 0:
        raise ValueError("model.loop.injection 'depth_mix' reads the embedding's output and the prelude's output as two candidates: "
                         "give the middle a prelude of at least one layer (first >= 1)")
    if lc.injection != "mix" and lc.recur_mix_init != fresh.recur_mix_init:
        raise ValueError("model.loop.recur_mix_init is the start of injection 'mix': leave it at its default otherwise")
    if lc.injection == "parcae":
        if lc.recur_inject_b not in B_FORMS or lc.recur_state_init not in STATE_INITS:
            raise ValueError(f"model.loop.recur_inject_b {lc.recur_inject_b!r} of {B_FORMS}; recur_state_init {lc.recur_state_init!r} of {STATE_INITS}")
        if not 0.0 < float(lc.parcae_init_decay) < 1.0:
            raise ValueError(f"model.loop.parcae_init_decay {lc.parcae_init_decay!r}: a decay in (0, 1)")
    for name, t in (("t_eval", lc.t_eval), *((f"t_choices[{i}]", t) for i, t in enumerate(lc.t_choices))):
        if type(t) is not int or t < 1:
            raise ValueError(f"model.loop.{name} {t!r}: a pass count >= 1")
    if len(lc.t_choices) != len(lc.t_probs) or not lc.t_choices or min(lc.t_probs) < 0 or sum(lc.t_probs) <= 0:
        raise ValueError("model.loop.t_choices / t_probs: equally long, non-empty, probabilities >= 0 with a positive sum")


class RecurInjection(nn.Module):
    """u = decay * h + dt * (B e) per channel; see the module docstring. No random number is drawn when it is built."""

    def __init__(self, d_model: int, init_decay: float, b_form: str = "dense"):
        super().__init__()
        step = -math.log(init_decay)
        self.b_form = b_form
        self.A_log = nn.Parameter(torch.zeros(d_model))
        self.dt_bias = nn.Parameter(torch.full((d_model,), step + math.log(-math.expm1(-step))))       # softplus^-1(step)
        self.B = nn.Parameter(torch.eye(d_model) if b_form == "dense" else torch.ones(d_model))

    def coefficients(self) -> tuple[torch.Tensor, torch.Tensor]:
        dt = F.softplus(self.dt_bias)
        return torch.exp(-(dt * torch.exp(self.A_log)).clamp(MIN_RATE, MAX_RATE)), dt

    def forward(self, h: torch.Tensor | None, e: torch.Tensor) -> torch.Tensor:
        """h None: the state is zero (the first pass under state init "zeros") and the decay term is not formed."""
        with torch.autocast(device_type=e.device.type, enabled=False):
            decay, dt = (t.to(e.dtype) for t in self.coefficients())
            B = self.B.to(e.dtype)
            driven = dt * (F.linear(e, B) if self.b_form == "dense" else e * B)
            return driven if h is None else decay * h + driven

    @torch.no_grad()
    def summary(self) -> dict:
        decay, dt = (t.double().cpu() for t in self.coefficients())
        B = self.B.detach().double().cpu()
        start = torch.eye(B.shape[0], dtype=B.dtype) if self.b_form == "dense" else torch.ones_like(B)
        span = lambda t: [round(float(t.min()), 6), round(float(t.mean()), 6), round(float(t.max()), 6)]
        return {"decay": span(decay), "dt": span(dt), "b_drift": round(float((B - start).norm() / start.norm()), 6),
                "b_size": round(float(B.norm() / start.norm()), 6)}


def input_mix(e: torch.Tensor, h: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """w e + (1 - w) h as one lerp in at least float32, outside autocast: exact at w = 1 (returns e) and w = 0 (returns h)."""
    dt = torch.promote_types(h.dtype, torch.float32)
    with torch.autocast(device_type=h.device.type, enabled=False):
        return torch.lerp(h.to(dt), e.to(dt), w.to(dt)).to(h.dtype)


def cache_length(recur: tuple[int, int], n_layers: int, T: int) -> int:
    first, end = recur
    return first + T * (end - first) + (n_layers - end)


def pass_count_for_step(loop, seed: int, step: int) -> int:
    """The T of an optimizer step: one draw from t_choices with weights t_probs out of a counter-based generator of
    (seed, step), the same on every rank and after a resume."""
    from ..data.synthetic import counter_generator

    if len(loop.t_choices) == 1:
        return int(loop.t_choices[0])
    g = counter_generator(seed, step, 1)
    i = int(torch.multinomial(torch.tensor(loop.t_probs, dtype=torch.float64), 1, generator=g))
    return int(loop.t_choices[i])


def rows_by_count(loop, batch_size: int) -> list:
    """`t_sampling: sequence`: the pass counts a step's rows hold, t_probs[i] x batch_size rows of t_choices[i] in the
    order of t_choices; refused unless every product is a whole number and they add up to the batch."""
    held = []
    for t, share in zip(loop.t_choices, loop.t_probs):
        rows = share * batch_size
        if round(rows) < 0 or abs(rows - round(rows)) > 1e-9:
            raise ValueError(f"model.loop.t_sampling 'sequence': t_probs {list(loop.t_probs)!r} x data.batch_size {batch_size} must be whole numbers of rows "
                             f"(T = {t}: {rows})")
        held.extend([int(t)] * round(rows))
    if len(held) != batch_size:
        raise ValueError(f"model.loop.t_sampling 'sequence': t_probs {list(loop.t_probs)!r} give {len(held)} rows of data.batch_size {batch_size} (they must sum to 1)")
    return held


def row_pass_counts(held: list, seed: int, step: int) -> list:
    """The pass count of every row of a step's batch, in row order: the step's multiset `held` dealt to the rows through
    a permutation out of the counter-based generator of (seed, step), so a resume needs only the step."""
    from ..data.synthetic import counter_generator

    deal = torch.randperm(len(held), generator=counter_generator(seed, step, 2)).tolist()
    counts = [0] * len(held)
    for slot, row in enumerate(deal):
        counts[row] = held[slot]
    return counts


def micro_plan(counts: list, rows_per_forward) -> list:
    """[(rows, T)]: the rows of each pass count (ascending T, rows in batch order) in groups of rows_per_forward(T); every
    forward has one T, and the groups' shapes are the same at every step because the multiset is."""
    plan = []
    for t in sorted(set(counts)):
        rows = [i for i, c in enumerate(counts) if c == t]
        size = rows_per_forward(t)
        plan.extend((rows[lo:lo + size], t) for lo in range(0, len(rows), size))
    return plan


def mean_pass_count(loop) -> float:
    return sum(t * p for t, p in zip(loop.t_choices, loop.t_probs)) / sum(loop.t_probs)
