"""Token-superposition training: for the first phases of a run a position holds a BAG of s consecutive tokens (input =
the mean of their embeddings; loss = weighted cross-entropy against every token of the next bag), then the run switches
to plain next-token training (method: arXiv 2605.06546; reference: ced/train/tst.py).

Schedule `[[start_0 = 0, s_0], [start_1, s_1], ...]`: phase p covers optimizer steps start_p .. start_{p+1} - 1 at bag
size s_p. A step always has data.batch_size rows of data.seq_len positions; only what a position holds changes.

Data. The data source is a sequence of base rows (row g = L inputs and the last one's target). A bag step reads B s
base rows: bag row b of step k is the concatenation of base rows g .. g + s - 1, g = R(k) + b s, where
R(k) = sum over j < k of B s_j counts the base rows read before step k. Its (L + 1) s tokens are L bags of s inputs
followed by one more bag that is only a target; position j's targets are the s tokens of bag j + 1. A position belongs
to the document of its LAST input token and a target token is valid iff it lies in that document. With s = 1 this is
the base row itself, so `[[0, 1]]` is plain training bit for bit, and over a whole run every base row is read exactly
once, in order, across every switch (tests/test_tst.py). A next-token phase after a bag phase reads base rows from R(k).

The switch (start of step start_p, p > 0, before its batch): the optimizer's moments and step counter are reset (not
with `keep_optimizer_state`); weights, LR schedule, RNG and data position are untouched, so a checkpoint on either
side of the switch resumes into the uninterrupted run. Options, each off by default:

* gdn_decay_rescale: A_log += ln(s' / s) in every GDN layer, so the decay per TOKEN is unchanged when a position
  shrinks from s to s' tokens.
* gdn_resolution_gates ("decay" | "E"): instead, the forward receives the phase's s and scales the gates itself
  (models/gdn.py), so no surgery is needed; refused together with gdn_decay_rescale.
* gdn_conv_reinit: at a switch INTO next-token, every GDN layer's short-conv taps are drawn again from their
  initial distribution U(-1/sqrt(K), 1/sqrt(K)), layer by layer, from a counter generator of (seed, switch step) —
  a pure function of the two, so a resume into the switch draws the same numbers.
* bag_lr_power p: the LR of a bag phase of size s is the schedule's times s^p.
* rewarm_steps N: after a switch into next-token at step S the LR is the schedule's times (k - S + 1) / N for
  S <= k < S + N.
* token_scale_rope: the rotary position of a bag position is s times its index (models/attention.py).

Data parallelism: rank r reads bag rows r B / W .. (r + 1) B / W - 1 of the step (`batch_at(step, first, count)`); the
switch is a function of the step, made by every rank at the same update.
"""

from __future__ import annotations

import math

import torch

from ..data.synthetic import Batch, counter_generator

CONV_REINIT_STREAM = 7700


def bag_weights(s: int) -> torch.Tensor:
    """Uniform 1/s for s < 8, proportional to 1/i (i = 1..s, normalised) from 8 on."""
    if s < 8:
        return torch.full((s,), 1.0 / s)
    w = 1.0 / torch.arange(1, s + 1, dtype=torch.float64)
    return (w / w.sum()).float()


class TSTSchedule:
    def __init__(self, schedule: list):
        if not schedule:
            raise ValueError("tst.schedule is empty")
        self.phases = sorted((int(a), int(s)) for a, s in schedule)
        starts = [a for a, _ in self.phases]
        if starts[0] != 0 or len(set(starts)) != len(starts):
            raise ValueError("tst.schedule: phases start at distinct steps, the first at step 0")
        if any(s < 1 for _, s in self.phases):
            raise ValueError("tst.schedule bag sizes must be >= 1")

    def phase_of(self, step: int) -> int:
        return max(i for i, (a, _) in enumerate(self.phases) if step >= a)

    def s_at(self, step: int) -> int:
        return self.phases[self.phase_of(step)][1]

    def is_switch(self, step: int) -> bool:
        return step > 0 and any(step == a for a, _ in self.phases) and self.s_at(step) != self.s_at(step - 1)

    def last_switch_into_plain(self, step: int) -> int | None:
        """The latest switch step S <= step whose phase is next-token after a bag phase; None before any."""
        found = None
        for (a, s), (_, prev) in zip(self.phases[1:], self.phases[:-1]):
            if a <= step and s == 1 and prev > 1:
                found = a
        return found

    def rows_before(self, step: int, batch_size: int) -> int:
        """R(step): base rows read by the steps before `step`."""
        total = 0
        bounds = [a for a, _ in self.phases[1:]] + [step]
        for (a, s), b in zip(self.phases, bounds):
            total += max(0, min(b, step) - min(a, step)) * batch_size * s
        return total


def _row_block(data, first_row: int, n_rows: int):
    """Base rows first_row .. first_row + n_rows - 1 as (tokens, docs) of shape (n_rows, L + 1): the L inputs and the last
    one's target, with the target's document."""
    b = data.rows(first_row, n_rows)
    seq = torch.cat([b.tokens, b.targets[:, -1:]], dim=1)
    last_doc = torch.where(b.target_valid[:, -1], b.doc_ids[:, -1], b.doc_ids[:, -1] + 1)
    return seq, torch.cat([b.doc_ids, last_doc[:, None]], dim=1)


def bag_row(data, first_row: int, s: int) -> dict:
    """One bag row from base rows first_row .. first_row + s - 1: inputs (L, s), the positions' documents (L,), targets
    (L, s) and their validity (L, s)."""
    seq, docs = _row_block(data, first_row, s)
    L = seq.shape[1] - 1
    # documents keep increasing along the concatenation: a base row's documents follow the row before's
    shift = torch.cat([torch.zeros(1, dtype=docs.dtype), (docs[:-1, -1] + 1).cumsum(0)])
    flat, fdoc = seq.reshape(-1), (docs + shift[:, None]).reshape(-1)
    inputs, targets = flat[: L * s].view(L, s), flat[s:(L + 1) * s].view(L, s)
    pos_doc = fdoc[s - 1: L * s: s]
    valid = fdoc[s:(L + 1) * s].view(L, s) == pos_doc[:, None]
    return {"tokens": inputs, "doc_ids": pos_doc, "multi_targets": targets, "multi_valid": valid}


def gdn_layers(model) -> list:
    from ..models.gdn import GatedDeltaNet

    return [m for m in model.modules() if isinstance(m, GatedDeltaNet)]


def conv_reinit_draws(model, seed: int, step: int) -> list[torch.Tensor]:
    """What a conv re-initialisation at switch `step` writes into each GDN layer's taps, in module order."""
    g = counter_generator(seed, step, CONV_REINIT_STREAM)
    out = []
    for m in gdn_layers(model):
        bound = 1.0 / math.sqrt(m.cfg.conv_kernel)
        out.append(torch.empty(tuple(m.conv_weight.shape), dtype=torch.float32).uniform_(-bound, bound, generator=g))
    return out


class TSTPlan:
    """The schedule, the batches, the switch and the LR factor of a token-superposition run (built by the Trainer only
    when tst.schedule is set)."""

    def __init__(self, cfg_tst, data, vocab_size: int, batch_size: int | None = None, seed: int = 0):
        self.cfg, self.data, self.vocab, self.seed = cfg_tst, data, vocab_size, seed
        self.schedule = TSTSchedule(cfg_tst.schedule)
        self.B = batch_size if batch_size is not None else data.cfg.batch_size
        t = cfg_tst
        refused = [name for name, on in (("phase1_exclude_sources", bool(t.phase1_exclude_sources)), ("aux_multi_hot", bool(t.aux_multi_hot)),
                                         ("output_only", bool(t.output_only)), ("bag_input 'sum_sqrt'", t.bag_input != "mean")) if on]
        if refused:
            raise ValueError(f"tst options without an implementation in this framework: {', '.join(refused)}")
        if t.gdn_resolution_gates not in ("none", "decay", "E", "decay_beta"):
            raise ValueError(f"tst.gdn_resolution_gates {t.gdn_resolution_gates!r}: 'none', 'decay' or 'E'")
        if t.gdn_decay_rescale and t.gdn_resolution_gates != "none":
            raise ValueError("tst.gdn_decay_rescale and tst.gdn_resolution_gates both rescale the GDN decay for the bag size: one of them")
        if t.keep_optimizer_state and t.gdn_conv_reinit:
            raise ValueError("tst.keep_optimizer_state with tst.gdn_conv_reinit: the re-drawn taps would carry the old taps' moments")
        if t.keep_optimizer_state and len(self.schedule.phases) < 2:
            raise ValueError("tst.keep_optimizer_state needs a schedule with a switch")
        if type(t.rewarm_steps) is not int or t.rewarm_steps < 0:
            raise ValueError(f"tst.rewarm_steps {t.rewarm_steps!r}: an integer >= 0")
        if not hasattr(data, "rows"):
            raise ValueError("token superposition reads base rows by global index: the data source has no rows(first, count)")

    def s_at(self, step: int) -> int:
        return self.schedule.s_at(step)

    # ------------------------------------------------------------------ data
    def batch_at(self, step: int, first: int, count: int) -> Batch:
        """Rows first .. first + count - 1 of step `step`'s B rows."""
        s = self.s_at(step)
        g0 = self.schedule.rows_before(step, self.B)
        if s == 1:
            return self.data.rows(g0 + first, count)
        rows = [bag_row(self.data, g0 + b * s, s) for b in range(first, first + count)]
        stack = lambda k: torch.stack([r[k] for r in rows]).contiguous()
        mv = stack("multi_valid")
        doc = stack("doc_ids")
        mt = stack("multi_targets")
        return Batch(tokens=stack("tokens"), targets=mt[..., 0].contiguous(), target_valid=mv[..., 0].contiguous(), doc_ids=doc,
                     multi_targets=mt, multi_valid=mv, single_doc=bool((doc == doc[:, :1]).all()) and bool(mv.all()))

    # ------------------------------------------------------------------ the switch
    @torch.no_grad()
    def switch(self, trainer, step: int) -> dict | None:
        """At a switch step, before its batch: the optimizer reset and the optional surgery. Returns the event record
        (None at every other step). A pure function of the step and the run's seed: every rank makes it at the same update and a
        resume into the switch step makes it again."""
        if not self.schedule.is_switch(step):
            return None
        t = self.cfg
        if getattr(trainer, "zero", None) is not None:
            trainer.zero.settle()        # parameter writes of the step before (a side stream under the fused step) have landed
        s_old, s_new = self.s_at(step - 1), self.s_at(step)
        event = {"step": step, "s_from": s_old, "s_to": s_new, "keep_optimizer_state": bool(t.keep_optimizer_state)}
        if t.gdn_decay_rescale:
            for m in gdn_layers(trainer.model):
                m.A_log.add_(math.log(s_new / s_old))
            event["gdn_decay_rescaled"] = len(gdn_layers(trainer.model))
        if t.gdn_conv_reinit and s_new == 1:
            layers = gdn_layers(trainer.model)
            for m, w in zip(layers, conv_reinit_draws(trainer.model, self.seed, step)):
                m.conv_weight.copy_(w.to(device=m.conv_weight.device, dtype=m.conv_weight.dtype))
            event["gdn_conv_reinit"] = len(layers)
        if t.gdn_decay_rescale or (t.gdn_conv_reinit and s_new == 1):
            trainer.flat.refresh_lp()
        if not t.keep_optimizer_state:
            trainer.optimizer.reset_moments()
            event["optimizer_states_reset"] = len(trainer.flat.segments)
        else:
            event["optimizer_states_reset"], event["optimizer_states_kept"] = 0, len(trainer.flat.segments)
        return event

    def lr_factor(self, step: int) -> float | None:
        """What multiplies the schedule's LR at `step`: s^p in a bag phase (bag_lr_power), the ramp after a switch into
        next-token (rewarm_steps); None where neither acts."""
        t = self.cfg
        s = self.s_at(step)
        if s > 1:
            return float(s) ** float(t.bag_lr_power) if t.bag_lr_power else None
        if t.rewarm_steps:
            S = self.schedule.last_switch_into_plain(step)
            if S is not None and S <= step < S + t.rewarm_steps:
                return (step - S + 1) / t.rewarm_steps
        return None

    def data_state(self) -> dict:
        return {"tst_schedule": [list(p) for p in self.schedule.phases]}
