"""Checkpoint cross-read (CCR, `model.encoder.gdn_ccr_spacing` = C > 0): a GDN layer also reads another GDN layer's state
as it was at the last multiple of C tokens of the document.

The checkpoint of a token at position p of its document is the source layer's state after the document's first
C floor(p / C) tokens (zero for p < C). A reader adds to its delta-rule output, before the gated output norm,

    o_t  +=  gate (*) ( S^src_ckpt(t) )^T q_t         gate (H_v,), q_t the reader's own normalised, scaled query

value head j reading key head j // (H_v / H_k). `gdn_ccr_target` names the source: "previous" (the GDN layer before the
reader), "lowest" (the stack's first GDN layer), "group_first" (the first GDN layer of the reader's group of
full_attn_interval layers). `gdn_ccr_translator: key_head` puts a d_k x d_k matrix M per key head between the query and
the read, stored as D = M - I (zeros) and applied as q + q D^T, so the start is the read without it bit for bit.
`gdn_ccr_gate_init` is the gates' start, `gdn_ccr_gate_floor` a lower bound the trainer holds them at after every step.

How it is formed here. A document of a row changes checkpoint only after a token whose position p has (p + 1) % C == 0,
and a call of L tokens holds at most L // C + 1 of those. The writer runs the delta rule once and takes the state after
exactly those tokens (`ops.reference.delta_rule_picks`: in the chunked form one small product per pick from the chunk's
own operands), so its record is K + 2 states a row: slot 0 zeros, slot 1 the checkpoint carried by the cache, slots
2.. the picks in order, with one slot index per position. No state per position is formed. The reader gathers by slot in
blocks of positions. Shapes depend on (B, L, C) only. A cached forward carries one more tensor per writer, the
checkpoint the next token reads (`GDNState.ckpt`).

Reference: ced/model/gdn_arms.py:100-160 (the definition), :212-262 (sources / writers), :265-345 (refusals),
:981-1185 (records and reads; there a state per position off the fused path, and the kernel's chunk-start states on it).
"""

from __future__ import annotations

import math
from dataclasses import dataclass

import torch

TARGETS = ("previous", "lowest", "group_first")
TRANSLATORS = ("none", "key_head")
CHECKPOINT_MODES = ("none", "layer")
READ_BLOCK_BYTES = 256 << 20       # the gathered states of one block of positions stay under this


def on(cfg) -> bool:
    return cfg.encoder.gdn_ccr_spacing != 0


def gdn_layers(cfg) -> list[int]:
    return [i for i, kind in enumerate(cfg.encoder.layer_kinds()) if kind == "gdn"]


def sources(cfg) -> dict[int, int]:
    """{reader layer: the layer it reads}, in stack order; {} with CCR off."""
    if not on(cfg):
        return {}
    gdn, target = gdn_layers(cfg), cfg.encoder.gdn_ccr_target
    if target == "previous":
        return {gdn[n]: gdn[n - 1] for n in range(1, len(gdn))}
    if target == "lowest":
        return {i: gdn[0] for i in gdn[1:]}
    S, first, out = cfg.encoder.full_attn_interval, {}, {}
    for i in gdn:
        if i // S in first:
            out[i] = first[i // S]
        else:
            first[i // S] = i
    return out


def writers(cfg) -> list[int]:
    return sorted(set(sources(cfg).values()))


def check_config(cfg) -> None:
    """ValueError, by name, for a bad value and for what CCR is not built with."""
    e = cfg.encoder
    C = e.gdn_ccr_spacing
    if isinstance(C, bool) or not isinstance(C, int) or C < 0:
        raise ValueError(f"model.encoder.gdn_ccr_spacing {C!r}: 0 (off) or a positive spacing in tokens")
    if e.gdn_ccr_target not in TARGETS:
        raise ValueError(f"model.encoder.gdn_ccr_target {e.gdn_ccr_target!r}: one of {TARGETS}")
    if e.gdn_ccr_translator not in TRANSLATORS:
        raise ValueError(f"model.encoder.gdn_ccr_translator {e.gdn_ccr_translator!r}: one of {TRANSLATORS}")
    gi, gf = e.gdn_ccr_gate_init, e.gdn_ccr_gate_floor
    for name, x, low in (("gdn_ccr_gate_init", gi, -math.inf), ("gdn_ccr_gate_floor", gf, 0.0)):
        if isinstance(x, bool) or not isinstance(x, (int, float)) or not math.isfinite(x) or x < low:
            raise ValueError(f"model.encoder.{name} {x!r}: a finite number" + (" >= 0 (0.0: no floor)" if low == 0.0 else ""))
    if not on(cfg):
        if (e.gdn_ccr_target, e.gdn_ccr_translator) != ("previous", "none") or gi != 0 or gf != 0:
            raise ValueError("model.encoder.gdn_ccr_target / gdn_ccr_translator / gdn_ccr_gate_init / gdn_ccr_gate_floor are read with "
                             "model.encoder.gdn_ccr_spacing > 0 (CCR on); with CCR off leave them at their defaults")
        return
    what = f"model.encoder.gdn_ccr_spacing {C!r}"
    if gf != 0 and gf > gi:
        raise ValueError(f"model.encoder.gdn_ccr_gate_floor {gf!r} is above model.encoder.gdn_ccr_gate_init {gi!r}: the gates would start below their floor")
    if e.attn_res not in ("none", "block_entry"):
        raise ValueError(f"{what} is built with model.encoder.attn_res 'none' or 'block_entry', not {e.attn_res!r}")
    if cfg.loop.recur_layers:
        raise ValueError(f"{what} is built for one pass through the stack (no loop.recur_layers): another pass would need records of its own")
    if e.layer_scalars != "none" or e.canon_kernel:
        raise ValueError(f"{what} is not built together with model.encoder.layer_scalars or canon_kernel")
    if cfg.fp8.mode != "none" or cfg.nvfp4.mode != "none":
        raise ValueError(f"{what} is not built together with model.fp8 / model.nvfp4")
    if cfg.mtp.enabled:
        raise ValueError(f"{what} is not built together with model.mtp (its drafter computes the GDN layers itself)")
    g = e.gdn
    if g.kda.decay != "scalar" or g.erase.mode != "none" or g.dprod.n_h != 1:
        raise ValueError(f"{what} is not built together with gdn.kda.decay 'channel', gdn.erase.mode 'eda' or gdn.dprod.n_h >= 2")
    if e.gdn_write_variant != "none" and e.gdn_write_mix != "none":
        raise ValueError(f"{what} is not built together with model.encoder.gdn_write_variant {e.gdn_write_variant!r}: nothing tests the pair")
    if e.gdn_shape_by_layer:
        raise ValueError(f"{what} is not built together with model.encoder.gdn_shape_by_layer: a reader's heads are its source's")
    if not sources(cfg):
        raise ValueError(f"model.encoder.gdn_ccr_target {e.gdn_ccr_target!r}: no GDN layer reads another in this stack "
                         f"(GDN layers {gdn_layers(cfg)}, full_attn_interval {e.full_attn_interval})")


@dataclass
class Record:
    """What a writer hands its readers. states (B, K + 2, H_v, d_k, d_v): slot 0 zeros, slot 1 the cache's checkpoint, then
    the picks; slot (B, L): the slot each position reads; source: the writer's layer index."""

    states: torch.Tensor
    slot: torch.Tensor
    source: int | None = None


def picks_and_slots(pos: torch.Tensor, C: int):
    """From the positions in the document (B, L): picks (B, K) the call indices after which a checkpoint is taken, in
    order, L for an unused entry (K = L // C + 1); slot (B, L) per position; next_slot (B,) for the token after the call.

    Position t with r = pos_t mod C reads the state after call index j = t - r - 1: the zeros if pos_t - r = 0 (the
    document's first C tokens), the cache's checkpoint if j < 0 (the document began before the call), else the pick at
    j, whose rank among the row's picks is the number of pick tokens before it."""
    B, L = pos.shape
    K = L // C + 1
    dev = pos.device
    take = (pos + 1) % C == 0
    order = torch.where(take, torch.arange(L, device=dev)[None, :], torch.full_like(pos, L)).sort(dim=1).values
    picks = order[:, :K] if K <= L else torch.nn.functional.pad(order, (0, K - L), value=L)
    rank = take.long().cumsum(1) - 1                             # at a pick token: its rank

    def slot_of(p, j):                                           # p: position in the document; j: call index of the token before its checkpoint
        r = p % C
        at = torch.gather(rank, 1, j.clamp(min=0))
        s = torch.where(j >= 0, at + 2, torch.ones_like(at))
        return torch.where(p - r > 0, s, torch.zeros_like(s))

    t = torch.arange(L, device=dev)[None, :].expand(B, L)
    slot = slot_of(pos, t - pos % C - 1)
    p1 = pos[:, -1:] + 1
    next_slot = slot_of(p1, L - p1 % C - 1)[:, 0]
    return picks, slot, next_slot


def write(q, k, v, g, beta, ctx, S0, ckpt0, C: int, kernel: str, chunk_size: int, source: int):
    """The writer's delta rule. q, k already repeated to the value heads. Returns (o, S, Record, the checkpoint the token
    after this call reads (B, H, d_k, d_v))."""
    from ..ops import reference as ref

    picks, slot, next_slot = picks_and_slots(ctx.pos, C)
    o, S, taken = ref.delta_rule_picks(q, k, v, g, beta, ctx.is_doc_start, S0, picks, kernel, chunk_size)
    zero = torch.zeros_like(taken[:, :1])
    before = zero if ckpt0 is None else ckpt0[:, None].to(taken.dtype)
    states = torch.cat([zero, before, taken], dim=1)
    nxt = states[torch.arange(states.shape[0], device=states.device), next_slot]
    return o, S, Record(states=states, slot=slot, source=source), nxt


def translate_query(arms, q: torch.Tensor) -> torch.Tensor:
    """q_x = M_h q for every position and key head, formed as q + q D_h^T (exactly q at D = 0)."""
    if arms.translator == "none":
        return q
    D = arms.ccr_translator_delta
    return q + torch.einsum("...hk,hjk->...hj", q, D.to(q.dtype)).to(q.dtype)


def read(arms, rec: Record, q: torch.Tensor, hv: int) -> torch.Tensor:
    """The reader's cross term before its gate: (B, L, H_v, d_v) = ckpt(t)^T q_x,t. q (B, L, H_k, d_k)."""
    if rec.source is not None and rec.source != arms.ccr_source:
        raise ValueError(f"layer {arms.layer} reads layer {arms.ccr_source}'s checkpoints (gdn_ccr_target {arms.ccr_target!r}); it was handed layer {rec.source}'s")
    q = translate_query(arms, q)
    B, L, hk, dk = q.shape
    states = rec.states
    qr = q.repeat_interleave(hv // hk, dim=2).to(states.dtype)
    per_pos = states[0, 0].numel() * states.element_size() * B
    step = max(1, min(L, READ_BLOCK_BYTES // max(per_pos, 1)))
    rows = torch.arange(B, device=q.device)[:, None]
    out = [torch.einsum("blhkv,blhk->blhv", states[rows, rec.slot[:, lo:lo + step]], qr[:, lo:lo + step]) for lo in range(0, L, step)]
    return (out[0] if len(out) == 1 else torch.cat(out, dim=1)).contiguous()


@torch.no_grad()
def floor_gates_(encoder) -> None:
    """After an optimizer step: every reader's gate clamped in place to at least its floor (no host read)."""
    for layer in encoder.layers:
        arms = getattr(layer, "gdn_arms", None)
        if arms is not None and arms.ccr_read and arms.gate_floor:
            arms.ccr_gate.clamp_(min=arms.gate_floor)


def take_record(cache):
    """(the record a layer's call left in its new cache entry, the entry without it)."""
    if cache is None:
        return None, None
    rec, cache.ccr = cache.ccr, None
    return rec, cache


class Walk:
    """The record handed down the stack: a writer's own record replaces the one held, a layer that writes none leaves it
    (under "previous" the layer's own always replaces it: the chain), and only a reader is called with it."""

    def __init__(self):
        self.rec = None

    def record_in(self, arms):
        return self.rec if arms.ccr_read else None

    def hand_record(self, arms, own) -> None:
        if arms.ccr_write or arms.ccr_target == "previous":
            self.rec = own
        elif own is not None:
            raise RuntimeError("a GDN layer that no reader reads made a CCR record")

    def hand(self, arms, cache):
        own, cache = take_record(cache)
        self.hand_record(arms, own)
        return cache
