"""The Copy-Paste head (`model.cp_head.enabled`): a pointer over the context mixed into the next-token distribution.

    h_t   the final norm's output (the LM head's input);  q_t = W_Q h_t, k_tau = W_K h_tau (d_c wide), a sink key k_sink
    e_tau = q_t . k_tau / sqrt(d_c) over tau <= t of t's document,  e_sink = q_t . k_sink / sqrt(d_c)
    s_t   = softmax over {sink} u ctx at the sink;   alpha_t = softmax over ctx alone
    p_CP(v) = sum of alpha_t(tau) over tau with x_tau = v
    c_t   = softmax over V u {<copy>} at <copy>, the <copy> logit z_copy = w_copy . h_t (a vector of its own, never a token)
    lambda_t = c_t (1 - s_t);    p(v) = (1 - lambda_t) p_LM(v) + lambda_t p_CP(v);   loss: cross entropy on p

Everything is formed in log space and nothing of size T x T x V exists: the training terms (`terms`, a `Pointer`) are
(log s, log(1 - s), log p_CP(target)) by blocks of queries against the keys up to the block's end, masks by comparisons
and `where` (fixed shapes); a query without a matching key gives log p_CP = -inf with a gradient of exactly zero. The
mixture at the target is `mixture_log_prob`. At inference `forward_logits` returns log p over V (p_CP over V by a
scatter-add of alpha, per block of queries), so every reader of logits reads the mixture; `score: lm` returns p_LM's
logits instead. Cached generation keeps, per earlier position, its key, token, document and index (`CopyCache`); a chunk
appends its own before its queries read (tau = t included).

Options built: `qk_norm` (q and k RMS-normed over d_c at eps 2^-23, q times 1 + `qk_gain`), `init: spec` (every tensor
N(0, init_std)) / `reference` (W_Q, W_K U(+-sqrt(3 / d)), the sink N(0, 1 / d_c)), the length rule (`temperature: ssmax`:
q times ln(n_t) / ln(ref); `sink_count`: e_sink + ln(n_t / ref); n_t the context positions a query sees, ref the global
layers' temperature_ref_len), `force_lambda_zero`, `query_chunk`, a band (`window` W: a query sees the W latest context
positions; without the length rule, which counts them all), and the pointer that reads the depth sources
(`pointer_input: mix`, on a block-entry stack: x^q and x^k are two depth reads of their own over the finished blocks
[b_0 .. b_N], each through a norm of its own, readers and norms zeros at the start so that both start as the stream's mean
read; q = W_Q x^q, k = W_K x^k, the <copy> row and the LM head still read h; `cp_head.mix.*`). The tensors are registered
after every other tensor and drawn from a generator of their own, so the base model starts as the model without the key.
`train_mode: aux` (on the `mix` pointer): nothing is mixed into the prediction; the pointer has no <copy> row and learns from
its own loss alone, L_aux(t) = -log of the pointer's mass on the context positions holding the next token (= -(log p_CP(y) +
log(1 - s))), or -log s where the next token is not in the context, added to p_LM's loss at `aux_weight`; in eval mode the
pointer is dropped (logits are p_LM's, no copy cache), so every scorer reads the model without the head (`aux_terms`).
`train_mode: addon` (on the `mix` pointer): the head is the mixture head and every evaluation reads the mixture; in training
the trunk and the LM head learn from p_LM's loss alone, and the head from the mixture's CE in which p_LM's numbers (LSE_V,
log p_LM(y)), the <copy> row's input h and the readers' sources are all detached, so no gradient of the mixture reaches a
trunk tensor (`addon_loss`); the trainer clips the two parts by their own norms.
Refused by name: the copy from the trunk's own attention (`trunk_copy`), the fused kernel. Several pointer
heads (`n_heads` H on the `mix` pointer with `qk_norm`): head h has its own pair of depth reads (`cp_head.mix.heads.<h>`), its
own rows h d_c .. (h + 1) d_c - 1 of W_Q / W_K, its own norm over d_c, gain and slice of the sink key; q and k are held flat
(H d_c) and scored at 1 / sqrt(d_c), which sums the heads' scores into one logit a position, one softmax; head 0 and the
<copy> row are drawn first, so they are the one-head pointer's of the same seed. `combine: or` keeps the heads apart: head h
has its own s_h, alpha_h, p_CP,h, and a router pi_t = softmax_h(W_route h_t) (`head_router`, zeros: uniform) mixes the
heads' distributions over {sink} u ctx: log s = LSE_h(log pi_h + log s_h), log(1 - s) = LSE_h(log pi_h + log(1 - s_h)),
w_h = pi_h (1 - s_h) / (1 - s), p_CP = sum_h w_h p_CP,h; at one head log pi = 0 and the router is never read.
Reference: ced/model/cp_head.py:1-100 (the form), :454-660 (the module), :899-1016 (length rule, block terms),
:1223-1245 (mixture), :1282-1370 (inference), :1443-1483 (cache).
"""

from __future__ import annotations

import math
import os
from dataclasses import dataclass, fields
from functools import partial
from typing import NamedTuple

import torch
import torch.nn as nn
import torch.nn.functional as F
from torch.utils.checkpoint import checkpoint as recompute

OWN_SEED_OFFSET = 0xC0_2610_19247        # shared with the reference: equal starts under equal seeds
NORM_EPS = 2.0 ** -23
BASE_FORM = dict(trunk_copy="none", kernel="reference")
COMBINES = ("and", "or")
TRAIN_MODES = ("mixture", "aux", "addon")
POINTER_INPUTS = ("final", "mix", "shared")
SOURCES_KEY = "cp_pointer_sources"       # where a block-entry stack leaves [b_0 .. b_N] for the pointer's readers (SeqContext.memo)
CHOICES = dict(init=("spec", "reference"), score=("mixture", "lm"), temperature=("none", "ssmax"))
ENV_SCORE = "GHB_CP_SCORE"               # a scoring process's override of model.cp_head.score


def check_config(cfg) -> None:
    head = cfg.cp_head
    if not head.enabled:
        return
    off_base = [f"{name} {getattr(head, name)!r}" for name, base in BASE_FORM.items() if getattr(head, name) != base]
    if off_base:
        raise ValueError(f"model.cp_head {', '.join(off_base)}: the head is built without the trunk copy, kernel 'reference'")
    if head.combine not in COMBINES:
        raise ValueError(f"model.cp_head.combine {head.combine!r}: one of {COMBINES}")
    if head.combine == "or" and (head.pointer_input != "mix" or not head.qk_norm or head.window or head.sink_count or head.train_mode != "mixture"
                                 or cfg.encoder.gdn_write_mix != "none"):
        raise ValueError("model.cp_head.combine 'or' (the heads mixed by a router) is built on the pointer on depth reads with qk_norm, without window or "
                         "sink_count, train_mode 'mixture', model.encoder.gdn_write_mix 'none'")
    if type(head.n_heads) is not int or head.n_heads < 1:
        raise ValueError(f"model.cp_head.n_heads {head.n_heads!r}: the pointer's heads, an integer >= 1")
    if head.n_heads > 1:
        single = {"pointer_input 'mix'": head.pointer_input == "mix", "qk_norm true (each head's own gain)": bool(head.qk_norm), "no window": not head.window,
                  "no sink_count": not head.sink_count, "train_mode 'mixture'": head.train_mode == "mixture",
                  "model.encoder.gdn_write_mix 'none'": cfg.encoder.gdn_write_mix == "none"}
        missing = [k for k, ok in single.items() if not ok]
        if missing:
            raise ValueError(f"model.cp_head.n_heads {head.n_heads} is built with: {', '.join(missing)}")
    if head.train_mode not in TRAIN_MODES:
        raise ValueError(f"model.cp_head.train_mode {head.train_mode!r}: built are {TRAIN_MODES} (the mixture's loss; the pointer's own auxiliary loss)")
    weight = head.aux_weight
    if type(weight) not in (int, float) or not math.isfinite(weight) or weight < 0:
        raise ValueError(f"model.cp_head.aux_weight {weight!r}: the auxiliary loss's weight, a finite number >= 0")
    if head.train_mode != "aux" and weight != 0:
        raise ValueError(f"model.cp_head.aux_weight {weight!r} without model.cp_head.train_mode 'aux': the key would be ignored")
    if head.train_mode == "addon":
        plain = type(head)()
        wrong = [k for k in ("force_lambda_zero", "temperature", "sink_count") if getattr(head, k) != getattr(plain, k)]
        if head.pointer_input != "mix" or wrong:
            raise ValueError("model.cp_head.train_mode 'addon' is built for the pointer on depth reads (pointer_input 'mix') without force_lambda_zero, temperature "
                             f"or sink_count (set: pointer_input {head.pointer_input!r}{', ' + ', '.join(wrong) if wrong else ''})")
    if head.train_mode == "aux":
        plain = type(head)()
        if weight <= 0:
            raise ValueError("model.cp_head.aux_weight 0 with model.cp_head.train_mode 'aux': the pointer's only loss is the auxiliary one; give the weight, > 0")
        wrong = [k for k in ("force_lambda_zero", "score", "temperature", "sink_count") if getattr(head, k) != getattr(plain, k)]
        if cfg.encoder.gdn_write_mix != "none":
            raise ValueError(f"model.cp_head.train_mode 'aux' is not built together with model.encoder.gdn_write_mix {cfg.encoder.gdn_write_mix!r} (nothing tests the pair)")
        if head.pointer_input != "mix" or wrong:
            raise ValueError("model.cp_head.train_mode 'aux' is built for the pointer on depth reads (pointer_input 'mix') without force_lambda_zero, score, "
                             f"temperature or sink_count (set: pointer_input {head.pointer_input!r}{', ' + ', '.join(wrong) if wrong else ''})")
    if head.pointer_input not in POINTER_INPUTS:
        raise ValueError(f"model.cp_head.pointer_input {head.pointer_input!r}: built are {POINTER_INPUTS} (the final norm's output, depth reads of the finished "
                         "blocks, or one head of a global attention layer)")
    if head.pointer_input == "shared":
        shared_layer_index(cfg)
        plain = type(head)()
        clash = {"d_c (the width is the shared head's)": head.d_c != plain.d_c, "qk_norm false": not head.qk_norm, "window": bool(head.window),
                 "temperature (the shared head's form is shared_ssmax)": head.temperature != "none", "n_heads": head.n_heads != 1,
                 "train_mode": head.train_mode != "mixture", "model.encoder.gdn_write_mix": cfg.encoder.gdn_write_mix != "none"}
        hit = [k for k, v in clash.items() if v]
        if hit:
            raise ValueError(f"model.cp_head.pointer_input 'shared' is not built together with: {', '.join(hit)}")
    elif (head.shared_layer, head.shared_head, head.shared_ssmax) != (-1, 0, False):
        raise ValueError("model.cp_head.shared_layer / shared_head / shared_ssmax are read with pointer_input 'shared'")
    if type(head.window) is not int or head.window < 0:
        raise ValueError(f"model.cp_head.window {head.window!r}: the pointer's reach in positions, an integer >= 1 (0: every earlier position)")
    if head.window and (head.temperature != "none" or head.sink_count or head.pointer_input != "final"):
        raise ValueError(f"model.cp_head.window {head.window} is built on the base pointer without the length rule: temperature 'none', sink_count false, "
                         "pointer_input 'final' (the rule counts every earlier position, which a band does not see)")
    if head.pointer_input == "mix" and (cfg.encoder.attn_res != "block_entry" or cfg.encoder.attn_res_query == "token" or cfg.encoder.attn_res_heads != 1):
        raise ValueError("model.cp_head.pointer_input 'mix' reads the finished blocks of model.encoder.attn_res 'block_entry' through static one-softmax readers")
    for name in ("d_c", "query_chunk"):
        if type(getattr(head, name)) is not int or getattr(head, name) < 1:
            raise ValueError(f"model.cp_head.{name} {getattr(head, name)!r}: an integer >= 1")
    for name, allowed in CHOICES.items():
        if getattr(head, name) not in allowed:
            raise ValueError(f"model.cp_head.{name} {getattr(head, name)!r}: one of {allowed}")
    enc, clashes = cfg.encoder, []
    if cfg.loop.recur_layers or cfg.loop.pass2_gate != "none":
        clashes.append("a looped middle or a second pass (one pass only)")
    if enc.attn_res not in ("none", "block_entry"):
        clashes.append(f"encoder.attn_res {enc.attn_res!r}")
    if enc.gdn_write_variant != "none" or enc.gdn_ccr_spacing:
        clashes.append("encoder.gdn_write_variant / gdn_ccr_spacing (nothing tests the pair)")
    if (cfg.fp8.mode, cfg.nvfp4.mode) != ("none", "none"):
        clashes.append("model.fp8 / model.nvfp4")
    if cfg.mtp.enabled:
        clashes.append("model.mtp")
    if clashes:
        raise ValueError(f"model.cp_head is not built with: {'; '.join(clashes)}")


def shared_layer_index(cfg) -> int:
    """The stack index of the global layer whose head the pointer shares (`shared_layer`; -1: the last global layer): a layer
    without a rotary part (its score is its own q . k), with QK-norm and the softmax normaliser, `shared_head` one of its heads."""
    head, enc = cfg.cp_head, cfg.encoder
    layers = enc.global_layers()
    if not layers:
        raise ValueError("model.cp_head.pointer_input 'shared' needs a global attention layer in the stack: there is none")
    at = layers[-1] if head.shared_layer == -1 else head.shared_layer
    if at not in layers:
        raise ValueError(f"model.cp_head.shared_layer {at}: not a global attention layer of the stack (they are {layers})")
    attn = enc.global_attention()[layers.index(at)]
    if attn.rope_fraction != 0.0 or not attn.qk_norm or attn.normalizer != "softmax" or attn.kv_sharing != "gqa":
        raise ValueError(f"model.cp_head.shared_layer {at}: the pointer shares a head of a global layer without a rotary part (model.encoder.nope_global_layers) "
                         "that has QK-norm, the softmax normaliser and grouped keys")
    if not 0 <= head.shared_head < attn.n_q_heads:
        raise ValueError(f"model.cp_head.shared_head {head.shared_head}: layer {at} has {attn.n_q_heads} query heads")
    return at


def _wide(x: torch.Tensor) -> torch.dtype:
    """float32 for the 16-bit types, the tensor's own type above."""
    return torch.promote_types(x.dtype, torch.float32)


def _no_autocast(x: torch.Tensor):
    return torch.autocast(x.device.type, enabled=False)


class PointerMix(nn.Module):
    """The two depth reads of `pointer_input: mix`: x^q = norm_q(read_q(sources)), x^k = norm_k(read_k(sources)); a reader is
    the stack's static block-entry reader (zeros: the sources' mean)."""

    def __init__(self, d_model: int, eps: float):
        super().__init__()
        from .depth_mix import DepthQuery
        from .norms import RMSNorm

        self.read_q, self.read_k = DepthQuery(d_model, eps), DepthQuery(d_model, eps)
        self.norm_q, self.norm_k = RMSNorm(d_model, eps), RMSNorm(d_model, eps)

    def forward(self, sources: list) -> "PointerInputs":
        return PointerInputs(self.norm_q(self.read_q(sources)), self.norm_k(self.read_k(sources)))


class HeadsMix(nn.Module):
    """One pair of depth reads a pointer head: (x^q, x^k), each (B, L, H, d), head h's on axis -2."""

    def __init__(self, d_model: int, eps: float, heads: int):
        super().__init__()
        self.heads = nn.ModuleList(PointerMix(d_model, eps) for _ in range(heads))

    def forward(self, sources: list) -> "PointerInputs":
        reads = [m(sources) for m in self.heads]
        return PointerInputs(torch.stack([r.q for r in reads], dim=-2), torch.stack([r.k for r in reads], dim=-2))


class PointerInputs(NamedTuple):
    """What the pointer's query and key projections read in one forward, each (B, L, d); the forward hands them on as
    `ModelOutput.cp_pointer` and every scoring function takes them as `pointer=`."""

    q: torch.Tensor
    k: torch.Tensor


def pointer_sides(head, hidden, pointer):
    """(the query side's input, the key side's input): h twice for the base pointer, the forward's reads under `mix`."""
    if head.cfg.pointer_input == "final":
        if pointer is not None:
            raise ValueError("pointer inputs were given to a Copy-Paste head whose pointer reads h (model.cp_head.pointer_input 'final')")
        return hidden, hidden
    if pointer is None:
        raise ValueError(f"this Copy-Paste head's pointer reads inputs of its own (model.cp_head.pointer_input {head.cfg.pointer_input!r}): pass the forward's "
                         "ModelOutput.cp_pointer as pointer=")
    return pointer.q, pointer.k


class CopyPasteHead(nn.Module):
    def __init__(self, d_model: int, cfg, ref_len: int = 8192, eps: float = 1e-6, shared_width: int | None = None):
        """shared_width: the shared head's head_dim under `pointer_input: shared` (the pointer's width and the sink key's)."""
        super().__init__()
        self.shared, self.shared_layer = shared_width is not None, None
        self.width = shared_width if self.shared else cfg.d_c
        self.cfg, self.ref_len, self.scale = cfg, int(ref_len), self.width ** -0.5
        self.gated = cfg.train_mode != "aux"            # the <copy> row exists only where something is mixed into the prediction
        H = self.heads = cfg.n_heads
        for name, shape in (("w_q", (H * cfg.d_c, d_model)), ("w_k", (H * cfg.d_c, d_model)), ("k_sink", (H * self.width,)), ("w_copy", (d_model,))):
            if (name != "w_copy" or self.gated) and not (self.shared and name in ("w_q", "w_k")):
                self.register_parameter(name, nn.Parameter(torch.empty(shape)))
        self.d_model = d_model
        if cfg.qk_norm:
            self.qk_gain = nn.Parameter(torch.zeros(H))
        if cfg.combine == "or":
            self.head_router = nn.Parameter(torch.zeros(H, d_model))
        if cfg.pointer_input == "mix":
            self.mix = PointerMix(d_model, eps) if H == 1 else HeadsMix(d_model, eps, H)

    @torch.no_grad()
    def reset_own(self, g: torch.Generator, std: float, init: str = "spec") -> None:
        """w_q, w_k, k_sink, w_copy ~ N(0, std) in that order; `reference` then redraws w_q / w_k as one uniform bank and
        the sink as N(0, 1 / d_c), w_copy keeping its draw."""
        draw = lambda shape: torch.randn(shape, generator=g, dtype=torch.float32)                  # noqa: E731
        d_c, d = self.cfg.d_c, self.d_model
        limit = 3 ** 0.5 * d ** -0.5                           # this product, not sqrt(3 / d): equal bits with the reference's bank

        def start(rows: slice) -> None:
            """The tensors' rows of some heads: N(0, std) each, and under `reference` one uniform bank for W_Q / W_K and the sink N(0, 1 / d_c)."""
            if self.shared:         # the base pointer's tensors drawn into stand-ins and dropped: the <copy> row is the base head's
                parts = [torch.empty(d_c, d), torch.empty(d_c, d), torch.empty(d_c)]
            else:
                parts = [getattr(self, name)[rows] for name in ("w_q", "w_k", "k_sink")]
            for t in parts:
                t.copy_(draw(t.shape) * std)
            if rows.start == 0:                                 # the <copy> row follows head 0's draws (taken and dropped without the row)
                row = draw((d,)) * std
                if self.gated:
                    self.w_copy.copy_(row)
            if init == "reference":
                n = parts[0].shape[0]
                both = torch.empty(2, n, d, dtype=torch.float32).uniform_(-limit, limit, generator=g)
                parts[0].copy_(both[0])
                parts[1].copy_(both[1])
                parts[2].copy_(draw(n) * d_c ** -0.5)

        start(slice(0, d_c))
        if self.heads > 1:
            start(slice(d_c, self.heads * d_c))
        if self.shared:             # the sink in the shared head's key space, after the base head's draws
            self.k_sink.copy_(draw(self.width) * (self.width ** -0.5 if init == "reference" else std))
        if self.cfg.qk_norm:
            self.qk_gain.zero_()
        if self.cfg.combine == "or":
            self.head_router.zero_()

    def _project(self, h, w, normed: bool):
        wide = _wide(h)
        with _no_autocast(h):
            y = F.linear(h.to(wide), w.to(wide))
            return F.rms_norm(y, y.shape[-1:], eps=NORM_EPS) if normed else y

    def _project_heads(self, x, w):
        """x (..., H, d), head h's own input, through head h's rows of w: (..., H, d_c), each head normed over its own d_c."""
        wide = _wide(x)
        with _no_autocast(x):
            y = torch.einsum("...hd,hcd->...hc", x.to(wide), w.to(wide).unflatten(0, (self.heads, self.cfg.d_c)))
            return F.rms_norm(y, y.shape[-1:], eps=NORM_EPS)

    def queries(self, h):
        if self.shared:             # h is the shared head's own QK-normed query
            wide = _wide(h)
            with _no_autocast(h):
                return h.to(wide) * (1.0 + self.qk_gain.to(wide))
        if self.heads > 1:
            q = self._project_heads(h, self.w_q)
            return (q * (1.0 + self.qk_gain.to(q.dtype)).unsqueeze(-1)).flatten(-2)
        q = self._project(h, self.w_q, self.cfg.qk_norm)
        return q * (1.0 + self.qk_gain.to(q.dtype)) if self.cfg.qk_norm else q

    def keys(self, h):
        if self.shared:
            return h.to(_wide(h))
        if self.heads > 1:
            return self._project_heads(h, self.w_k).flatten(-2)
        return self._project(h, self.w_k, self.cfg.qk_norm)

    def route(self, h):
        """log pi (..., H) of `combine: or` from the final norm's output; zeros at one head, without reading h or the router."""
        wide = _wide(h)
        if self.heads == 1:
            return h.new_zeros(*h.shape[:-1], 1, dtype=wide)
        with _no_autocast(h):
            return F.linear(h.to(wide), self.head_router.to(wide)).log_softmax(-1)

    def copy_logit(self, h):
        if not self.gated:
            raise ValueError("this Copy-Paste head trains on its auxiliary loss (model.cp_head.train_mode 'aux'): it has no <copy> row and nothing is mixed "
                             "into the prediction")
        return self._project(h, self.w_copy.unsqueeze(0), False)[..., 0]

    def rule(self) -> "LengthRule":
        return LengthRule(self.cfg.temperature == "ssmax", bool(self.cfg.sink_count), self.ref_len, self.scale, self.cfg.window)


def attach(model) -> None:
    """Registers the head on the model, drawn from a generator of its own."""
    mc = model.cfg
    seed = (torch.initial_seed() + OWN_SEED_OFFSET) % (1 << 63)
    width = None
    if mc.cp_head.pointer_input == "shared":
        at = shared_layer_index(mc)
        mixer = model.encoder.layers[at].mixer
        mixer.cp_query, width = (mc.cp_head.shared_head, bool(mc.cp_head.shared_ssmax)), mixer.cfg.head_dim
    model.cp_head = CopyPasteHead(mc.d_model, mc.cp_head, mc.encoder.attention.temperature_ref_len, mc.norm_eps, width)
    if width is not None:
        model.cp_head.shared_layer = at
    if mc.cp_head.pointer_input == "mix":
        model.encoder.keep_sources = True        # the stack leaves [b_0 .. b_N] in the forward's memo
    model.cp_head.reset_own(torch.Generator().manual_seed(seed), mc.init_std, mc.cp_head.init)


def score_mode(model) -> str:
    return os.environ.get(ENV_SCORE) or model.cfg.cp_head.score


def _lm_only(model) -> bool:
    head = getattr(model, "cp_head", None)
    return head is None or not head.gated or head.cfg.force_lambda_zero or score_mode(model) == "lm"


def aux_terms(ptr: "Pointer"):
    """(L_aux, at the sink) per position from the pointer's terms: -(log p_CP(y) + log(1 - s)) where the next token is in the
    context, else -log s; the branch not taken gets a zero gradient."""
    found = torch.isfinite(ptr.log_copy)
    return torch.where(found, -(ptr.log_copy.masked_fill(~found, 0.0) + ptr.log_ctx), -ptr.log_sink), ~found


# ------------------------------------------------------------------------------------------------------- the pointer

@dataclass
class CopyKeys:
    """The positions a query may copy from: k (B, S, d_c) and their token, document and absolute index (B, S)."""

    k: torch.Tensor
    tok: torch.Tensor
    doc: torch.Tensor
    idx: torch.Tensor

    def upto(self, S: int) -> "CopyKeys":
        return CopyKeys(*(getattr(self, f.name)[:, :S] for f in fields(self)))

    def extend(self, more: "CopyKeys") -> "CopyKeys":
        return CopyKeys(*(torch.cat([getattr(self, f.name), getattr(more, f.name)], dim=1) for f in fields(self)))


@dataclass
class CopyCache:
    keys: CopyKeys | None = None


class Pointer(NamedTuple):
    """log s (the sink's share), log(1 - s), log p_CP(target); each (B, n)."""

    log_sink: torch.Tensor
    log_ctx: torch.Tensor
    log_copy: torch.Tensor


class LengthRule(NamedTuple):
    ssmax: bool
    sink_count: bool
    ref_len: int
    scale: float
    window: int = 0


class Scores(NamedTuple):
    e: torch.Tensor            # (B, C, S) scaled scores, -inf outside a query's context
    sink: torch.Tensor         # (B, C)
    norm_ctx: torch.Tensor     # LSE over the context
    norm_all: torch.Tensor     # LSE over the context and the sink

    def pointer(self, log_copy) -> Pointer:
        return Pointer(self.sink - self.norm_all, self.norm_ctx - self.norm_all, log_copy)


def context_mask(k_idx, k_doc, q_idx, q_doc, window: int = 0):
    """(B, C, S): key s is a context position of query i (not later, same document; with a band, fewer than `window` back)."""
    back = q_idx.unsqueeze(2) - k_idx.unsqueeze(1)
    seen = (k_doc.unsqueeze(1) == q_doc.unsqueeze(2)).logical_and_(back >= 0)
    return seen.logical_and_(back < window) if window else seen


def attend(rule: LengthRule, q, k, k_sink, visible) -> Scores:
    """The pointer's scores of C queries over S keys. The length rule needs each query's context count, which is the
    visible mask's row sum: q is scaled (ssmax) and the sink's logit raised (sink_count) before anything is normalised."""
    sink_shift = None
    if rule.ssmax or rule.sink_count:
        log_ratio = torch.log(visible.sum(-1).clamp_min(1).to(q.dtype) / rule.ref_len)
        if rule.ssmax:
            q = q * (1.0 + log_ratio / math.log(rule.ref_len)).unsqueeze(-1)
        sink_shift = log_ratio if rule.sink_count else None
    e = (q @ k.mT * rule.scale).masked_fill(~visible, float("-inf"))
    sink = (q @ k_sink) * rule.scale
    if sink_shift is not None:
        sink = sink + sink_shift
    norm_ctx = e.logsumexp(-1)
    return Scores(e, sink, norm_ctx, torch.logaddexp(sink, norm_ctx))


def _head_terms(rule, q, k, k_sink, seen, same_token):
    """One head's (scores, log p_CP(target) where a key matches, the rows without a match). A row without a matching key is
    read as zeros: its LSE is finite and its gradient exactly zero; the caller writes -inf there."""
    sc = attend(rule, q, k, k_sink, seen)
    hit = same_token & seen
    none = ~hit.any(-1)
    picked = sc.e.masked_fill(~hit, float("-inf")).masked_fill(none.unsqueeze(-1), 0.0)
    return sc, picked.logsumexp(-1) - sc.norm_ctx, none


def _train_block(rule, q, k, k_sink, k_tok, k_doc, k_idx, q_idx, q_doc, q_tgt, log_pi=None):
    """One block of queries: the three terms as a plain tuple (what a recomputed block returns). log_pi (B, C, H): the
    router's log weights of `combine: or`, the heads then scored one by one on their slices and mixed."""
    seen = context_mask(k_idx, k_doc, q_idx, q_doc, rule.window)
    same_token = k_tok.unsqueeze(1) == q_tgt.unsqueeze(2)
    if log_pi is None:
        sc, log_copy, none = _head_terms(rule, q, k, k_sink, seen, same_token)
        return tuple(sc.pointer(log_copy.masked_fill(none, float("-inf"))))
    H = log_pi.shape[-1]
    per = [_head_terms(rule, qh, kh, sh, seen, same_token) for qh, kh, sh in zip(q.chunk(H, -1), k.chunk(H, -1), k_sink.chunk(H, -1))]
    sink = torch.stack([sc.sink - sc.norm_all for sc, _, _ in per], -1) + log_pi              # log pi_h + log s_h
    ctx = torch.stack([sc.norm_ctx - sc.norm_all for sc, _, _ in per], -1) + log_pi             # log pi_h + log(1 - s_h)
    log_copy = (ctx.log_softmax(-1) + torch.stack([c for _, c, _ in per], -1)).logsumexp(-1)
    return sink.logsumexp(-1), ctx.logsumexp(-1), log_copy.masked_fill(per[0][2], float("-inf"))


def terms(head, hidden, tokens, targets, doc_ids, chunk: int | None = None, checkpoint: bool = False, keys: CopyKeys | None = None,
          q_idx: torch.Tensor | None = None, pointer: PointerInputs | None = None) -> Pointer:
    """The pointer's terms at every position of a forward. keys: the key side (default this forward's own positions at
    indices 0 .. L - 1: a block of queries then reads the keys up to its own end only)."""
    B, L = tokens.shape
    step = chunk or head.cfg.query_chunk
    q_side, k_side = pointer_sides(head, hidden, pointer)
    q = head.queries(q_side)
    causal_cut = keys is None
    if causal_cut:
        at = torch.arange(L, device=tokens.device).expand(B, L)
        keys, q_idx = CopyKeys(head.keys(k_side), tokens, doc_ids, at), at
    sink_key = head.k_sink.to(q.dtype)
    log_pi = head.route(hidden).to(q.dtype) if head.cfg.combine == "or" else None
    block = partial(_train_block, head.rule())
    if checkpoint and torch.is_grad_enabled():
        block = partial(recompute, block, use_reentrant=False)
    blocks = []
    for lo in range(0, L, step):
        hi = min(lo + step, L)
        ks = keys.upto(hi) if causal_cut else keys
        blocks.append(block(q[:, lo:hi], ks.k, sink_key, ks.tok, ks.doc, ks.idx, q_idx[:, lo:hi], doc_ids[:, lo:hi], targets[:, lo:hi],
                            None if log_pi is None else log_pi[:, lo:hi]))
    return Pointer(*(torch.cat(column, dim=1) for column in zip(*blocks)))


def terms_naive(head, hidden, tokens, targets, doc_ids, pointer: PointerInputs | None = None) -> Pointer:
    """The same three terms with every score of a row at once and the softmaxes taken explicitly (tests; small rows)."""
    B, L = tokens.shape
    at = torch.arange(L, device=tokens.device).expand(B, L)
    q_side, k_side = pointer_sides(head, hidden, pointer)
    if head.cfg.combine == "or":
        raise ValueError("terms_naive states the single softmax of combine 'and'")
    sc = attend(head.rule(), head.queries(q_side), head.keys(k_side), head.k_sink.to(_wide(hidden)), context_mask(at, doc_ids, at, doc_ids, head.cfg.window))
    with_sink = torch.cat([sc.sink.unsqueeze(-1), sc.e], dim=-1).softmax(-1)
    share = with_sink[..., 0]
    p_copy = (sc.e.softmax(-1) * (tokens.unsqueeze(1) == targets.unsqueeze(2))).sum(-1)
    return Pointer(share.log(), torch.log1p(-share), p_copy.log())


# ------------------------------------------------------------------------------------------------------- the mixture

@dataclass
class Mixture:
    """lambda = c (1 - s) in logs, with c the share of <copy> in softmax over V u {<copy>}."""

    log_lam: torch.Tensor
    log_keep: torch.Tensor          # log(1 - lambda) = log((1 - c) + c s)
    log_c: torch.Tensor
    lse_v: torch.Tensor

    @classmethod
    def of(cls, lse_v, z_copy, ptr: Pointer) -> "Mixture":
        total = torch.logaddexp(lse_v, z_copy)
        log_c = z_copy - total
        return cls(log_c + ptr.log_ctx, torch.logaddexp(lse_v - total, log_c + ptr.log_sink), log_c, lse_v)

    def at_target(self, z_y, log_copy):
        """log p(y) from the target's logit and log p_CP(y)."""
        return torch.logaddexp(self.log_keep + (z_y - self.lse_v), self.log_lam + log_copy)

    def at_target_given(self, log_lm_y, log_copy):
        """log p(y) with log p_LM(y) given as a number of its own (no LSE_V - LSE_V cancellation)."""
        return torch.logaddexp(self.log_keep + log_lm_y, self.log_lam + log_copy)

    def over_vocab(self, logits, log_copy):
        """log p over V from the logits and log p_CP over V, both (..., V)."""
        return torch.logaddexp((self.log_keep - self.lse_v).unsqueeze(-1) + logits, self.log_lam.unsqueeze(-1) + log_copy)


def logprobs_rows(head, hidden_q, q_idx, q_doc, keys: CopyKeys, weight_v, chunk: int | None = None, q_side=None):
    """log p over V (B, P, V) at the queries, block by block ((B, C, S) alpha and (B, C, V) p_CP at a time). q_side: what the
    query projection reads when that is not the hidden states (`pointer_input: mix`)."""
    wide = _wide(hidden_q)
    step = chunk or head.cfg.query_chunk
    rule, rows = head.rule(), []
    with _no_autocast(hidden_q):
        vocab, sink_key, k = weight_v.to(wide), head.k_sink.to(wide), keys.k.to(wide)
        for lo in range(0, hidden_q.shape[1], step):
            span = slice(lo, lo + step)
            h = hidden_q[:, span].to(wide)
            q = head.queries(h if q_side is None else q_side[:, span].to(wide))
            seen = context_mask(keys.idx, keys.doc, q_idx[:, span], q_doc[:, span], rule.window)
            if head.cfg.combine == "or":            # each head's own softmaxes, mixed by the router's weights
                H, log_pi = head.heads, head.route(h)
                per = [attend(rule, qh, kh, sh, seen) for qh, kh, sh in zip(q.chunk(H, -1), k.chunk(H, -1), sink_key.chunk(H, -1))]
                ctx = torch.stack([x.norm_ctx - x.norm_all for x in per], -1) + log_pi
                share = ctx.softmax(-1)
                weights = sum(share[..., i:i + 1] * (x.e - x.norm_ctx.unsqueeze(-1)).exp() for i, x in enumerate(per))
                log_sink = (torch.stack([x.sink - x.norm_all for x in per], -1) + log_pi).logsumexp(-1)
                sc = Scores(None, log_sink, ctx.logsumexp(-1), torch.zeros_like(log_sink))      # already normalised: sink and context in logs
            else:
                sc = attend(rule, q, k, sink_key, seen)
                weights = (sc.e - sc.norm_ctx.unsqueeze(-1)).exp()                                  # alpha: softmax over the context alone
            logits = F.linear(h, vocab)
            p_copy = torch.zeros_like(logits).scatter_add_(2, keys.tok.unsqueeze(1).expand_as(weights), weights)
            log_copy = p_copy.clamp_min(torch.finfo(wide).tiny).log().masked_fill(p_copy <= 0, float("-inf"))
            mix = Mixture.of(logits.logsumexp(-1), head.copy_logit(h), sc.pointer(None))
            rows.append(mix.over_vocab(logits, log_copy))
    return torch.cat(rows, dim=1)


def forward_logits(model, hidden, tokens, doc_ids, idx, cache: CopyCache | None, pointer: PointerInputs | None = None):
    """(the model's `logits` of a forward: log p over V, or p_LM's logits under score 'lm'; the copy cache after the chunk)."""
    wide = _wide(hidden)
    q_side, k_side = pointer_sides(model.cp_head, hidden, pointer)
    with _no_autocast(hidden):
        keys = CopyKeys(model.cp_head.keys(k_side.to(wide)), tokens, doc_ids, idx)
        if cache is not None and cache.keys is not None:
            keys = cache.keys.extend(keys)                              # a chunk appends its own keys before its queries read
        if _lm_only(model):
            out = F.linear(hidden.to(wide), model.lm_head_weight().to(wide))
        else:
            out = logprobs_rows(model.cp_head, hidden, idx, doc_ids, keys, model.lm_head_weight(), q_side=None if pointer is None else q_side)
    return out, CopyCache(keys)


def token_lse_zy(hidden, weight, targets, chunk: int = 1024):
    """(LSE over V, the target's logit) per position, by blocks of positions under activation checkpointing when gradients
    are on: the (block, V) logits exist only while a block's forward or backward runs."""
    wide = _wide(hidden)
    flat_h, flat_t = hidden.flatten(0, -2), targets.flatten()

    def rows(h, t, w):
        with _no_autocast(h):
            z = F.linear(h.to(wide), w.to(wide))
            return z.logsumexp(-1), z.gather(1, t.unsqueeze(1))[:, 0]

    run = partial(recompute, rows, use_reentrant=False) if torch.is_grad_enabled() else rows
    lse, z_y = zip(*(run(flat_h[lo:lo + chunk], flat_t[lo:lo + chunk], weight) for lo in range(0, flat_h.shape[0], chunk)))
    return torch.cat(lse).view_as(targets), torch.cat(z_y).view_as(targets)


def _mixture_at_targets(head, hidden, lse, tokens, targets, doc_ids, checkpoint: bool, pointer=None):
    with _no_autocast(hidden):
        ptr = Pointer(*(t.to(lse.dtype) for t in terms(head, hidden, tokens, targets, doc_ids, checkpoint=checkpoint, pointer=pointer)))
        return Mixture.of(lse, head.copy_logit(hidden).to(lse.dtype), ptr), ptr


def head_token_ce(model, hidden, targets, tokens, doc_ids, chunk: int = 1024, pointer: PointerInputs | None = None):
    """(CE, LSE over V) per position of the model's next-token distribution from a forward's hidden states: p_LM's for a model
    without the head or under score 'lm', else the mixture's."""
    lse, z_y = token_lse_zy(hidden, model.lm_head_weight(), targets, chunk)
    if _lm_only(model):
        return lse - z_y, lse
    mix, ptr = _mixture_at_targets(model.cp_head, hidden, lse, tokens, targets, doc_ids, False, pointer)
    return -mix.at_target(z_y, ptr.log_copy), lse


def addon_loss(model, hidden, targets, tokens, doc_ids, weights, chunk: int = 1024, pointer: PointerInputs | None = None):
    """sum(weights x the mixture's CE) with everything of the trunk and the LM head detached, and the detached per-position
    (mixture CE, lambda): the gradient reaches the head's own tensors alone."""
    head = model.cp_head
    still = hidden.detach()
    with torch.no_grad():
        lse, z_y = token_lse_zy(still, model.lm_head_weight().detach(), targets, chunk)
    with _no_autocast(hidden):
        ptr = Pointer(*(t.to(lse.dtype) for t in terms(head, still, tokens, targets, doc_ids, checkpoint=True, pointer=pointer)))
        mix = Mixture.of(lse, head.copy_logit(still).to(lse.dtype), ptr)
        ce = -mix.at_target_given(z_y - lse, ptr.log_copy)
    return (ce * weights.to(ce.dtype)).sum(), ce.detach(), mix.log_lam.detach().exp()


def mixture_loss(model, hidden, targets, tokens, doc_ids, a, b, chunk: int = 1024, pointer: PointerInputs | None = None):
    """The training loss sum(a CE + b LSE_V^2) of the mixture and the detached per-position (CE, lambda). a, b: per-position
    weights (0 where a target does not count)."""
    lse, z_y = token_lse_zy(hidden, model.lm_head_weight(), targets, chunk)
    if model.cp_head.cfg.force_lambda_zero:
        ce, lam = lse - z_y, torch.zeros_like(lse)
    else:
        mix, ptr = _mixture_at_targets(model.cp_head, hidden, lse, tokens, targets, doc_ids, True, pointer)
        ce, lam = -mix.at_target(z_y, ptr.log_copy), mix.log_lam.detach().exp()
    total = (ce * a.to(ce.dtype)).sum() + (lse.square() * b.to(ce.dtype)).sum()
    return total, ce.detach(), lam
