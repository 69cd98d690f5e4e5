"""The Copy-Paste head (`model.cp_head.enabled`): a pointer over the context mixed into the next-token distribution.

    h_t   the final norm's output (the LM head's input);  q_t = W_Q h_t, k_tau = W_K h_tau (d_c wide), a sink key k_sink
    e_tau = q_t . k_tau / sqrt(d_c) over tau <= t of t's document,  e_sink = q_t . k_sink / sqrt(d_c)
    s_t   = softmax over {sink} u ctx at the sink;   alpha_t = softmax over ctx alone
    p_CP(v) = sum of alpha_t(tau) over tau with x_tau = v
    c_t   = softmax over V u {<copy>} at <copy>, the <copy> logit z_copy = w_copy . h_t (a vector of its own, never a token)
    lambda_t = c_t (1 - s_t);    p(v) = (1 - lambda_t) p_LM(v) + lambda_t p_CP(v);   loss: cross entropy on p

Everything is formed in log space and nothing of size T x T x V exists: the training terms (`terms`) are
(log s, log(1 - s), log p_CP(target)) by blocks of queries against the keys up to the block's end, masks by comparisons
and `where` (fixed shapes); a query without a matching key gives log p_CP = -inf with a gradient of exactly zero. The
mixture at the target is `mixture_log_prob`. At inference `forward_logits` returns log p over V (p_CP over V by a
scatter-add of alpha, per block of queries), so every reader of logits reads the mixture; `score: lm` returns p_LM's
logits instead. Cached generation keeps, per earlier position, its key, token, document and index (`CopyCache`); a chunk
appends its own before its queries read (tau = t included).

Options built: `qk_norm` (q and k RMS-normed over d_c at eps 2^-23, q times 1 + `qk_gain`), `init: spec` (every tensor
N(0, init_std)) / `reference` (W_Q, W_K U(+-sqrt(3 / d)), the sink N(0, 1 / d_c)), the length rule (`temperature: ssmax`:
q times ln(n_t) / ln(ref); `sink_count`: e_sink + ln(n_t / ref); n_t the context positions a query sees, ref the global
layers' temperature_ref_len), `force_lambda_zero`, `query_chunk`. The tensors are registered after every other tensor and
drawn from a generator of their own, so the base model starts as the model without the key. Refused by name: pointers that
read the depth sources or an attention head (`pointer_input` mix / shared), several pointer heads, the copy from the trunk's
own attention (`trunk_copy`), the auxiliary and add-on training modes, a band (`window`), the fused kernel.
Reference: ced/model/cp_head.py:1-100 (the form), :454-660 (the module), :899-1016 (length rule, block terms),
:1223-1245 (mixture), :1282-1370 (inference), :1443-1483 (cache).
"""

from __future__ import annotations

import math
import os
from dataclasses import dataclass

import torch
import torch.nn as nn
import torch.utils.checkpoint as ckpt

OWN_SEED_OFFSET = 0xC0_2610_19247        # shared with the reference: equal starts under equal seeds
QK_NORM_EPS = float(torch.finfo(torch.float32).eps)
INITS, SCORES, TEMPERATURES = ("spec", "reference"), ("mixture", "lm"), ("none", "ssmax")
ENV_SCORE = "GHB_CP_SCORE"               # a scoring process's override of model.cp_head.score
PARAMETERS = ("cp_head.w_q", "cp_head.w_k", "cp_head.k_sink", "cp_head.w_copy", "cp_head.qk_gain")


def check_config(cfg) -> None:
    c = cfg.cp_head
    if not c.enabled:
        return
    fixed = {"pointer_input": "final", "n_heads": 1, "combine": "and", "trunk_copy": "none", "train_mode": "mixture", "window": 0, "kernel": "reference"}
    moved = [f"{k} {getattr(c, k)!r}" for k, v in fixed.items() if getattr(c, k) != v]
    if moved:
        raise ValueError(f"model.cp_head {', '.join(moved)}: the head is built in its base form (pointer_input 'final', one pointer head, "
                         "train_mode 'mixture', no band, no trunk copy, kernel 'reference')")
    if type(c.d_c) is not int or c.d_c < 1 or type(c.query_chunk) is not int or c.query_chunk < 1:
        raise ValueError(f"model.cp_head.d_c {c.d_c!r} / query_chunk {c.query_chunk!r}: integers >= 1")
    if c.init not in INITS or c.score not in SCORES or c.temperature not in TEMPERATURES:
        raise ValueError(f"model.cp_head.init {c.init!r} / score {c.score!r} / temperature {c.temperature!r}: of {INITS} / {SCORES} / {TEMPERATURES}")
    e = cfg.encoder
    refused = [(bool(cfg.loop.recur_layers) or cfg.loop.pass2_gate != "none", "a looped middle or a second pass (one pass only)"),
               (e.attn_res not in ("none", "block_entry"), f"encoder.attn_res {e.attn_res!r}"),
               (e.gdn_write_variant != "none" or bool(e.gdn_ccr_spacing), "encoder.gdn_write_variant / gdn_ccr_spacing (nothing tests the pair)"),
               (cfg.fp8.mode != "none" or cfg.nvfp4.mode != "none", "model.fp8 / model.nvfp4"), (bool(cfg.mtp.enabled), "model.mtp")]
    bad = [why for cond, why in refused if cond]
    if bad:
        raise ValueError(f"model.cp_head is not built with: {'; '.join(bad)}")


def work_dtype(x: torch.Tensor) -> torch.dtype:
    return torch.promote_types(x.dtype, torch.float32)


class CopyPasteHead(nn.Module):
    def __init__(self, d_model: int, cfg, ref_len: int = 8192):
        super().__init__()
        self.cfg, self.ref_len = cfg, int(ref_len)
        self.w_q = nn.Parameter(torch.empty(cfg.d_c, d_model))
        self.w_k = nn.Parameter(torch.empty(cfg.d_c, d_model))
        self.k_sink = nn.Parameter(torch.empty(cfg.d_c))
        self.w_copy = nn.Parameter(torch.empty(d_model))
        if cfg.qk_norm:
            self.qk_gain = nn.Parameter(torch.zeros(1))
        self.scale = 1.0 / math.sqrt(cfg.d_c)

    @torch.no_grad()
    def reset_own(self, g: torch.Generator, std: float, init: str = "spec") -> None:
        """w_q, w_k, k_sink, w_copy ~ N(0, std) in that order; `reference` then redraws w_q / w_k as one uniform bank and
        the sink as N(0, 1 / d_c), w_copy keeping its draw."""
        for p in (self.w_q, self.w_k, self.k_sink, self.w_copy):
            p.copy_(torch.randn(p.shape, generator=g, dtype=torch.float32).to(p.dtype) * std)
        if init == "reference":
            d_c, d = self.w_q.shape
            bound = (3 ** 0.5) * d ** -0.5
            bank = torch.empty(2, d_c, d, dtype=torch.float32).uniform_(-bound, bound, generator=g)
            self.w_q.copy_(bank[0].to(self.w_q.dtype))
            self.w_k.copy_(bank[1].to(self.w_k.dtype))
            self.k_sink.copy_((torch.randn(d_c, generator=g, dtype=torch.float32) * d_c ** -0.5).to(self.k_sink.dtype))
        if self.cfg.qk_norm:
            self.qk_gain.zero_()

    def _proj(self, h, w):
        dt = work_dtype(h)
        with torch.autocast(h.device.type, enabled=False):
            return torch.nn.functional.linear(h.to(dt), w.to(dt))

    @staticmethod
    def _norm(x):
        with torch.autocast(x.device.type, enabled=False):
            return torch.nn.functional.rms_norm(x, (x.shape[-1],), eps=QK_NORM_EPS)

    def queries(self, h):
        q = self._proj(h, self.w_q)
        return self._norm(q) * (1.0 + self.qk_gain.to(q.dtype)) if self.cfg.qk_norm else q

    def keys(self, h):
        k = self._proj(h, self.w_k)
        return self._norm(k) if self.cfg.qk_norm else k

    def copy_logit(self, h):
        return self._proj(h, self.w_copy[None, :]).squeeze(-1)


def attach(model) -> None:
    cfg = model.cfg
    head = CopyPasteHead(cfg.d_model, cfg.cp_head, cfg.encoder.attention.temperature_ref_len)
    head.reset_own(torch.Generator().manual_seed((torch.initial_seed() + OWN_SEED_OFFSET) % (1 << 63)), cfg.init_std, cfg.cp_head.init)
    model.cp_head = head


def score_mode(model) -> str:
    return os.environ.get(ENV_SCORE) or model.cfg.cp_head.score


# ------------------------------------------------------------------------------------------------------- keys and terms

@dataclass
class CopyKeys:
    """The positions a query may copy from: k (B, S, d_c) and their token, document and absolute index (B, S)."""

    k: torch.Tensor
    tok: torch.Tensor
    doc: torch.Tensor
    idx: torch.Tensor

    def extend(self, other: "CopyKeys") -> "CopyKeys":
        return CopyKeys(*(torch.cat([getattr(self, n), getattr(other, n)], dim=1) for n in ("k", "tok", "doc", "idx")))


@dataclass
class CopyCache:
    keys: CopyKeys | None = None


def _neg_inf(like):
    return torch.full((), float("-inf"), dtype=like.dtype, device=like.device)


def context_mask(k_idx, k_doc, q_idx, q_doc):
    """(B, C, S): key s is a context position of query i (not later, same document)."""
    return (k_idx[:, None, :] <= q_idx[:, :, None]) & (k_doc[:, None, :] == q_doc[:, :, None])


def length_terms(head, q, n):
    """(q for the scores, what is added to the sink's logit or None) under the length rule; n (B, C) context counts."""
    c = head.cfg
    if c.temperature == "none" and not c.sink_count:
        return q, None
    n = n.clamp_min(1).to(q.dtype)
    add = torch.log(n / head.ref_len) if c.sink_count else None
    if c.temperature == "ssmax":
        q = q * (1.0 + torch.log(n / head.ref_len) / math.log(head.ref_len))[..., None]
    return q, add


def block_terms(q, k, k_sink, k_tok, k_doc, k_idx, q_idx, q_doc, q_tgt, scale: float, sink_add=None):
    """(log s, log(1 - s), log p_CP(target)), each (B, C), for C queries over S keys."""
    neg = _neg_inf(q)
    s = torch.matmul(q, k.transpose(1, 2)) * scale
    e_sink = torch.matmul(q, k_sink) * scale
    if sink_add is not None:
        e_sink = e_sink + sink_add
    ctx = context_mask(k_idx, k_doc, q_idx, q_doc)
    match = ctx & (k_tok[:, None, :] == q_tgt[:, :, None])
    lse_ctx = torch.logsumexp(torch.where(ctx, s, neg), dim=-1)
    has = match.any(dim=-1)
    fill = torch.where(has, neg, torch.zeros((), dtype=s.dtype, device=s.device))[..., None]      # a row without a match reads zeros: finite, gradient 0
    lse_match = torch.logsumexp(torch.where(match, s, fill), dim=-1)
    lse_all = torch.logaddexp(e_sink, lse_ctx)
    return e_sink - lse_all, lse_ctx - lse_all, torch.where(has, lse_match - lse_ctx, neg)


def terms(head, hidden, tokens, targets, doc_ids, chunk: int | None = None, checkpoint: bool = False, keys: CopyKeys | None = None,
          q_idx: torch.Tensor | None = None):
    """(log s, log(1 - s), log p_CP(target)), each (B, L), at every position of a forward. keys: the key side (default this
    forward's own positions at indices 0 .. L - 1: a block of queries then reads the keys up to its own end only)."""
    B, L = tokens.shape
    q = head.queries(hidden)
    own = keys is None
    idx = torch.arange(L, device=tokens.device).expand(B, L)
    if own:
        keys = CopyKeys(head.keys(hidden), tokens, doc_ids, idx)
    q_idx = idx if q_idx is None else q_idx
    C = chunk or head.cfg.query_chunk
    sink_add = None
    if head.cfg.temperature != "none" or head.cfg.sink_count:
        if own:
            from .sequence import sequence_context

            n = sequence_context(doc_ids, None)[0].pos + 1
        else:
            n = torch.cat([context_mask(keys.idx, keys.doc, q_idx[:, a:a + C], doc_ids[:, a:a + C]).sum(-1) for a in range(0, L, C)], 1)
        q, sink_add = length_terms(head, q, n)
    k_sink = head.k_sink.to(q.dtype)
    parts = []
    for a in range(0, L, C):
        S = min(a + C, L) if own else keys.k.shape[1]
        args = (q[:, a:a + C], keys.k[:, :S], k_sink, keys.tok[:, :S], keys.doc[:, :S], keys.idx[:, :S], q_idx[:, a:a + C], doc_ids[:, a:a + C],
                targets[:, a:a + C], head.scale, None if sink_add is None else sink_add[:, a:a + C])
        parts.append(ckpt.checkpoint(block_terms, *args, use_reentrant=False) if checkpoint and torch.is_grad_enabled() else block_terms(*args))
    return tuple(torch.cat([p[i] for p in parts], dim=1) for i in range(3))


def terms_naive(head, hidden, tokens, targets, doc_ids):
    """The same three terms with every score of a row at once and the softmaxes taken explicitly (tests; small rows)."""
    B, L = tokens.shape
    q, k = head.queries(hidden), head.keys(hidden)
    idx = torch.arange(L, device=tokens.device).expand(B, L)
    ctx = context_mask(idx, doc_ids, idx, doc_ids)
    add = None
    if head.cfg.temperature != "none" or head.cfg.sink_count:
        q, add = length_terms(head, q, ctx.sum(-1))
    e = torch.einsum("bqd,bkd->bqk", q, k) * head.scale
    e_sink = (q @ head.k_sink.to(q.dtype)) * head.scale + (0 if add is None else add)
    full = torch.cat([e_sink[..., None], e.masked_fill(~ctx, float("-inf"))], dim=-1).softmax(-1)
    s = full[..., 0]
    alpha = e.masked_fill(~ctx, float("-inf")).softmax(-1)
    p_cp = (alpha * (tokens[:, None, :] == targets[:, :, None])).sum(-1)
    return torch.log(s), torch.log1p(-s), torch.log(p_cp)


def mixture_log_prob(lse_v, z_y, z_c, log_s, log_1ms, log_pcp):
    """log p(y) from per-position LSE over V, the target's logit, the <copy> logit and the pointer's three terms."""
    lse_all = torch.logaddexp(lse_v, z_c)
    log_c, log_1mc = z_c - lse_all, lse_v - lse_all
    log_lam = log_c + log_1ms
    log_1mlam = torch.logaddexp(log_1mc, log_c + log_s)              # 1 - lambda = (1 - c) + c s
    return torch.logaddexp(log_1mlam + z_y - lse_v, log_lam + log_pcp)


def mixture_parts(lse_v, z_c, log_s, log_1ms):
    """(log lambda, log(1 - lambda), log c)."""
    lse_all = torch.logaddexp(lse_v, z_c)
    log_c = z_c - lse_all
    return log_c + log_1ms, torch.logaddexp(lse_v - lse_all, log_c + log_s), log_c


# ---------------------------------------------------------------------------------------------------------- inference

def logprobs_rows(head, hidden_q, q_idx, q_doc, keys: CopyKeys, weight_v, chunk: int | None = None):
    """log p over V (B, P, V) at the queries, block by block ([B, C, S] alpha and [B, C, V] p_CP at a time)."""
    B, P, _ = hidden_q.shape
    V = weight_v.shape[0]
    dt = work_dtype(hidden_q)
    C = chunk or head.cfg.query_chunk
    out = []
    with torch.autocast(hidden_q.device.type, enabled=False):
        W, k_sink = weight_v.to(dt), head.k_sink.to(dt)
        for a in range(0, P, C):
            h = hidden_q[:, a:a + C].to(dt)
            qi, qd = q_idx[:, a:a + C], q_doc[:, a:a + C]
            ctx = context_mask(keys.idx, keys.doc, qi, qd)
            q, add = length_terms(head, head.queries(h), ctx.sum(-1))
            e = torch.matmul(q, keys.k.to(dt).transpose(1, 2)) * head.scale
            e_sink = torch.matmul(q, k_sink) * head.scale + (0 if add is None else add)
            masked = torch.where(ctx, e, _neg_inf(e))
            lse_ctx = torch.logsumexp(masked, dim=-1)
            alpha = torch.exp(masked - lse_ctx[..., None])
            lse_all = torch.logaddexp(e_sink, lse_ctx)
            log_s, log_1ms = e_sink - lse_all, lse_ctx - lse_all
            n = h.shape[1]
            p_cp = torch.zeros(B, n, V, dtype=dt, device=h.device).scatter_add_(2, keys.tok[:, None, :].expand(B, n, keys.tok.shape[1]), alpha)
            logits = torch.nn.functional.linear(h, W)
            lse_v = torch.logsumexp(logits, dim=-1)
            log_lam, log_1mlam, _ = mixture_parts(lse_v, head.copy_logit(h), log_s, log_1ms)
            pos = p_cp > 0
            log_pcp = torch.where(pos, torch.log(torch.where(pos, p_cp, torch.ones((), dtype=dt, device=h.device))), _neg_inf(p_cp))
            out.append(torch.logaddexp((log_1mlam - lse_v)[..., None] + logits, log_lam[..., None] + log_pcp))
    return torch.cat(out, dim=1)


def forward_logits(model, hidden, tokens, doc_ids, idx, cache: CopyCache | None):
    """(the model's `logits` of a forward: log p over V, or p_LM's logits under score 'lm'; the copy cache after the chunk)."""
    head = model.cp_head
    W = model.lm_head_weight()
    dt = work_dtype(hidden)
    with torch.autocast(hidden.device.type, enabled=False):
        own = CopyKeys(head.keys(hidden.to(dt)), tokens, doc_ids, idx)
        keys = own if cache is None or cache.keys is None else cache.keys.extend(own)
        if score_mode(model) == "lm" or head.cfg.force_lambda_zero:
            logits = torch.nn.functional.linear(hidden.to(dt), W.to(dt))
        else:
            logits = logprobs_rows(head, hidden, idx, doc_ids, keys, W)
    return logits, CopyCache(keys=keys)


def token_lse_zy(hidden, weight, targets, chunk: int = 1024):
    """(LSE over V, the target's logit) per position, by blocks of positions under activation checkpointing when gradients
    are on: the (block, V) logits exist only while a block's forward or backward runs."""
    dt = work_dtype(hidden)
    h, t = hidden.reshape(-1, hidden.shape[-1]), targets.reshape(-1)

    def block(hb, tb, W):
        with torch.autocast(hb.device.type, enabled=False):
            logits = torch.nn.functional.linear(hb.to(dt), W.to(dt))
            return torch.logsumexp(logits, dim=-1), logits.gather(1, tb[:, None]).squeeze(1)

    parts = [ckpt.checkpoint(block, h[s:s + chunk], t[s:s + chunk], weight, use_reentrant=False) if torch.is_grad_enabled()
             else block(h[s:s + chunk], t[s:s + chunk], weight) for s in range(0, h.shape[0], chunk)]
    return torch.cat([p[0] for p in parts]).reshape(targets.shape), torch.cat([p[1] for p in parts]).reshape(targets.shape)


def head_token_ce(model, hidden, targets, tokens, doc_ids, chunk: int = 1024):
    """(CE, LSE over V) per position of the model's next-token distribution from a forward's hidden states: p_LM's for a model
    without the head or under score 'lm', else the mixture's."""
    head = getattr(model, "cp_head", None)
    W = model.lm_head_weight()
    lse, z_y = token_lse_zy(hidden, W, targets, chunk)
    if head is None or score_mode(model) == "lm" or head.cfg.force_lambda_zero:
        return lse - z_y, lse
    with torch.autocast(hidden.device.type, enabled=False):
        log_s, log_1ms, log_pcp = (x.to(lse.dtype) for x in terms(head, hidden, tokens, targets, doc_ids))
        return -mixture_log_prob(lse, z_y, head.copy_logit(hidden).to(lse.dtype), log_s, log_1ms, log_pcp), lse


def mixture_loss(model, hidden, targets, tokens, doc_ids, a, b, chunk: int = 1024):
    """The training loss sum(a CE + b LSE_V^2) of the mixture and the detached per-position (CE, lambda). a, b: per-position
    weights (0 where a target does not count)."""
    head = model.cp_head
    W = model.lm_head_weight()
    lse, z_y = token_lse_zy(hidden, W, targets, chunk)
    if head.cfg.force_lambda_zero:
        ce, lam = lse - z_y, torch.zeros_like(lse)
    else:
        with torch.autocast(hidden.device.type, enabled=False):
            log_s, log_1ms, log_pcp = (x.to(lse.dtype) for x in terms(head, hidden, tokens, targets, doc_ids, checkpoint=True))
            z_c = head.copy_logit(hidden).to(lse.dtype)
            ce = -mixture_log_prob(lse, z_y, z_c, log_s, log_1ms, log_pcp)
            lam = torch.exp(mixture_parts(lse, z_c, log_s, log_1ms)[0]).detach()
    loss = (a.to(ce.dtype) * ce + b.to(ce.dtype) * lse * lse).sum()
    return loss, ce.detach(), lam
