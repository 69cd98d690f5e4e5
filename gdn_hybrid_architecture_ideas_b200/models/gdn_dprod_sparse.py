"""Gated DeltaProduct with the second step on a subset of the tokens (`gdn.dprod.stride` s, `summary`, `conv: false`,
`first_beta`; n_h 2).

    S_t = R(k2, v2, beta2) R(k1_t, v1_t, beta1_t) (a_t S_{t-1})    for the carrying tokens: row index p with p mod s = s - 1
    S_t =                  R(k1_t, v1_t, beta1_t) (a_t S_{t-1})    otherwise;     o_t = S_t^T q_t

with R(k, v, beta) S = (I - beta k k^T) S + beta k v^T, the decay once before step 1 and the read after the token's last
update. The second step of a carrying token comes from

    summary none     the token's own x:  k2 = unit(SiLU(W_k x)), v2 = SiLU(W_v x), beta2 = M sigmoid(w_b x), with
                     `dprod.in_proj_kv` / `dprod.in_proj_b` run on the carrying rows only and no short conv
    summary xmean    the same matrices on the mean of x over the tokens of the group of s that are in the carrying (last)
                     token's document
    summary kvmean   no matrix: k2 = unit(mean of k1), v2 = mean of v1 over the same tokens, beta2 = M sigmoid(c),
                     c = `dprod.beta_const` (H_v,) zeros

M = `dprod.beta_max`. Step 1's beta is M sigmoid(b) on a carrying token and sigmoid(b) elsewhere (`first_beta: carry`, so a
token that does not carry is the plain layer's token) or M sigmoid(b) everywhere (`first_beta: all`). An update never
crosses a document boundary, and a group summarises only its last token's document.

How it runs here. The loop (`sparse_recurrence`) is the rule as written. The chunked form runs the ordinary chunked delta
rule on a ROW layout: one row per token plus one row after each carrying token, (k1, v1, beta1, g, q = 0) then
(k2, v2, beta2, g = 0, q); the layout is one concatenation [tokens ; extra rows] followed by one gather through an index
that depends on (L, s, phase) only and is built on the host, and the outputs come back through the inverse gather. A cached
forward needs the phase (the absolute index of the call's first token, one host read) and, with a summary, the running
sums of the group still open (`GDNState.acc`, `GDNState.cnt`). `dprod.sparse_path` names copy strategies of the same
function in the reference; every value runs this one layout. Tensor ops on every device
(reference: ced/model/gdn_dprod_sparse.py:1-701, ced/model/gdn_dprod_sparse_fast.py:39).
"""

from __future__ import annotations

import torch
import torch.nn as nn
import torch.nn.functional as F

from .. import ops
from .linear import Linear

SUMMARIES = ("none", "xmean", "kvmean")
FIRST_BETAS = ("carry", "all")
PATHS = (None, "plain", "fast", "rows")
DEFAULTS = {"stride": 1, "summary": "none", "conv": True, "first_beta": "carry"}


def keys_of(cfg) -> tuple:
    d = cfg.dprod
    s, summary, conv, fb = d.stride, d.summary, d.conv, d.first_beta
    if isinstance(s, bool) or not isinstance(s, int) or s < 1:
        raise ValueError(f"gdn.dprod.stride {s!r}: an integer >= 1 (1: the second step on every token)")
    if summary not in SUMMARIES:
        raise ValueError(f"gdn.dprod.summary {summary!r}: one of {SUMMARIES}")
    if not isinstance(conv, bool):
        raise ValueError(f"gdn.dprod.conv {conv!r}: true or false")
    if fb not in FIRST_BETAS:
        raise ValueError(f"gdn.dprod.first_beta {fb!r}: one of {FIRST_BETAS}")
    if d.sparse_path not in PATHS:
        raise ValueError(f"gdn.dprod.sparse_path {d.sparse_path!r}: not set or one of {PATHS[1:]}")
    return s, summary, conv, fb


def is_sparse(cfg) -> bool:
    """The layer runs this module: key proj with a stride other than 1, a summary, or conv false."""
    s, summary, conv, _ = keys_of(cfg)
    return cfg.dprod.key == "proj" and (s != 1 or summary != "none" or conv is False)


def check_keys(cfg) -> None:
    s, summary, conv, fb = keys_of(cfg)
    d, n = cfg.dprod, cfg.dprod.n_h
    used = [k for k, v in zip(DEFAULTS, (s, summary, conv, fb)) if v != DEFAULTS[k]] + (["sparse_path"] if d.sparse_path not in (None, "plain") else [])
    if n == 1:
        if used and d.key == "proj" and (d.value, d.beta, d.rank, d.perm) == ("proj", "proj", 16, "roll"):
            raise ValueError(f"gdn.dprod.{', '.join(used)} set with dprod.n_h 1: these keys place the second step and are read only with n_h 2")
        return
    if d.key != "proj":
        moved = [k for k in used if k != "conv"]
        if moved:
            raise ValueError(f"gdn.dprod.{', '.join(moved)} with dprod.key {d.key!r}: the strided and summarised second step is not built together "
                             "with a second step derived from the first")
        return
    if not is_sparse(cfg):
        if d.sparse_path not in (None, "plain"):
            raise ValueError(f"gdn.dprod.sparse_path {d.sparse_path!r} with the stride, summary and conv at their defaults: the key would change nothing")
        return
    if n != 2:
        raise ValueError(f"gdn.dprod.n_h {n} with stride {s} / summary {summary!r} / conv {conv}: the second step on a subset of the tokens is n_h 2 only")
    if conv and (s > 1 or summary != "none"):
        raise ValueError(f"gdn.dprod.conv true with stride {s} / summary {summary!r}: the strided and summarised second step has no short conv "
                         "(set dprod.conv=false)")
    stray = [k for k, v in (("value", "proj"), ("beta", "proj"), ("rank", 16), ("perm", "roll"), ("route", "interleave"), ("beta_init", None))
             if getattr(d, k) != v]
    if stray:
        raise ValueError(f"gdn.dprod.{', '.join(stray)} with stride {s} / summary {summary!r} / conv {conv}: not built together")


def params_per_layer(d_model: int, cfg) -> int:
    if cfg.dprod.summary == "kvmean":
        return cfg.n_v_heads
    return d_model * (cfg.n_k_heads * cfg.k_head_dim + cfg.n_v_heads * cfg.v_head_dim) + d_model * cfg.n_v_heads


# ------------------------------------------------------------------------------------------------ the layout (host integers)

def first_carry(pos0: int, s: int) -> int:
    return (s - 1 - pos0) % s


def carry_flags(L: int, s: int, pos0: int = 0) -> list:
    return [(pos0 + i) % s == s - 1 for i in range(L)]


def row_maps(L: int, s: int, off: int):
    """For a call of L tokens whose first carrying token is at index `off`: (rows, last) as Python lists. rows[r] is where
    row r of the layout comes from in [tokens ; extra rows] (token i at i, the j-th extra row at L + j); last[i] is the row
    token i's output is read on (its extra row when it carries)."""
    rows, last, j = [], [], 0
    for i in range(L):
        rows.append(i)
        if i >= off and (i - off) % s == 0:
            rows.append(L + j)
            j += 1
        last.append(len(rows) - 1)
    return rows, last, j


def group_sums(u, doc, s: int, off: int, carry_in=None):
    """The sums of the features u (B, L, F) and the token counts over each group closed in the call, restricted to the
    tokens in the document of the group's last token: (sums (B, n_c, F), counts (B, n_c)). carry_in (acc, cnt, ok): the sums
    of the head group's tokens seen in earlier calls, added where ok (the carried tokens are in the closing token's document)."""
    B, L = u.shape[:2]
    closes = list(range(off, L, s))
    sums, counts = [], []
    for n, end in enumerate(closes):
        lo = max(0, end - s + 1)
        m = (doc[:, lo:end + 1] == doc[:, end:end + 1]).to(u.dtype)
        su, sc = (m[..., None] * u[:, lo:end + 1]).sum(1), m.sum(1)
        if carry_in is not None and n == 0 and end - lo + 1 < s:
            acc, cnt, ok = carry_in
            su, sc = su + ok[:, None] * acc, sc + ok * cnt
        sums.append(su)
        counts.append(sc)
    return torch.stack(sums, dim=1), torch.stack(counts, dim=1)


def tail_sums(u, doc, s: int, off: int, carry_in=None):
    """The sums over the group still open when the call ends (zeros on a group boundary), restarted at a document start."""
    B, L = u.shape[:2]
    closes = list(range(off, L, s))
    a_end = closes[-1] + 1 if closes else 0
    if a_end >= L:
        return u.new_zeros(B, u.shape[-1]), u.new_zeros(B)
    m = (doc[:, a_end:] == doc[:, -1:]).to(u.dtype)
    acc, cnt = (m[..., None] * u[:, a_end:]).sum(1), m.sum(1)
    if carry_in is not None and not closes:
        c_acc, c_cnt, ok = carry_in
        acc, cnt = acc + ok[:, None] * c_acc, cnt + ok * c_cnt
    return acc, cnt


def sparse_recurrence(q, k1, v1, g, beta1, is_doc_start, S, carry, k2, v2, beta2):
    """The rule one token at a time. q, k1 (B, L, H, dk) at the value heads; carry: L bools; k2 / v2 / beta2 (B, n_c, ...)."""
    outs, j = [], 0
    for q_t, k_t, v_t, g_t, b_t, s_t, carries in zip(q.unbind(1), k1.unbind(1), v1.unbind(1), g.unbind(1), beta1.unbind(1),
                                                     is_doc_start.unbind(1), carry):
        S = S * (~s_t).to(S.dtype)[:, None, None, None]
        S = S * torch.exp(g_t)[:, :, None, None]
        steps = [(k_t, v_t, b_t)]
        if carries:
            steps.append((k2[:, j], v2[:, j], beta2[:, j]))
            j += 1
        for kj, vj, bj in steps:
            S = S + torch.einsum("bhk,bhv->bhkv", kj, bj[:, :, None] * (vj - torch.einsum("bhkv,bhk->bhv", S, kj)))
        outs.append(torch.einsum("bhkv,bhk->bhv", S, q_t))
    return torch.stack(outs, dim=1), S


# ------------------------------------------------------------------------------------------------ tensors and forward

class SparseSteps(nn.Module):
    n_extra = 1

    def __init__(self, d_model: int, cfg):
        super().__init__()
        check_keys(cfg)
        self.stride, self.summary, self.conv, self.first_beta = keys_of(cfg)
        self.channels = cfg.n_k_heads * cfg.k_head_dim + cfg.n_v_heads * cfg.v_head_dim
        if self.summary == "kvmean":
            self.in_proj_kv = self.in_proj_b = None
            self.beta_const = nn.Parameter(torch.zeros(cfg.n_v_heads))
        else:
            with torch.random.fork_rng(devices=[]):
                self.in_proj_kv = Linear(d_model, self.channels)
                self.in_proj_b = Linear(d_model, cfg.n_v_heads)
            self.in_proj_kv.own_init = self.in_proj_b.own_init = True
        self._maps: dict = {}
        self.reset_own(torch.Generator().manual_seed(0xD9_0D), 0.02)

    @torch.no_grad()
    def reset_own(self, g: torch.Generator, std: float) -> None:
        if self.summary == "kvmean":
            self.beta_const.zero_()
            return
        for p in (self.in_proj_kv.weight, self.in_proj_b.weight):
            if not p.is_meta:
                p.copy_((torch.randn(p.shape, generator=g, dtype=torch.float32) * std).to(device=p.device, dtype=p.dtype))

    def maps(self, L: int, off: int, device):
        key = (L, off, str(device))
        if key not in self._maps:
            rows, last, _ = row_maps(L, self.stride, off)
            self._maps[key] = (torch.tensor(rows, dtype=torch.long, device=device), torch.tensor(last, dtype=torch.long, device=device))
        return self._maps[key]


def _unit(x):
    return ops.ref.l2_normalize(x.to(torch.promote_types(x.dtype, torch.float32))).to(x.dtype)


def forward(layer, x, ctx, state):
    """(o, conv history, its document ids, S, acc, cnt)."""
    cfg, steps = layer.cfg, layer.dprod
    B, L = ctx.doc.shape
    hk, hv, dk, dv = cfg.n_k_heads, cfg.n_v_heads, cfg.k_head_dim, cfg.v_head_dim
    s, summary, fb = steps.stride, steps.summary, steps.first_beta
    u_pre = layer.in_proj_qkv(x)
    if state is not None and state.conv_input.shape[-1] != u_pre.shape[-1]:
        raise ValueError(f"this GDN cache holds {state.conv_input.shape[-1]} conv channels; a layer with the strided second step carries {u_pre.shape[-1]}")
    hist, hist_doc = (None, None) if state is None else (state.conv_input, state.conv_doc)
    q, k1, v1, conv_input, conv_doc = ops.ref.gdn_prep(u_pre, ctx.doc, layer.conv_weight, hk, hv, dk, dv, hist, hist_doc)
    pos0 = 0 if state is None else int(ctx.idx[0, 0])          # the stride's phase: the absolute index of the call's first token
    off = first_carry(pos0, s)
    n_c = 0 if off >= L else (L - 1 - off) // s + 1
    bmax = cfg.dprod.beta_max
    g, beta1 = ops.ref.gdn_gates(layer.in_proj_a(x), layer.in_proj_b(x), layer.A_log, layer.dt_bias)
    if fb == "all" or s == 1 or bmax == 1:
        beta1 = bmax * beta1
    else:
        mask = ((torch.arange(L, device=x.device) + pos0) % s == s - 1).to(beta1.dtype)[None, :, None]
        beta1 = beta1 * (1 + (bmax - 1) * mask)
    feats = carry_in = mean = None
    if summary == "xmean":
        feats = x.to(torch.promote_types(x.dtype, torch.float32))
    elif summary == "kvmean":
        feats = torch.cat([k1.reshape(B, L, hk * dk), v1.reshape(B, L, hv * dv)], dim=-1)
        feats = feats.to(torch.promote_types(feats.dtype, torch.float32))
    if summary != "none":
        if state is not None and pos0 % s != 0:                # the call's first group began in an earlier call
            if state.acc is None:
                raise ValueError("this GDN cache has no running sums: it was not written by a layer with a summarised second step")
            ok = ~ctx.is_doc_start[:, :min(off + 1, L)].any(dim=1)
            carry_in = (state.acc.to(feats.dtype), state.cnt.to(feats.dtype), ok.to(feats.dtype))
        if n_c:
            sums, counts = group_sums(feats, ctx.doc, s, off, carry_in)
            mean = sums / counts[..., None]
    k2 = v2 = beta2 = None
    if n_c and summary == "kvmean":
        k_bar, v_bar = torch.split(mean, [hk * dk, hv * dv], dim=-1)
        k2 = _unit(k_bar.reshape(B, n_c, hk, dk).to(k1.dtype))
        v2 = v_bar.reshape(B, n_c, hv, dv).to(v1.dtype)
        beta2 = (bmax * torch.sigmoid(steps.beta_const))[None, None, :].expand(B, n_c, hv).to(beta1.dtype)
    elif n_c:
        src = x[:, off::s] if summary == "none" else mean.to(x.dtype)
        k_part, v_part = torch.split(F.silu(steps.in_proj_kv(src)), [hk * dk, hv * dv], dim=-1)
        k2 = _unit(k_part.reshape(B, n_c, hk, dk))
        v2 = v_part.reshape(B, n_c, hv, dv)
        beta2 = bmax * torch.sigmoid(steps.in_proj_b(src))
    acc = cnt = None
    if summary != "none":
        acc, cnt = tail_sums(feats, ctx.doc, s, off, carry_in)
    rep = hv // hk
    dt = ops.ref.work_dtype(q)
    q_r, k1_r = q.repeat_interleave(rep, dim=2).to(dt), k1.repeat_interleave(rep, dim=2).to(dt)
    v1, g, beta1 = v1.to(dt), g.to(dt), beta1.to(dt)
    k2_r = k2.repeat_interleave(rep, dim=2).to(dt) if n_c else k1_r[:, :0]
    v2 = v2.to(dt) if n_c else v1[:, :0]
    beta2 = beta2.to(dt) if n_c else beta1[:, :0]
    S0 = x.new_zeros(B, hv, dk, dv, dtype=dt) if state is None else state.S.to(dt)
    if cfg.kernel != "recurrence" and L > 1:
        rows, last = steps.maps(L, off, x.device)
        carries = torch.tensor(carry_flags(L, s, pos0), device=x.device)
        lay = lambda t, extra: torch.cat([t, extra], dim=1).index_select(1, rows)      # noqa: E731
        qr = lay(q_r * (~carries).to(dt)[None, :, None, None], q_r[:, off::s])         # q is read on a token's last row only
        kr, vr = lay(k1_r, k2_r), lay(v1, v2)
        gr, br = lay(g, torch.zeros_like(beta2)), lay(beta1, beta2)
        sr = lay(ctx.is_doc_start, torch.zeros(B, n_c, dtype=torch.bool, device=x.device))
        o_rows, S = ops.ref.chunked_delta_rule(qr, kr, vr, gr, br, sr, S0, cfg.chunk_size)
        o = o_rows.index_select(1, last)
    else:
        o, S = sparse_recurrence(q_r, k1_r, v1, g, beta1, ctx.is_doc_start, S0, carry_flags(L, s, pos0), k2_r, v2, beta2)
    return o, conv_input, conv_doc, S, acc, cnt
