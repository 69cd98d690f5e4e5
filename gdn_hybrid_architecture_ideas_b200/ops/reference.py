"""Pure-PyTorch statement of every op of the model: the numerical oracle of the CUDA kernels and the CPU path.

Each function here defines WHAT the corresponding sm_100a kernel computes; kernels are tested against these in
float32/float64. Dtype rule throughout: reductions, softmaxes and norms run in at least float32 (float64 inputs stay
float64) and results return in the input dtype unless `out_dtype` says otherwise.
"""

from __future__ import annotations

import math
from functools import reduce

import torch
import torch.nn.functional as F


def work_dtype(x: torch.Tensor) -> torch.dtype:
    return torch.promote_types(x.dtype, torch.float32)


# ------------------------------------------------------------------------------------------------ norms

def rmsnorm(x, weight, eps, out_dtype=None):
    """y = x rsqrt(mean x^2 + eps) (1 + w) (reference: ced/model/norms.py:70-74)."""
    dt = work_dtype(x)
    xf = x.to(dt)
    y = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)
    return (y * (1.0 + weight.to(dt))).to(out_dtype or x.dtype)


def gated_rmsnorm(x, z, weight, eps, gate, out_dtype=None):
    """rmsnorm(x) * act(z), act SiLU or sigmoid, the product formed in the inputs' dtype
    (reference: ced/model/norms.py:77-94)."""
    act = F.silu(z) if gate == "silu" else torch.sigmoid(z)
    y = rmsnorm(x, weight, eps) * act
    return y.to(out_dtype) if out_dtype is not None else y


# ------------------------------------------------------------------------------------------------ GEMMs

def linear(x, lin):
    return F.linear(x, lin.weight)


def swiglu_mlp(x, w_gate, w_up, w_down):
    return linear(F.silu(linear(x, w_gate)) * linear(x, w_up), w_down)


# ------------------------------------------------------------------------------------------------ GDN

def l2_normalize(x, eps: float = 1e-6):
    return x * torch.rsqrt(x.pow(2).sum(-1, keepdim=True) + eps)


def causal_doc_conv(u, doc, weight, hist=None, hist_doc=None):
    """Depthwise causal conv over [history ; u] that only reads taps of the position's own document.

    u (B, L, C); doc (B, L); weight (C, K) with weight[:, K-1] on the current input; hist (B, K-1, C) and
    hist_doc (B, K-1) from earlier chunks (None: zeros / id -1). Returns (out, new_hist, new_hist_doc)
    (reference: ced/model/gdn.py:222-258)."""
    B, L, C = u.shape
    K = weight.shape[1]
    if hist is None:
        hist = u.new_zeros(B, K - 1, C)
        hist_doc = torch.full((B, K - 1), -1, dtype=torch.long, device=u.device)
    full = torch.cat([hist.to(u.dtype), u], dim=1)
    full_doc = torch.cat([hist_doc, doc], dim=1)
    out = torch.zeros_like(u)
    for back in range(K):
        lo = K - 1 - back
        same = (full_doc[:, lo:lo + L] == doc).to(u.dtype)
        out = out + full[:, lo:lo + L] * same[..., None] * weight[:, K - 1 - back].to(u.dtype)
    return out, full[:, L:], full_doc[:, L:]


def gdn_prep(u_pre, doc, conv_weight, hk, hv, dk, dv, hist=None, hist_doc=None):
    """conv (K taps, document-masked) -> SiLU -> split -> L2-normalise q and k, scale q by dk^-0.5.
    Returns q (B,L,hk,dk), k (B,L,hk,dk), v (B,L,hv,dv), new conv history and its document ids
    (reference: ced/model/gdn.py:692-699)."""
    B, L, _ = u_pre.shape
    u, h, hd = causal_doc_conv(u_pre, doc, conv_weight, hist, hist_doc)
    u = F.silu(u)
    q, k, v = torch.split(u, [hk * dk, hk * dk, hv * dv], dim=-1)
    q = l2_normalize(q.view(B, L, hk, dk)) * dk ** -0.5
    k = l2_normalize(k.view(B, L, hk, dk))
    return q, k, v.view(B, L, hv, dv), h, hd


def gdn_gates(a_lin, b_lin, A_log, dt_bias, scale: int = 1, beta_power: bool = False):
    """g = -exp(A_log) softplus(a + dt_bias) (log decay per step), beta = sigmoid(b); with `scale` s a position
    stands for s tokens: g *= s and, with beta_power, beta = 1 - (1 - sigmoid(b))^s
    (reference: ced/model/gdn.py:506-547)."""
    g = -torch.exp(A_log) * F.softplus(a_lin + dt_bias)
    if scale != 1:
        g = g * scale
    if scale != 1 and beta_power:
        bf = b_lin.to(work_dtype(b_lin))
        beta = (-torch.expm1(-scale * F.softplus(bf))).to(b_lin.dtype)
    else:
        beta = torch.sigmoid(b_lin)
    return g, beta


def delta_rule_recurrence(q, k, v, g, beta, is_doc_start, S):
    """Gated delta rule one token at a time (the ground truth): per token reset at a document start,
    S *= exp(g); S += k (x) beta (v - S^T k); o = S^T q. q,k (B,L,H,dk); v (B,L,H,dv); g,beta (B,L,H);
    S (B,H,dk,dv) (reference: ced/model/gdn.py:1153-1189)."""
    outs = []
    for q_t, k_t, v_t, g_t, b_t, s_t in zip(q.unbind(1), k.unbind(1), v.unbind(1), g.unbind(1), beta.unbind(1),
                                            is_doc_start.unbind(1)):
        S = S * (~s_t).to(S.dtype)[:, None, None, None]
        S = S * torch.exp(g_t)[:, :, None, None]
        pred = torch.einsum("bhkv,bhk->bhv", S, k_t)
        S = S + torch.einsum("bhk,bhv->bhkv", k_t, b_t[:, :, None] * (v_t - pred))
        outs.append(torch.einsum("bhkv,bhk->bhv", S, q_t))
    return torch.stack(outs, dim=1), S


def chunk_local(q, k, v, g, beta, is_doc_start, C, extras: bool = False):
    """Everything of the chunked delta rule that does not depend on the carried state, for all chunks at once.

    Inputs as delta_rule_recurrence's, L a multiple of C. Returns a dict of (B,H,n,C,...) tensors:
      U (.., dv) = (I+A)^-1 beta v;  W (.., dk) = (I+A)^-1 beta gamma k [first segment only];
      Aqk (.., C) = q_i.k_j exp(c_i-c_j) for j<=i in one document;  q_in = q gamma [first segment];
      k_out = k exp(c_last - c_j) [last segment];  carry (B,H,n) = gamma_last if the chunk has no document start else 0.
    These are exactly the operands of the sequential state pass (`chunk_scan`). Documents inside a chunk are handled
    by segment masks, so shapes never depend on where documents start (reference: ced/model/gdn_chunked.py:71-140)."""
    B, L, H, dk = q.shape
    n = L // C
    wd = reduce(torch.promote_types, (t.dtype for t in (q, k, v, g, beta)), torch.float32)

    def heads(x):
        x = x.to(wd).transpose(1, 2)
        return x.reshape(B, H, n, C, *x.shape[3:])

    q, k, v, g, beta = map(heads, (q, k, v, g, beta))
    seg = is_doc_start.to(torch.long).reshape(B, 1, n, C).cumsum(-1)
    tril = torch.ones(C, C, dtype=torch.bool, device=q.device).tril()
    pair = (seg[..., :, None] == seg[..., None, :]) & tril
    first = (seg == 0).to(wd)
    last = (seg == seg[..., -1:]).to(wd)
    zero = torch.zeros((), dtype=wd, device=q.device)
    c = g.cumsum(-1)
    strict = tril.tril(-1)
    pexp = torch.where(strict, g[..., :, None].expand(*g.shape, C), zero).cumsum(-2)   # c_i - c_j, summed directly
    decay = torch.where(pair, torch.exp(torch.where(pair, pexp, zero)), zero)
    gamma = torch.exp(c)
    to_end = torch.exp(pexp[..., -1, :])
    kb = k * beta[..., None]
    A = (kb @ k.transpose(-1, -2)) * torch.where(strict, decay, zero)
    eye = torch.eye(C, dtype=wd, device=q.device)
    rhs = torch.cat([v * beta[..., None], kb * (gamma * first)[..., None]], dim=-1)
    sol = torch.linalg.solve_triangular(eye + A, rhs, upper=False, unitriangular=True)
    U, W = sol.split([v.shape[-1], dk], dim=-1)
    parts = dict(U=U, W=W, Aqk=(q @ k.transpose(-1, -2)) * decay, q_in=q * (gamma * first)[..., None],
                 k_out=k * (to_end * last)[..., None], carry=gamma[..., -1] * (seg[..., -1] == 0).to(wd))
    if extras:          # what `delta_rule_picks` reads to form the state after a position inside a chunk
        parts.update(k=k, decay=decay, gamma_first=gamma * first)
    return parts


def chunk_scan(parts, S):
    """The sequential pass over chunks: v_new = U - W S; o = q_in S + Aqk v_new; S = carry S + k_out^T v_new.
    Returns o (B,H,n,C,dv) and the final state (reference: ced/model/gdn_chunked.py:142-160)."""
    outs = []
    for U, W, qi, Aqk, ko, cy in zip(*(parts[n].unbind(2) for n in ("U", "W", "q_in", "Aqk", "k_out", "carry"))):
        vn = U - W @ S
        outs.append(qi @ S + Aqk @ vn)
        S = S * cy[..., None, None] + ko.transpose(-1, -2) @ vn
    return torch.stack(outs, dim=2), S


def chunked_delta_rule(q, k, v, g, beta, is_doc_start, S, chunk_size: int = 64):
    """delta_rule_recurrence computed chunk by chunk (WY / UT-transform form, arXiv 2412.06464 section 3.3)."""
    B, L, H, dk = q.shape
    out_dt = reduce(torch.promote_types, (t.dtype for t in (q, k, v, g, beta, S)))
    C = min(chunk_size, L)
    pad = (-L) % C
    if pad:
        q, k, v = (F.pad(t, (0, 0, 0, 0, 0, pad)) for t in (q, k, v))
        g, beta = (F.pad(t, (0, 0, 0, pad)) for t in (g, beta))
        is_doc_start = F.pad(is_doc_start, (0, pad))
    parts = chunk_local(q, k, v, g, beta, is_doc_start, C)
    o, S = chunk_scan(parts, S.to(parts["U"].dtype))
    o = o.reshape(B, H, L + pad, -1)[:, :, :L].transpose(1, 2)
    return o.to(out_dt), S.to(out_dt)


def delta_rule_picks(q, k, v, g, beta, is_doc_start, S, picks, kernel: str = "chunked", chunk_size: int = 64):
    """The gated delta rule that also returns the state AFTER chosen positions. picks (B, K) long: indices into the call,
    any value >= L for an unused entry (its state is returned as zeros). Returns (o, S_final, states (B, K, H, dk, dv)).

    "recurrence": the token loop, each pick copied out when its token has been written. "chunked": the WY form; the
    state after local index i of a chunk that starts at S_n is
        [no document start up to i] exp(c_i) S_n + sum_{j <= i, same document} exp(c_i - c_j) k_j (x) v_new_j
    with v_new = U - W S_n the chunk's corrected values, so each pick is one gather of its chunk's operands and one
    small product, whatever the number of positions (fixed shapes; no state per position is formed)."""
    B, L, H, dk = q.shape
    K = picks.shape[1]
    ok = picks < L
    if kernel == "recurrence" or L == 1:
        out = S.new_zeros(B, K, *S.shape[1:]) if K else S.new_zeros(B, 0, *S.shape[1:])
        outs = []
        for t, (q_t, k_t, v_t, g_t, b_t, s_t) in enumerate(zip(q.unbind(1), k.unbind(1), v.unbind(1), g.unbind(1), beta.unbind(1),
                                                                is_doc_start.unbind(1))):
            S = S * (~s_t).to(S.dtype)[:, None, None, None]
            S = S * torch.exp(g_t)[:, :, None, None]
            pred = torch.einsum("bhkv,bhk->bhv", S, k_t)
            S = S + torch.einsum("bhk,bhv->bhkv", k_t, b_t[:, :, None] * (v_t - pred))
            outs.append(torch.einsum("bhkv,bhk->bhv", S, q_t))
            if K:
                out = torch.where((picks == t)[:, :, None, None, None], S[:, None], out)
        return torch.stack(outs, dim=1), S, out
    out_dt = reduce(torch.promote_types, (t.dtype for t in (q, k, v, g, beta, S)))
    C = min(chunk_size, L)
    pad = (-L) % C
    if pad:
        q, k, v = (F.pad(t, (0, 0, 0, 0, 0, pad)) for t in (q, k, v))
        g, beta = (F.pad(t, (0, 0, 0, pad)) for t in (g, beta))
        is_doc_start = F.pad(is_doc_start, (0, pad))
    parts = chunk_local(q, k, v, g, beta, is_doc_start, C, extras=True)
    S = S.to(parts["U"].dtype)
    outs, starts, news = [], [], []
    for U, W, qi, Aqk, ko, cy in zip(*(parts[n].unbind(2) for n in ("U", "W", "q_in", "Aqk", "k_out", "carry"))):
        starts.append(S)
        vn = U - W @ S
        news.append(vn)
        outs.append(qi @ S + Aqk @ vn)
        S = S * cy[..., None, None] + ko.transpose(-1, -2) @ vn
    o = torch.stack(outs, dim=2).reshape(B, H, L + pad, -1)[:, :, :L].transpose(1, 2)
    at = picks.clamp(max=L - 1)
    n_i, i_i = at // C, at % C
    rows = torch.arange(B, device=q.device)[:, None]
    S_n = torch.stack(starts, dim=2)[rows, :, n_i]                                       # (B, K, H, dk, dv)
    v_new = torch.stack(news, dim=2)[rows, :, n_i]                                       # (B, K, H, C, dv)
    keys = parts["k"][rows, :, n_i]                                                      # (B, K, H, C, dk)
    weight = parts["decay"].expand(B, H, -1, -1, -1)[rows, :, n_i, i_i]                  # (B, K, H, C): exp(c_i - c_j), 0 outside the document or after i
    lead = parts["gamma_first"][rows, :, n_i, i_i]                                       # (B, K, H)
    states = lead[..., None, None] * S_n + torch.einsum("bkhc,bkhcd,bkhce->bkhde", weight, keys, v_new)
    states = states * ok[:, :, None, None, None].to(states.dtype)
    return o.to(out_dt), S.to(out_dt), states.to(out_dt)


# ------------------------------------------------------------------------------------------------ attention

def attention(q, k, v, q_idx, q_doc, k_idx, k_doc, k_ok=None, q_far=None, k_far=None, cap=None, return_lse=False):
    """Causal, document-masked softmax attention with grouped KV heads and an optional rotary distance cap.

    q (B,Lq,Hq,hd) and k,v (B,S,Hkv,hd), Hq a multiple of Hkv (KV head j serves query heads j*g .. (j+1)*g-1).
    A key is allowed iff k_ok, k_idx <= q_idx and k_doc == q_doc. With a cap C, a pair with q_idx - k_idx > C is
    scored q_far . k_far (query rotated by C against the unrotated key) instead of q . k. One softmax in >= float32,
    scale hd^-0.5 (reference: ced/model/attention.py:227-260, 519-553)."""
    hq, hkv = q.shape[2], k.shape[2]
    rep = hq // hkv
    dt = work_dtype(q)
    scale = q.shape[-1] ** -0.5
    allow = (k_idx[:, None, :] <= q_idx[:, :, None]) & (k_doc[:, None, :] == q_doc[:, :, None])
    if k_ok is not None:
        allow = allow & k_ok[:, None, :]
    kk = k.repeat_interleave(rep, dim=2).to(dt)
    vv = v.repeat_interleave(rep, dim=2).to(dt)
    s = torch.einsum("bqhd,bshd->bhqs", q.to(dt), kk) * scale
    if cap is not None:
        far = (q_idx[:, :, None] - k_idx[:, None, :]) > cap
        sf = torch.einsum("bqhd,bshd->bhqs", q_far.to(dt), k_far.repeat_interleave(rep, dim=2).to(dt)) * scale
        s = torch.where(far[:, None], sf, s)
    s = s.masked_fill(~allow[:, None], float("-inf"))
    p = torch.softmax(s, dim=-1)
    o = torch.einsum("bhqs,bshd->bqhd", p, vv).to(q.dtype)
    if return_lse:
        return o, torch.logsumexp(s, dim=-1)
    return o


# ------------------------------------------------------------------------------------------------ depth mix

def depth_mix(sources, query, gain, eps, return_weights=False):
    """Per position, h = sum_i softmax_i(w . RMSNorm(v_i)) v_i over the sources v_i (B,L,d), with the logit formed
    without a normalised copy: (v @ (w (1+g))) rsqrt(mean v^2 + eps); >= float32, autocast off
    (reference: ced/model/attn_res.py:457-482)."""
    v0 = sources[0]
    dt = work_dtype(v0)
    with torch.autocast(v0.device.type, enabled=False):
        u = query.to(dt) * (1.0 + gain.to(dt))
        logits = [(v.to(dt) @ u) * torch.rsqrt(v.to(dt).pow(2).mean(-1) + eps) for v in sources]
        alpha = torch.softmax(torch.stack(logits, dim=-1), dim=-1)
        h = alpha[..., 0:1] * v0.to(dt)
        for i in range(1, len(sources)):
            h = h + alpha[..., i:i + 1] * sources[i].to(dt)
    h = h.to(v0.dtype)
    return (h, alpha) if return_weights else h


def depth_mix_heads(sources, query, gain, eps, heads: int):
    """`depth_mix` with `heads` softmaxes over the sources, one per contiguous slice of d / heads channels: the logit of
    slice h is sum over the slice of u_c v_c times rsqrt(mean over ALL d of v^2 + eps) (the key norm over the full row,
    then sliced); each slice of the output is its own weighted sum (reference: ced/model/attn_res.py:553-577)."""
    v0 = sources[0]
    dt = work_dtype(v0)
    with torch.autocast(v0.device.type, enabled=False):
        u = query.to(dt) * (1.0 + gain.to(dt))
        logits = []
        for v in sources:
            vf = v.to(dt)
            r = torch.rsqrt(vf.pow(2).mean(-1) + eps)
            logits.append((vf * u).unflatten(-1, (heads, -1)).sum(-1) * r[..., None])
        alpha = torch.softmax(torch.stack(logits, dim=-1), dim=-1)                # (B, L, H, n)
        h = alpha[..., 0:1] * v0.to(dt).unflatten(-1, (heads, -1))
        for i in range(1, len(sources)):
            h = h + alpha[..., i:i + 1] * sources[i].to(dt).unflatten(-1, (heads, -1))
    return h.flatten(-2).to(v0.dtype)


def kda_recurrence(q, k, v, g, beta, is_doc_start, S):
    """The delta rule with one decay per key channel (KDA), a token at a time: at a document start S = 0; then
    S <- Diag(exp(g_t)) S (row i of S by its own decay), S += k (beta (v - S^T k))^T, o = S^T q. q, k (B, L, H, dk)
    already repeated to the value heads, v (B, L, H, dv), g (B, L, H, dk) <= 0, beta (B, L, H), S (B, H, dk, dv). With g the
    same in every channel this is the scalar rule (reference: ced/model/gdn_kda.py:285-300)."""
    dt = work_dtype(q)
    q, k, v, g, beta, S = (t.to(dt) for t in (q, k, v, g, beta, S))
    outs = []
    for t in range(q.shape[1]):
        S = S * (~is_doc_start[:, t]).to(dt)[:, None, None, None]
        S = S * torch.exp(g[:, t])[..., None]
        delta = beta[:, t, :, None] * (v[:, t] - torch.einsum("bhkv,bhk->bhv", S, k[:, t]))
        S = S + torch.einsum("bhk,bhv->bhkv", k[:, t], delta)
        outs.append(torch.einsum("bhkv,bhk->bhv", S, q[:, t]))
    return torch.stack(outs, dim=1), S


def kda_chunked(q, k, v, g, beta, is_doc_start, S, chunk_size: int = 64):
    """The same function in chunks of C tokens. With c_t the running sum of g inside the chunk (per channel) and
    D[t, j] = exp(c_t - c_j) for j <= t in the same document segment (taken per channel inside the products, so nothing
    overflows), the writes u solve the unit lower-triangular system

        (I + diag(beta) M) U = diag(beta) (V - [t before the chunk's first document start] (exp(c_t) k_t)^T S_0),
        M[t, j] = sum_c k_t[c] k_j[c] D[t, j, c]  (j < t),

    the reads are o_t = [..] S_0^T (exp(c_t) q_t) + sum_{j <= t} (sum_c q_t[c] k_j[c] D[t, j, c]) u_j, and the state
    after the chunk is [no start in the chunk] Diag(exp(c_C)) S_0 + sum_{j in the last segment} (exp(c_C - c_j) k_j) u_j^T
    (reference: ced/model/gdn_kda.py:303-382 states the same WY form)."""
    dt = work_dtype(q)
    q, k, v, g, beta, S = (t.to(dt) for t in (q, k, v, g, beta, S))
    B, L, H, dk = k.shape
    outs = []
    for a in range(0, L, chunk_size):
        sl = slice(a, min(a + chunk_size, L))
        qc, kc, vc, gc, bc = (t[:, sl].transpose(1, 2) for t in (q, k, v, g, beta))     # (B, H, C, .)
        C = qc.shape[2]
        seg = is_doc_start[:, sl].long().cumsum(1)                                        # (B, C)
        c = gc.cumsum(2)                                                                  # (B, H, C, dk)
        same = (seg[:, :, None] == seg[:, None, :]) & torch.tril(torch.ones(C, C, dtype=torch.bool, device=q.device))
        D = torch.exp((c[:, :, :, None, :] - c[:, :, None, :, :]).clamp(max=0.0)) * same[:, None, :, :, None].to(dt)
        M = torch.einsum("bhtc,bhjc,bhtjc->bhtj", kc, kc, D)
        P = torch.einsum("bhtc,bhjc,bhtjc->bhtj", qc, kc, D)
        first = (seg == 0).to(dt)[:, None, :, None]                                       # still the incoming document
        ec = torch.exp(c)
        rhs = bc[..., None] * (vc - first * torch.einsum("bhtc,bhcv->bhtv", ec * kc, S))
        lower = torch.eye(C, dtype=dt, device=q.device) + bc[..., None] * M.tril(-1)
        U = torch.linalg.solve_triangular(lower, rhs, upper=False, unitriangular=True)
        o = first * torch.einsum("bhtc,bhcv->bhtv", ec * qc, S) + torch.einsum("bhtj,bhjv->bhtv", P, U)
        outs.append(o.transpose(1, 2))
        last = (seg == seg[:, -1:]).to(dt)[:, None, :, None]
        tail = torch.exp(c[:, :, -1:, :] - c) * kc * last                                 # exp(c_C - c_j) k_j: <= |k_j|
        S = (seg[:, -1] == 0).to(dt)[:, None, None, None] * ec[:, :, -1, :, None] * S + torch.einsum("bhjc,bhjv->bhcv", tail, U)
    return torch.cat(outs, dim=1), S


def entmax15(x: torch.Tensor, allow: torch.Tensor) -> torch.Tensor:
    """alpha = 1.5 entmax over the last dimension of x (already halved scores: p = [x - tau]_+^2 summing to 1) among the
    allowed entries, by the sort-based closed form: a support of the k largest entries gives tau_k = mean_k -
    sqrt((1 - k var_k) / k), the support size is the largest k with tau_k <= x_(k). Every support entry lies within 1 of
    the row maximum, so entries below max - 2 (and the masked ones) are placed at max - 2, where they never enter the
    support. tau is recomputed from the support with two-pass sums (reference: ced/model/entmax.py:14-45)."""
    any_ok = allow.any(-1, keepdim=True)
    xm = torch.where(allow, x, torch.full_like(x, float("-inf"))).amax(-1, keepdim=True)
    xs = torch.where(allow, (x - torch.where(any_ok, xm, torch.zeros_like(xm))).clamp(min=-2.0), torch.full_like(x, -2.0))
    srt = xs.sort(dim=-1, descending=True).values
    k = torch.arange(1, x.shape[-1] + 1, device=x.device, dtype=x.dtype)
    mean = srt.cumsum(-1) / k
    meansq = srt.square().cumsum(-1) / k
    delta = (1.0 - k * (meansq - mean.square())) / k
    tau_k = mean - delta.clamp(min=0.0).sqrt()
    kstar = (tau_k <= srt).sum(-1, keepdim=True).clamp(min=1)
    in_top = torch.arange(x.shape[-1], device=x.device) < kstar
    kf = kstar.to(x.dtype)
    m = (srt * in_top).sum(-1, keepdim=True) / kf
    ssd = ((srt - m).square() * in_top).sum(-1, keepdim=True)
    tau = m - ((1.0 - ssd).clamp(min=0.0) / kf).sqrt()
    p = (xs - tau).clamp(min=0.0).square()
    return torch.where(any_ok, p, torch.zeros_like(p))


ENTMAX_AUTO_ELEMENTS = 1 << 25     # score elements of one query chunk when the chunk size is 0 (auto): 128 MiB in float32


def entmax_attention(q, k, v, q_idx, q_doc, k_idx, k_doc, k_ok=None, chunk: int = 0):
    """Causal, document-masked attention with the alpha = 1.5 entmax in place of the softmax: z = q . k hd^-0.5 over the
    allowed keys, p = entmax15(z / 2), out = p v; grouped KV heads as `attention`; >= float32, autocast off. Queries go
    in chunks of `chunk` rows (0: as many as keep one chunk's (B, Hq, rows, S) scores at ENTMAX_AUTO_ELEMENTS); with a
    gradient each chunk is recomputed in the backward, so only one chunk's scores are alive at a time
    (reference: ced/model/entmax.py:1-13, 372-377)."""
    B, Lq, hq, _ = q.shape
    S, rep = k.shape[1], hq // k.shape[2]
    dt = work_dtype(q)
    scale = q.shape[-1] ** -0.5

    def rows_out(qc, kk, vv, qi, qd):
        allow = (k_idx[:, None, :] <= qi[:, :, None]) & (k_doc[:, None, :] == qd[:, :, None])
        if k_ok is not None:
            allow = allow & k_ok[:, None, :]
        with torch.autocast(qc.device.type, enabled=False):
            z = torch.einsum("bqhd,bshd->bhqs", qc.to(dt), kk.repeat_interleave(rep, dim=2).to(dt)) * scale
            p = entmax15(z * 0.5, allow[:, None].expand_as(z))
            return torch.einsum("bhqs,bshd->bqhd", p, vv.repeat_interleave(rep, dim=2).to(dt))

    rows = chunk if chunk > 0 else ENTMAX_AUTO_ELEMENTS // max(1, B * hq * S)
    rows = max(1, min(rows, Lq))
    if rows >= Lq:
        return rows_out(q, k, v, q_idx, q_doc).to(q.dtype)
    grad = torch.is_grad_enabled() and any(t.requires_grad for t in (q, k, v))
    outs = []
    for a in range(0, Lq, rows):
        args = (q[:, a:a + rows], k, v, q_idx[:, a:a + rows], q_doc[:, a:a + rows])
        if grad:
            from torch.utils.checkpoint import checkpoint
            outs.append(checkpoint(rows_out, *args, use_reentrant=False))
        else:
            outs.append(rows_out(*args))
    return torch.cat(outs, dim=1).to(q.dtype)


# ------------------------------------------------------------------------------------------------ loss

def lm_loss_sums(hidden, weight, targets, weights=None, z_loss: float = 0.0):
    """Sum over positions of weight * (CE + z_loss * lse^2) with fp32 logits, and the plain CE sum.
    hidden (N,d), weight (V,d), targets (N,) (or (N,s) with weights (N,s) for bags); a target < 0 is ignored
    (reference: ced/train/loss.py:20-58, ced/train/fused_head.py:56-66)."""
    dt = work_dtype(hidden)
    logits = F.linear(hidden.to(dt), weight.to(dt))
    lse = torch.logsumexp(logits, dim=-1)
    if targets.dim() == 1:
        targets, weights = targets[:, None], (torch.ones_like(targets, dtype=dt)[:, None] if weights is None else weights[:, None])
    valid = targets >= 0
    picked = logits.gather(1, targets.clamp(min=0))
    w = weights.to(dt) * valid.to(dt)
    ce = ((lse[:, None] - picked) * w).sum()
    wsum = w.sum(1)
    total = ce + z_loss * (lse.pow(2) * wsum).sum()
    return total, ce


def embedding(tokens, weight):
    """Rows of `weight`; bags (B,L,s) give the mean of their s rows in the table's dtype
    (reference: ced/model/control.py:436-455)."""
    e = F.embedding(tokens, weight)
    return e.mean(dim=2) if tokens.dim() == 3 else e


def input_mixes(x, y_write, lam_write, y_read=None, lam_read=None):
    """(x + lam_w (y_write - x), x + lam_r (y_read - x) or None): the write and query inputs of a GDN layer with mixes,
    formed in >= fp32 and returned in the dtype projections compute in (reference: ced/model/gdn.py:599-640)."""
    wd = torch.promote_types(x.dtype, torch.float32)
    dev = x.device.type
    out_dtype = torch.get_autocast_dtype(dev) if torch.is_autocast_enabled(dev) else x.dtype

    def mix(y, lam):
        return torch.addcmul(x.to(wd), y.to(wd) - x.to(wd), lam.to(wd)).to(out_dtype)

    return mix(y_write, lam_write), (None if y_read is None else mix(y_read, lam_read))
