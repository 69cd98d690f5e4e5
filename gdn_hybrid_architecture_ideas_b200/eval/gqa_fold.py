"""Grouped-query attention reads without expanding the keys: the query heads of a group are folded into the query
length axis, so the (B, S, Hkv, hd) keys and values are used as stored. At decode-time context lengths the expanded
copy of `repeat_interleave` is the largest tensor of the read (reference: ced/eval/gqa_fold.py:31-85)."""

from __future__ import annotations

import torch


def _fold(q: torch.Tensor, hkv: int) -> torch.Tensor:
    B, Lq, Hq, hd = q.shape
    g = Hq // hkv
    return q.view(B, Lq, hkv, g, hd).permute(0, 2, 1, 3, 4).reshape(B, hkv, Lq * g, hd)      # (B, Hkv, Lq g, hd)


def _unfold(o: torch.Tensor, Lq: int, Hq: int) -> torch.Tensor:
    B, hkv, _, hd = o.shape
    g = Hq // hkv
    return o.view(B, hkv, Lq, g, hd).permute(0, 2, 1, 3, 4).reshape(B, Lq, Hq, hd)


def attend_folded(q, k, v, allow):
    """q (B, Lq, Hq, hd); k, v (B, S, Hkv, hd); allow (B, Lq, S) bool. fp32 softmax, scale hd^-0.5."""
    B, Lq, Hq, hd = q.shape
    hkv = k.shape[2]
    g = Hq // hkv
    qf = _fold(q.float(), hkv)
    scores = torch.einsum("bhqd,bshd->bhqs", qf, k.float()) * hd ** -0.5
    mask = allow[:, None, :, None, :].expand(B, hkv, Lq, g, allow.shape[-1]).reshape(B, hkv, Lq * g, -1)
    probs = torch.softmax(scores.masked_fill(~mask, float("-inf")), dim=-1).nan_to_num(0.0)
    return _unfold(torch.einsum("bhqs,bshd->bhqd", probs, v.float()), Lq, Hq).to(q.dtype)


def attend_capped_folded(q, q_far, k, k_far, v, allow, far):
    """Distance-capped read: pairs flagged `far` (B, Lq, S) score q_far . k_far, the others q . k."""
    B, Lq, Hq, hd = q.shape
    hkv = k.shape[2]
    g = Hq // hkv
    near_s = torch.einsum("bhqd,bshd->bhqs", _fold(q.float(), hkv), k.float())
    far_s = torch.einsum("bhqd,bshd->bhqs", _fold(q_far.float(), hkv), k_far.float())

    def grow(m):
        return m[:, None, :, None, :].expand(B, hkv, Lq, g, m.shape[-1]).reshape(B, hkv, Lq * g, -1)

    scores = torch.where(grow(far), far_s, near_s) * hd ** -0.5
    probs = torch.softmax(scores.masked_fill(~grow(allow), float("-inf")), dim=-1).nan_to_num(0.0)
    return _unfold(torch.einsum("bhqs,bshd->bhqd", probs, v.float()), Lq, Hq).to(q.dtype)
