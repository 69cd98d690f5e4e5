"""Diagnostics for token-superposition training: where a bits-per-byte difference between two models lives.

Pure functions of arrays and evaluation rows (reference: ced/eval/tst_diag.py:1-75 defines the quantities):

* frequency classes of token ids from training counts: ids ranked by (count descending, id ascending); with m_i the
  share of training tokens held by the ids ranked before i, "frequent" m_i < 1/3, "mid" < 2/3, "rare" < 0.95, "rarest"
  the rest (exact integer comparisons);
* position buckets: row position [0,128) [128,512) [512,2048) [2048,L) and context inside the document [0,512) [512,inf)
  (context counted from the row's start for a document that began in an earlier row);
* bucket sums of per-position cross-entropy: nats, bytes and tokens per class, whose contributions N / (ln 2 B_total)
  add up to the set's bits per byte;
* grafts: one model's body with another's embedding and head tensors;
* the short convolution's span: per channel the energy per lag e_j = w_j^2 / sum w^2, its centroid lag, the smallest
  number of taps holding 90 % of the energy, and the share of pass-through channels (e_0 >= 0.9);
* the change of the embedding norm's output when a bag's mean is replaced by sum / sqrt(s).
"""

from __future__ import annotations

import math

import numpy as np
import torch

CLASSES = ("frequent", "mid", "rare", "rarest")
ROW_EDGES = (0, 128, 512, 2048)
CONTEXT_EDGES = (0, 512)
EMBED_KEYS = ("embed.weight", "out_embed.weight")
NORM_KEYS = ("embed_norm.weight", "final_norm.weight")


def frequency_classes(counts):
    """(classes (V,) uint8 in 0..3, info) from the training count of every token id."""
    counts = np.asarray(counts, dtype=np.int64)
    if counts.ndim != 1 or counts.size == 0 or counts.min() < 0 or counts.sum() <= 0:
        raise ValueError("counts: a 1-D array of non-negative counts with a positive sum")
    total = int(counts.sum())
    order = np.lexsort((np.arange(counts.size), -counts))          # count descending, id ascending
    ranked = counts[order]
    before = np.cumsum(ranked) - ranked
    by_rank = np.where(before * 3 < total, 0, np.where(before * 3 < 2 * total, 1, np.where(before * 20 < 19 * total, 2, 3))).astype(np.uint8)
    classes = np.empty(counts.size, dtype=np.uint8)
    classes[order] = by_rank
    info = {"total_tokens": total, "vocab": int(counts.size), "zero_count_ids": int((counts == 0).sum()), "classes": {}}
    for k, name in enumerate(CLASSES):
        c = counts[classes == k]
        info["classes"][name] = {"ids": int(c.size), "mass": float(c.sum() / total), "min_count": int(c.min()) if c.size else None,
                                 "max_count": int(c.max()) if c.size else None}
    return classes, info


def class_name_three(k: int) -> str:
    """Three-bucket name: rare absorbs rarest."""
    return ("frequent", "mid", "rare", "rare")[k]


def context_in_document(doc_ids: torch.Tensor) -> torch.Tensor:
    """(N, L): how many earlier positions of the same document the row holds."""
    N, L = doc_ids.shape
    idx = torch.arange(L, device=doc_ids.device).expand(N, L)
    start = torch.ones_like(doc_ids, dtype=torch.bool)
    start[:, 1:] = doc_ids[:, 1:] != doc_ids[:, :-1]
    first = torch.where(start, idx, torch.zeros_like(idx)).cummax(dim=1).values
    return idx - first


def bucket_of(x: torch.Tensor, edges) -> torch.Tensor:
    """Index of the last lower edge <= x (edges ascending, edges[0] = 0)."""
    return torch.bucketize(x.contiguous(), torch.tensor(edges[1:], dtype=x.dtype, device=x.device), right=True)


def sum_by(key: torch.Tensor, K: int, scored: torch.Tensor, value: torch.Tensor) -> torch.Tensor:
    """(N, K) float64: per row the sum of `value` over scored positions whose key is k."""
    N = key.shape[0]
    flat = (torch.arange(N, device=key.device)[:, None] * K + key).reshape(-1)
    out = torch.zeros(N * K, dtype=torch.float64, device=key.device)
    out.index_add_(0, flat, torch.where(scored, value.double(), torch.zeros((), dtype=torch.float64, device=key.device)).reshape(-1))
    return out.view(N, K)


def aggregate_ce(ce: torch.Tensor, tokens: torch.Tensor, targets: torch.Tensor, doc_ids: torch.Tensor, scored: torch.Tensor,
                 byte_lens: torch.Tensor, classes: np.ndarray) -> dict[str, np.ndarray]:
    """Per-row sums of nats / bytes / tokens split four ways: by the target token's class, the input token's class, the row
    position bucket and the in-document context bucket. Arrays (N, K, 3) with the last axis (nats, bytes, tokens)."""
    cls = torch.from_numpy(classes.astype(np.int64))
    keys = {"target_class": (cls[targets.clamp_min(0)], len(CLASSES)), "input_class": (cls[tokens], len(CLASSES)),
            "row_position": (bucket_of(torch.arange(tokens.shape[1]).expand_as(tokens), ROW_EDGES), len(ROW_EDGES)),
            "context": (bucket_of(context_in_document(doc_ids), CONTEXT_EDGES), len(CONTEXT_EDGES))}
    ones = torch.ones_like(ce)
    return {name: torch.stack([sum_by(k, K, scored, ce), sum_by(k, K, scored, byte_lens.to(ce.dtype)), sum_by(k, K, scored, ones)], dim=-1).numpy()
            for name, (k, K) in keys.items()}


def contributions(agg: np.ndarray) -> dict:
    """From one split's (N, K, 3) sums: each class's own bits per byte and its contribution to the set's (they add up)."""
    s = agg.sum(0)
    total_bytes = s[:, 1].sum()
    own = np.divide(s[:, 0], math.log(2) * s[:, 1], out=np.full(s.shape[0], np.nan), where=s[:, 1] > 0)
    return {"bpb": own, "contribution": s[:, 0] / (math.log(2) * total_bytes), "tokens": s[:, 2], "set_bpb": s[:, 0].sum() / (math.log(2) * total_bytes)}


def graft_state(body: dict, donor: dict, norms: bool = False) -> dict:
    """`body`'s tensors with the embedding and (untied) head of `donor`; with norms also the two gains beside them."""
    keys = EMBED_KEYS + (NORM_KEYS if norms else ())
    for k in keys:
        for who, sd in (("body", body), ("donor", donor)):
            if k not in sd:
                raise ValueError(f"{who} state has no {k}" + (" (a tied head has no out_embed.weight)" if k == "out_embed.weight" else ""))
        if tuple(body[k].shape) != tuple(donor[k].shape):
            raise ValueError(f"{k}: shape {tuple(body[k].shape)} against {tuple(donor[k].shape)}")
    out = dict(body)
    out.update({k: donor[k].detach().clone() for k in keys})
    return out


def conv_span_stats(weight: torch.Tensor, groups: dict[str, tuple[int, int]]) -> dict:
    """Span of a (channels, K) depthwise causal conv ([:, K-1] multiplies the current token), for all channels and per group."""
    w = weight.detach().double()
    K = w.shape[1]
    e = w.flip(1).square()                                   # column j = lag j
    tot = e.sum(1, keepdim=True)
    e = torch.where(tot > 0, e / tot.clamp_min(1e-300), torch.full_like(e, 1.0 / K))
    span90 = (e.cumsum(1) < 0.9 - 1e-12).sum(1) + 1
    lag = torch.arange(K, dtype=torch.float64)
    out = {}
    for name, (a, b) in {"all": (0, w.shape[0]), **groups}.items():
        g = e[a:b]
        out[name] = {"channels": int(b - a), "lag_energy": g.mean(0).tolist(), "centroid_lag": float((g * lag).sum(1).mean()),
                     "span90": float(span90[a:b].double().mean()), "pass_through": float((g[:, 0] >= 0.9).double().mean())}
    return out


def gdn_conv_groups(cfg_gdn) -> dict[str, tuple[int, int]]:
    """Channel ranges of q, k, v in a GDN layer's convolution."""
    nq = cfg_gdn.n_k_heads * cfg_gdn.k_head_dim
    return {"q": (0, nq), "k": (nq, 2 * nq), "v": (2 * nq, 2 * nq + cfg_gdn.n_v_heads * cfg_gdn.v_head_dim)}


def bag_norm_eps_change(mean_sq, s: int, eps: float) -> np.ndarray:
    """Relative change of the embedding norm's output when a bag's mean m becomes sqrt(s) m, per bag with ms = mean(m^2)."""
    ms = np.asarray(mean_sq, dtype=np.float64)
    return np.sqrt((ms + eps) / (ms + eps / s)) - 1.0
