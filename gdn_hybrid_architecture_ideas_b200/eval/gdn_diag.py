"""GDN state diagnostics: how the recurrent state of each GDN layer evolves along a long row.

The row is read in blocks through the cache; after each block the per-layer state S (B, Hv, dk, dv) is measured:
Frobenius norm, largest singular value, stable rank ||S||_F^2 / sigma_max^2, and the relative change since the last
block. Drift of these along the row shows saturation or forgetting (reference: ced/eval/gdn_diag.py:82-430).
"""

from __future__ import annotations

import torch


def state_measures(S: torch.Tensor) -> dict[str, torch.Tensor]:
    """Per head: (B, Hv) tensors."""
    Sf = S.float()
    fro = Sf.flatten(-2).norm(dim=-1)
    top = torch.linalg.matrix_norm(Sf, ord=2)
    return {"fro": fro, "sigma_max": top, "stable_rank": (fro / top.clamp_min(1e-30)) ** 2}


@torch.no_grad()
def encoder_gdn_diag(model, tokens: torch.Tensor, doc_ids: torch.Tensor, block: int = 2048, autocast_dtype=None) -> list[dict]:
    """One record per block: position reached and, per GDN layer, the head-averaged measures."""
    dev = next(model.parameters()).device
    tokens, doc_ids = tokens.to(dev), doc_ids.to(dev)
    cache, prev, out = None, {}, []
    for s in range(0, tokens.shape[1], block):
        with torch.autocast(dev.type, dtype=autocast_dtype, enabled=autocast_dtype is not None):
            res = model.forward(tokens[:, s:s + block], doc_ids[:, s:s + block], cache=cache, return_cache=True, return_hidden=True)
        cache = res.cache
        rec = {"position": min(s + block, tokens.shape[1]), "layers": {}}
        for i, (layer, c) in enumerate(zip(model.encoder.layers, cache.encoder)):
            if layer.kind != "gdn" or c is None or c.S is None:
                continue
            m = {k: float(v.mean()) for k, v in state_measures(c.S).items()}
            if i in prev:
                m["rel_change"] = float((c.S.float() - prev[i]).norm() / prev[i].norm().clamp_min(1e-30))
            prev[i] = c.S.float().clone()
            rec["layers"][i] = m
        out.append(rec)
    return out
