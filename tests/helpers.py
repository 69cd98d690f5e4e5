"""Shared test helpers: packed multi-document rows, parameter perturbation (so zero-initialised gates and queries do
not make a test vacuous), tiny models in float64."""

from __future__ import annotations

import os
from pathlib import Path

import torch

from gdn_hybrid_architecture_ideas_b200 import config as C
from gdn_hybrid_architecture_ideas_b200.models import build_model


REFERENCE = Path(os.environ.get("GHB_REFERENCE_PATH") or Path(__file__).resolve().parent.parent.parent / "reference") / "code"


def perturb(model, scale: float = 0.05, seed: int = 1):
    g = torch.Generator().manual_seed(seed)
    with torch.no_grad():
        for p in model.parameters():
            p.add_(torch.randn(p.shape, generator=g, dtype=torch.float64).to(p.dtype) * scale)
    return model


def make_model(cfg=None, dtype=torch.float64, seed: int = 0, perturbed: bool = True):
    torch.manual_seed(seed)
    m = build_model(cfg or C.tiny_full_config()).to(dtype)
    return perturb(m) if perturbed else m


def random_rows(B: int, L: int, vocab: int = 256, seed: int = 2, docs: bool = True):
    g = torch.Generator().manual_seed(seed)
    tok = torch.randint(0, vocab, (B, L), generator=g)
    doc = torch.zeros(B, L, dtype=torch.long)
    if docs:
        for b in range(B):
            cuts = sorted(torch.randint(1, L, (2,), generator=g).tolist())
            for c in cuts:
                doc[b, c:] += 1
    return tok, doc
