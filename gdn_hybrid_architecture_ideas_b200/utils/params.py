"""Parameter and FLOP accounting of the hybrid model, from the config alone (models are built on the meta device).

FLOP convention: a weight matrix entry costs 2 FLOPs per token forward and 6 in training; attention costs
4 * Hq * head_dim per (query, key) pair and attention layer forward (QK^T and PV), three times that in training; the GDN
recurrence about 6 * Hv * dk * dv per token forward; norms, gates, softmax and elementwise work are not counted
(reference: ced/utils/params.py:44-427, the control-architecture lines of `flops_per_token` :182-330).
"""

from __future__ import annotations

from collections import OrderedDict

import torch

from ..config import ModelConfig


def build_on_meta(cfg: ModelConfig) -> torch.nn.Module:
    """The model with shapes only (no memory)."""
    from ..models.hybrid import build_model
    with torch.device("meta"):
        return build_model(cfg)


def parameter_breakdown(model: torch.nn.Module) -> "OrderedDict[str, int]":
    groups: OrderedDict[str, int] = OrderedDict((k, 0) for k in (
        "embedding (tied)", "output embedding", "encoder GDN layers", "encoder global layers", "attention residuals",
        "GDN mixes", "norms (outside layers)", "other"))
    for name, p in model.named_parameters():
        n = p.numel()
        if name.startswith("embed."):
            groups["embedding (tied)"] += n
        elif name.startswith("out_embed."):
            groups["output embedding"] += n
        elif ".attn_res." in name:
            groups["attention residuals"] += n
        elif ".gdn_arms." in name:
            groups["GDN mixes"] += n
        elif name.startswith("encoder.layers."):
            idx = int(name.split(".")[2])
            kind = model.encoder.layers[idx].kind
            groups["encoder GDN layers" if kind == "gdn" else "encoder global layers"] += n
        elif "norm" in name:
            groups["norms (outside layers)"] += n
        else:
            groups["other"] += n
    total = sum(groups.values())
    emb = groups["embedding (tied)"] + groups["output embedding"]
    groups["embeddings"] = emb
    groups["non-embedding"] = total - emb
    groups["total"] = total
    return groups


def matrix_params(module) -> int:
    """Entries of the 2-D weights that cost FLOPs per token (embeddings excluded)."""
    if module is None:
        return 0
    return sum(p.numel() for n, p in module.named_parameters() if p.dim() == 2 and not n.startswith("embed.") and ".conv_weight" not in n and not n.endswith("conv_weight"))


def gdn_recurrence_flops(g) -> int:
    return 6 * g.n_v_heads * g.k_head_dim * g.v_head_dim


def flops_per_token(cfg: ModelConfig, seq_len: int, attn_context: float | None = None) -> dict[str, float]:
    """training: averaged over a packed row of `seq_len` (keys per query `attn_context`, default seq_len / 2: causal
    over the whole row, an upper bound under document masking); prefill_context: forward FLOPs to read one context token
    at context length seq_len (no head); decode_generated: forward FLOPs to generate one token at that context."""
    model = build_on_meta(cfg)
    head = cfg.vocab_size * cfg.d_model
    enc = matrix_params(model.encoder)
    kinds = cfg.encoder.layer_kinds()
    a = cfg.encoder.attention
    per_key = 4 * a.n_q_heads * a.head_dim * kinds.count("attention")
    recur = sum(gdn_recurrence_flops(g) for g in cfg.encoder.gdn_shapes())
    k_train = seq_len / 2 if attn_context is None else attn_context
    return {
        "matrix_params": float(enc), "head_params": float(head),
        "training": 6.0 * (enc + head) + 3.0 * (per_key * k_train + recur),
        "prefill_context": 2.0 * enc + per_key * seq_len / 2 + recur,
        "decode_generated": 2.0 * (enc + head) + per_key * seq_len + recur,
    }


def model_flops_utilisation(cfg: ModelConfig, seq_len: int, tokens_per_second: float, peak_flops: float) -> float:
    """Achieved training FLOP/s over a peak (e.g. the measured dense bf16 GEMM rate of the device)."""
    return flops_per_token(cfg, seq_len)["training"] * tokens_per_second / peak_flops
