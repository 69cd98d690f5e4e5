"""Tensor-parallel form of the hybrid model.

Each rank builds the same module tree from a local config whose head counts (GDN key / value heads, attention query /
KV heads) and SwiGLU hidden size are divided by the world size, so every projection into heads is naturally the
rank's column slice and every projection out of heads its row slice; `apply` tags those `Linear`s with the
tensor-parallel context so that `ops.linear` runs them through the fused all-gather / reduce-scatter GEMMs. The
residual stream, norms and depth mixes work on the rank's token shard. Replicated parameters (embedding, norm gains,
depth-mix queries, mix lambdas) see only the shard's tokens, so their gradients are summed over ranks after the
backward; sharded parameters' gradients are complete as computed. `shard_state_dict` cuts a full model's weights into
one rank's, for tests and for loading unsharded checkpoints. The reference has no tensor parallelism.
"""

from __future__ import annotations

import copy

import torch

from ..config import ModelConfig

COLUMN = ("in_proj_qkv", "in_proj_z", "in_proj_a", "in_proj_b", "q_proj", "k_proj", "v_proj", "g_proj", "w_gate", "w_up")
ROW = ("out_proj", "o_proj", "w_down")
SHARDED_VECTORS = ("conv_weight", "A_log", "dt_bias", "temp_w")


def local_model_config(cfg: ModelConfig, world: int) -> ModelConfig:
    enc = cfg.encoder
    if enc.gdn_shape_by_layer:
        raise ValueError("tensor parallel shards one GDN shape for the whole stack: model.encoder.gdn_shape_by_layer is not built with it")
    a, g = enc.attention, enc.gdn
    if enc.attn_res == "ldm":
        raise ValueError("tensor parallel is not built with model.encoder.attn_res 'ldm' (the depth memory walks the full stream)")
    if g.kda.decay != "scalar" or g.erase.mode != "none" or g.dprod.n_h != 1:
        raise ValueError("tensor parallel shards the scalar-decay GDN layer: gdn.kda.decay 'channel', gdn.erase.mode 'eda' and "
                         "gdn.dprod.n_h >= 2 are not built with it")
    if a.normalizer != "softmax":
        raise ValueError("tensor parallel shards the softmax attention: attention.normalizer 'asentmax' is not built with it")
    sizes = {"gdn.n_k_heads": g.n_k_heads, "gdn.n_v_heads": g.n_v_heads, "attention.n_q_heads": a.n_q_heads,
             "attention.n_kv_heads": a.n_kv_heads, "ffn_hidden": cfg.ffn_hidden}
    bad = [k for k, v in sizes.items() if v % world]
    if bad:
        raise ValueError(f"tensor parallel over {world} ranks needs {bad} divisible by {world}: {sizes}")
    if a.kv_sharing != "gqa":
        raise ValueError("tensor parallel shards attention by KV head: attention.kv_sharing must be 'gqa'")
    if (cfg.ffn_hidden // world) % 8:
        raise ValueError("tensor parallel: ffn_hidden / world must be a multiple of 8")
    out = copy.deepcopy(cfg)
    out.ffn_hidden = cfg.ffn_hidden // world
    out.encoder.gdn.n_k_heads, out.encoder.gdn.n_v_heads = g.n_k_heads // world, g.n_v_heads // world
    out.encoder.attention.n_q_heads, out.encoder.attention.n_kv_heads = a.n_q_heads // world, a.n_kv_heads // world
    return out


def apply(model, tp) -> None:
    """Tags the sharded projections and parameters of a model built from `local_model_config`."""
    from ..models.linear import Linear

    model.tp = tp
    for name, mod in model.named_modules():
        leaf = name.rsplit(".", 1)[-1]
        if isinstance(mod, Linear) and ".layers." in name:
            if leaf in COLUMN:
                mod.tp, mod.tp_mode = tp, "column"
            elif leaf in ROW:
                mod.tp, mod.tp_mode = tp, "row"
    for name, p in model.named_parameters():
        leaf = name.rsplit(".", 1)[-1]
        owner = name.rsplit(".", 2)[-2] if name.count(".") else ""
        p.tp_sharded = (leaf == "weight" and owner in COLUMN + ROW and ".layers." in name) or leaf in SHARDED_VECTORS


def replicated_parameters(model) -> list:
    return [p for p in model.parameters() if not getattr(p, "tp_sharded", False)]


def _head_rows(n_heads: int, dim: int, rank: int, world: int, base: int = 0):
    per = n_heads // world
    return slice(base + rank * per * dim, base + (rank + 1) * per * dim)


def shard_state_dict(full: dict, cfg: ModelConfig, rank: int, world: int) -> dict:
    """One rank's slice of a full model's state dict."""
    enc = cfg.encoder
    a, g = enc.attention, enc.gdn
    nq, nv = g.n_k_heads * g.k_head_dim, g.n_v_heads * g.v_head_dim
    out = {}
    for name, t in full.items():
        leaf = name.rsplit(".", 1)[-1]
        owner = name.rsplit(".", 2)[-2] if name.count(".") else ""
        if ".layers." not in name:
            out[name] = t.clone()
            continue
        if owner == "in_proj_qkv" or leaf == "conv_weight":
            parts = [t[_head_rows(g.n_k_heads, g.k_head_dim, rank, world)], t[_head_rows(g.n_k_heads, g.k_head_dim, rank, world, nq)],
                     t[_head_rows(g.n_v_heads, g.v_head_dim, rank, world, 2 * nq)]]
            out[name] = torch.cat(parts, 0).clone()
        elif owner == "in_proj_z":
            out[name] = t[_head_rows(g.n_v_heads, g.v_head_dim, rank, world)].clone()
        elif owner in ("in_proj_a", "in_proj_b") or leaf in ("A_log", "dt_bias"):
            out[name] = t[_head_rows(g.n_v_heads, 1, rank, world)].clone()
        elif owner == "out_proj":
            out[name] = t[:, _head_rows(g.n_v_heads, g.v_head_dim, rank, world)].clone()
        elif owner == "q_proj":
            out[name] = t[_head_rows(a.n_q_heads, a.head_dim * (2 if a.gate == "elementwise" else 1), rank, world)].clone()
        elif owner == "g_proj" or leaf == "temp_w":
            out[name] = t[_head_rows(a.n_q_heads, 1, rank, world)].clone()
        elif owner in ("k_proj", "v_proj"):
            out[name] = t[_head_rows(a.n_kv_heads, a.head_dim, rank, world)].clone()
        elif owner == "o_proj":
            out[name] = t[:, _head_rows(a.n_q_heads, a.head_dim, rank, world)].clone()
        elif owner in ("w_gate", "w_up"):
            out[name] = t[_head_rows(cfg.ffn_hidden, 1, rank, world)].clone()
        elif owner == "w_down":
            out[name] = t[:, _head_rows(cfg.ffn_hidden, 1, rank, world)].clone()
        else:
            out[name] = t.clone()
    return out
