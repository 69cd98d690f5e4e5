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
    if enc.gdn_write_mix == "head":
        raise ValueError("tensor parallel is not built with model.encoder.gdn_write_mix 'head' (its lambdas are indexed by the full stack's heads)")
    if cfg.loop.pass2_gate != "none":
        raise ValueError("tensor parallel is not built with a gated second pass (model.loop.pass2_gate)")
    if enc.gdn_ccr_spacing:
        raise ValueError("tensor parallel is not built with the checkpoint cross-read (model.encoder.gdn_ccr_spacing)")
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


def _split_plan(name: str, cfg: ModelConfig):
    """How one named tensor of the full model is cut over ranks: (dim, [(units, unit width), ...]) — along `dim` the
    tensor is a concatenation of sections, each `units` equal pieces of `width` entries, and rank r owns pieces
    r*units/W .. (r+1)*units/W - 1 of every section — or None for a replicated tensor."""
    enc = cfg.encoder
    a, g = enc.attention, enc.gdn
    if ".layers." not in name:
        return None
    leaf = name.rsplit(".", 1)[-1]
    owner = name.rsplit(".", 2)[-2] if name.count(".") else ""
    if owner == "in_proj_qkv" or leaf == "conv_weight":
        return 0, [(g.n_k_heads, g.k_head_dim), (g.n_k_heads, g.k_head_dim), (g.n_v_heads, g.v_head_dim)]
    if owner == "in_proj_z":
        return 0, [(g.n_v_heads, g.v_head_dim)]
    if owner in ("in_proj_a", "in_proj_b") or leaf in ("A_log", "dt_bias"):
        return 0, [(g.n_v_heads, 1)]
    if owner == "out_proj":
        return 1, [(g.n_v_heads, g.v_head_dim)]
    if owner == "q_proj":
        return 0, [(a.n_q_heads, a.head_dim * (2 if a.gate == "elementwise" else 1))]
    if owner == "g_proj" or leaf == "temp_w":
        return 0, [(a.n_q_heads, 1)]
    if owner in ("k_proj", "v_proj"):
        return 0, [(a.n_kv_heads, a.head_dim)]
    if owner == "o_proj":
        return 1, [(a.n_q_heads, a.head_dim)]
    if owner in ("w_gate", "w_up"):
        return 0, [(cfg.ffn_hidden, 1)]
    if owner == "w_down":
        return 1, [(cfg.ffn_hidden, 1)]
    return None


def shard_tensor(name: str, t: torch.Tensor, cfg: ModelConfig, rank: int, world: int) -> torch.Tensor:
    plan = _split_plan(name, cfg)
    if plan is None:
        return t.clone()
    dim, sections = plan
    parts, base = [], 0
    for units, width in sections:
        per = units // world * width
        parts.append(t.narrow(dim, base + rank * per, per))
        base += units * width
    return torch.cat(parts, dim).clone()


def merge_tensor(name: str, shards: list, cfg: ModelConfig) -> torch.Tensor:
    """Inverse of `shard_tensor`: the full tensor from every rank's slice (replicated tensors: rank 0's)."""
    plan = _split_plan(name, cfg)
    if plan is None:
        return shards[0].clone()
    dim, sections = plan
    world = len(shards)
    out, base = [], 0
    for units, width in sections:
        per = units // world * width
        out.extend(s.narrow(dim, base, per) for s in shards)
        base += per
    return torch.cat(out, dim).clone()


def shard_state_dict(full: dict, cfg: ModelConfig, rank: int, world: int) -> dict:
    """One rank's slice of a full model's state dict (or of any by-name dict of tensors shaped like the parameters:
    gradients, optimizer moments)."""
    return {name: shard_tensor(name, t, cfg, rank, world) for name, t in full.items()}


def merge_state_dicts(shards: list[dict], cfg: ModelConfig) -> dict:
    """The full model's by-name dict from the ranks' dicts, rank order."""
    return {name: merge_tensor(name, [s[name] for s in shards], cfg) for name in shards[0]}


def init_full_then_shard(cfg: ModelConfig, local_cfg: ModelConfig, rank: int, world: int, seed: int, prepare=None):
    """This rank's model holding ITS slice of the full model's seeded start: every rank draws the full model from the
    same seed and keeps its cut, so the sharded run starts where the unsharded run with that seed does (ranks that
    each seeded a local model would all hold the same slice-shaped draw). `prepare(full_model)` runs on the full
    model before the cut (start-time rescalings)."""
    from ..models import build_model

    torch.manual_seed(seed)
    full = build_model(cfg)
    if prepare is not None:
        prepare(full)
    local = build_model(local_cfg)
    local.load_state_dict(shard_state_dict(full.state_dict(), cfg, rank, world))
    return local


def shard_optimizer_state(sd: dict, cfg: ModelConfig, rank: int, world: int) -> dict:
    """A full-model optimizer state (FlatAdamW.state_dict form: by-index state plus `names`) cut to one rank."""
    out = {**sd, "state": {}}
    for index, name in enumerate(sd["names"]):
        st = sd["state"].get(index)
        if st is not None:
            out["state"][index] = {"step": st["step"], "exp_avg": shard_tensor(name, st["exp_avg"], cfg, rank, world),
                                   "exp_avg_sq": shard_tensor(name, st["exp_avg_sq"], cfg, rank, world)}
    return out


def merge_optimizer_states(sds: list[dict], cfg: ModelConfig) -> dict:
    """The full-model optimizer state from the ranks' states, rank order."""
    out = {**sds[0], "state": {}}
    for index, name in enumerate(sds[0]["names"]):
        sts = [sd["state"].get(index) for sd in sds]
        if sts[0] is not None:
            out["state"][index] = {"step": sts[0]["step"], "exp_avg": merge_tensor(name, [s["exp_avg"] for s in sts], cfg),
                                   "exp_avg_sq": merge_tensor(name, [s["exp_avg_sq"] for s in sts], cfg)}
    return out
