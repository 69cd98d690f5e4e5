"""Wiring of the block-scaled low-precision recipes onto a built model (reference: ced/model/fp8.py:544-600,
ced/model/nvfp4.py:664-757). Which linears are quantised: every projection of mixers and FFNs whose two dimensions
are multiples of 16/32, except in_proj_a / in_proj_b (kept high precision); embeddings and the head never."""

from __future__ import annotations

from .linear import Linear

KEPT_SUFFIXES = ("in_proj_a", "in_proj_b", ".kda.f_down", ".kda.f_up", ".erase.e_down", ".erase.e_up", ".erase.in_proj_gamma")


def quantised_linears(model, mode: str, align: int):
    """(name, module) of the linears a recipe quantises under `mode`."""
    for name, m in model.named_modules():
        if not isinstance(m, Linear) or ".mixer." not in name and ".mlp." not in name:
            continue
        if name.endswith(KEPT_SUFFIXES) or m.in_features % align or m.out_features % align:
            continue
        layer = model.encoder.layers[int(name.split(".")[2])]
        in_gdn = layer.kind == "gdn" and ".mixer." in name
        in_mixer = ".mixer." in name
        if mode == "mlp_only" and in_mixer:
            continue
        if mode == "all_but_gdn_mixer" and in_gdn:
            continue
        if mode == "all_but_gdn" and layer.kind == "gdn":
            continue
        yield name, m


def apply_low_precision(model, cfg) -> list[str]:
    done = []
    if cfg.fp8.mode == "none" and cfg.nvfp4.mode == "none":
        return done
    from ..ops import lowp

    if cfg.fp8.mode == "linears":
        for name, m in quantised_linears(model, "all_linears", 32 if cfg.fp8.scaling == "mxfp8" else 16):
            m.precision, m.lowp = cfg.fp8.scaling if cfg.fp8.scaling == "mxfp8" else "fp8_" + cfg.fp8.scaling, lowp.recipe_for(cfg, name)
            done.append(name)
    elif cfg.nvfp4.mode != "none":
        nv = cfg.nvfp4
        if nv.recipe == "quartet2" and (not nv.stochastic_rounding or not nv.rht or not nv.weight_2d):
            raise ValueError("model.nvfp4.recipe 'quartet2' has its own roundings and transform: stochastic_rounding, rht and weight_2d are the "
                             "'nvidia' recipe's switches and keep their defaults under it")
        names = list(quantised_linears(model, cfg.nvfp4.mode, 16))
        keep_last = int(round(cfg.nvfp4.keep_last_fraction * cfg.encoder.n_layers))
        for name, m in names:
            li = int(name.split(".")[2])
            if li < cfg.nvfp4.keep_first_layers or li >= cfg.encoder.n_layers - keep_last:
                continue
            if any(name.endswith(k) or k in name for k in cfg.nvfp4.keep_names):
                continue
            m.precision, m.lowp = "nvfp4", lowp.recipe_for(cfg, name)
            done.append(name)
    return done
