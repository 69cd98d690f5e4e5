"""qmix with a static top-2 query mix (`model.encoder.gdn_qmix_select_step` = S >= 1, under the write variant "qmix").

Until the start of optimizer step S every GDN layer's query mix m'_q is qmix's: the per-token softmax over all the finished
blocks. At the start of step S, once, every layer whose query mix reads more than two sources keeps the two with the
largest TOKEN-MEAN weight on the step's first micro-batch (float64 means of the per-token weights; ties go to the lower
source). The pair is written, ascending, into the layer's buffer `gdn_arms.qmix_keep` ((2,) int64, -1 before the choice; it
is part of the state dict, so a resume after S keeps the choice), and from then on m'_q is the per-token softmax over
those two sources' logits only: the others are neither read nor given weight or gradient. No parameter is added. A layer
with two sources or fewer keeps them all and has no buffer. Off (0): qmix as it is, bit for bit.

Reference: ced/model/gdn_arms.py:53-61 (the form), :377-401 (what it is refused with), :616-641 (buffer and post-load
hook), :1187-1261 (record, choice, log); ced/model/attn_res.py:500-540 (the pair mix and the weight sums).
"""

from __future__ import annotations

import torch

from .. import ops

KEEP = 2


def check_config(cfg) -> None:
    """cfg: ModelConfig. ValueError, by name, for a value that is not a non-negative int and for what the option is not built
    with: another write variant or write mix, MXFP8 / NVFP4 weights."""
    e = cfg.encoder
    s = e.gdn_qmix_select_step
    if isinstance(s, bool) or not isinstance(s, int) or s < 0:
        raise ValueError(f"model.encoder.gdn_qmix_select_step {s!r}: 0 (off) or the optimizer step >= 1 at whose start each layer's "
                         f"{KEEP} sources are chosen")
    if s == 0:
        return
    what = f"model.encoder.gdn_qmix_select_step {s!r}"
    if e.gdn_write_variant != "qmix" or e.gdn_write_mix != "layer":
        raise ValueError(f"{what} restricts the query mix of model.encoder.gdn_write_variant 'qmix' (with gdn_write_mix 'layer'), "
                         f"not {e.gdn_write_variant!r} / {e.gdn_write_mix!r}")
    if cfg.fp8.mode != "none" or cfg.nvfp4.mode != "none":
        raise ValueError(f"{what} is not built together with model.fp8 / model.nvfp4: nothing tests the pair")


def pair_sources(sources: list, keep: torch.Tensor) -> list:
    """The two sources `keep` names, gathered through the index buffer (a fixed shape: no host read, no mask); the gradient
    of the gather writes zeros to the sources left out."""
    dt = sources[0].dtype
    for s in sources[1:]:
        dt = torch.promote_types(dt, s.dtype)
    pair = torch.stack([s.to(dt) for s in sources]).index_select(0, keep)
    return [pair[0], pair[1]]


def depth_mix_pair(sources: list, reader, keep: torch.Tensor) -> torch.Tensor:
    """h = alpha_a v_a + alpha_b v_b with alpha the softmax of the two chosen sources' logits alone (the reader's
    pseudo-query and key norm), in the first source's dtype."""
    if getattr(reader, "heads", 1) != 1:
        raise ValueError("the static pair is built for a pseudo-query with one head")
    a, b = pair_sources(sources, keep)
    return ops.depth_mix([a, b], reader.query, reader.key_norm.weight, reader.key_norm.eps).to(sources[0].dtype)


def _weights(sources: list, reader) -> torch.Tensor:
    """(B, L, n) softmax weights of `reader` over `sources`, >= float32."""
    _, alpha = ops.ref.depth_mix(sources, reader.query, reader.key_norm.weight, reader.key_norm.eps, return_weights=True)
    return alpha


@torch.no_grad()
def depth_weight_sums(sources: list, reader, keep: torch.Tensor | None = None) -> tuple[torch.Tensor, int]:
    """(sum over the tokens of the reader's weights, (n,) float64; the number of tokens). keep None: the softmax over all n
    sources; else over the two it names, zero on the others. Each token's weights are formed in >= float32 and summed in
    float64."""
    srcs = [s.detach() for s in sources]
    if keep is None:
        sums = _weights(srcs, reader).double().sum(dim=(0, 1))
    else:
        alpha = _weights(pair_sources(srcs, keep), reader)
        sums = torch.zeros(len(srcs), dtype=torch.float64, device=alpha.device).index_copy(0, keep, alpha.double().sum(dim=(0, 1)))
    return sums, int(srcs[0].shape[0] * srcs[0].shape[1])


def record_query_weights(rec: dict, i: int, layer, sources: list | None) -> None:
    """Before layer i of a forward whose encoder has `qmix_record` set: rec[i] = (token-sums of the layer's query-mix
    weights as it is about to use them, tokens). A layer without a query mix of its own adds nothing."""
    arms = getattr(layer, "gdn_arms", None)
    if arms is None or arms.variant != "qmix" or arms.qmix_query is None or sources is None:
        return
    rec[i] = depth_weight_sums(sources, arms.qmix_query, arms.qmix_keep if arms.qmix_static else None)


def read_query_weights(rec: dict) -> dict:
    """{layer: (token-mean weights as Python floats, tokens)}: the sums over the tokens, divided in float64; one host read."""
    if not rec:
        return {}
    layers = sorted(rec)
    flat = torch.cat([rec[i][0] for i in layers]).cpu()
    out, at = {}, 0
    for i in layers:
        sums, tokens = rec[i]
        out[i] = ((flat[at:at + sums.numel()] / tokens).tolist(), tokens)
        at += sums.numel()
    return out


def _arms(encoder):
    return [(i, getattr(layer, "gdn_arms", None)) for i, layer in enumerate(encoder.layers)]


def sync_static(encoder) -> None:
    """After tensors were copied into the model's buffers without `load_state_dict` (a trainer's resume): every layer's
    form follows its buffer, as the post-load hook would set it."""
    from .gdn import _sync_qmix_static

    for _, arms in _arms(encoder):
        if arms is not None and hasattr(arms, "qmix_keep"):
            _sync_qmix_static(arms, None)


def pending(encoder) -> bool:
    """Whether a layer has the buffer and has not chosen yet."""
    return any(a is not None and hasattr(a, "qmix_keep") and not a.qmix_static for _, a in _arms(encoder))


@torch.no_grad()
def select_pairs(encoder, rec: dict) -> dict:
    """The choice: every layer with the buffer that has not chosen takes the KEEP sources with the largest token-mean weight
    in `rec` (a record of the full softmax), ties to the lower index, written ascending into its buffer. Returns
    {layer: {"pair", "weights" (every source's token-mean), "tokens"}} for the layers chosen now, in stack order."""
    means = read_query_weights(rec)
    out = {}
    for i, arms in _arms(encoder):
        if arms is None or not hasattr(arms, "qmix_keep") or arms.qmix_static:
            continue
        if i not in means:
            raise ValueError(f"layer {i} has no recorded query-mix weights: the choice follows a forward with encoder.qmix_record set")
        w, tokens = means[i]
        if len(w) != arms.n_sources:
            raise ValueError(f"layer {i}: {len(w)} recorded weights for its {arms.n_sources} sources")
        pair = sorted(sorted(range(len(w)), key=lambda s: (-w[s], s))[:KEEP])
        arms.qmix_keep.copy_(torch.tensor(pair, dtype=torch.long, device=arms.qmix_keep.device))
        arms.qmix_static = True
        out[i] = {"pair": pair, "weights": w, "tokens": tokens}
    return out


def weights_metrics(encoder, rec: dict) -> dict:
    """The log of a recorded forward: layers, their source counts, every source's token-mean weight as the layer used it
    (after the choice: the pair's, zero on the others), the tokens, and each layer's pair (None before the choice)."""
    means = read_query_weights(rec)
    layers = sorted(means)
    chosen = []
    for i in layers:
        arms = encoder.layers[i].gdn_arms
        chosen.append(arms.chosen_sources() if hasattr(arms, "qmix_keep") else None)
    return {"layers": layers, "n_sources": [len(means[i][0]) for i in layers],
            "weights": [[round(x, 8) for x in means[i][0]] for i in layers],
            "tokens": means[layers[0]][1] if layers else 0, "chosen": chosen}


def choose(encoder, forward) -> dict:
    """Runs `forward()` (the training forward of the step's first micro-batch; its result is discarded) with the encoder's
    record set, then makes the choice. Returns the log record {"layers", "pair", "weights", "tokens"}."""
    encoder.qmix_record = {}
    try:
        forward()
    finally:
        rec, encoder.qmix_record = encoder.qmix_record, None
    chosen = select_pairs(encoder, rec)
    layers = list(chosen)
    return {"layers": layers, "pair": [chosen[i]["pair"] for i in layers], "weights": [chosen[i]["weights"] for i in layers],
            "tokens": chosen[layers[0]]["tokens"] if layers else 0}
