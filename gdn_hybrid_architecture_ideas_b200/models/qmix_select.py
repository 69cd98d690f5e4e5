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
_KEY = "model.encoder.gdn_qmix_select_step"


def check_config(cfg) -> None:
    """cfg: ModelConfig. ValueError, by name, for a value that is not a non-negative int and for what the option is not built
    with: another write variant or write mix, MXFP8 / NVFP4 weights."""
    enc = cfg.encoder
    step = enc.gdn_qmix_select_step
    if type(step) is not int or step < 0:
        raise ValueError(f"{_KEY} {step!r}: 0 (off) or the optimizer step >= 1 at whose start each layer's {KEEP} sources are chosen")
    if step == 0:
        return
    if (enc.gdn_write_variant, enc.gdn_write_mix) != ("qmix", "layer"):
        raise ValueError(f"{_KEY} {step!r} restricts the query mix of model.encoder.gdn_write_variant 'qmix' (with gdn_write_mix 'layer'), "
                         f"not {enc.gdn_write_variant!r} / {enc.gdn_write_mix!r}")
    if "none" != cfg.fp8.mode or "none" != cfg.nvfp4.mode:
        raise ValueError(f"{_KEY} {step!r} is not built together with model.fp8 / model.nvfp4: nothing tests the pair")


def pair_sources(sources: list, keep: torch.Tensor) -> list:
    """The two sources `keep` names, gathered through the index buffer (a fixed shape: no host read, no mask); the gradient
    of the gather writes zeros to the sources left out."""
    wide = sources[0].dtype
    for other in sources[1:]:
        wide = torch.promote_types(wide, other.dtype)
    first, second = torch.stack([t.to(wide) for t in sources], dim=0).index_select(0, keep).unbind(0)
    return [first, second]


def depth_mix_pair(sources: list, reader, keep: torch.Tensor) -> torch.Tensor:
    """h = alpha_a v_a + alpha_b v_b with alpha the softmax of the two chosen sources' logits alone (the reader's
    pseudo-query and key norm), in the first source's dtype."""
    if getattr(reader, "heads", 1) != 1:
        raise ValueError("the static pair is built for a pseudo-query with one head")
    mixed = ops.depth_mix(pair_sources(sources, keep), reader.query, reader.key_norm.weight, reader.key_norm.eps)
    return mixed.to(sources[0].dtype)


def _token_weight_sums(sources: list, reader) -> torch.Tensor:
    """(n,) float64: the reader's softmax weights over `sources` (formed in >= float32), summed over every token."""
    weights = ops.ref.depth_mix(sources, reader.query, reader.key_norm.weight, reader.key_norm.eps, return_weights=True)[1]
    return weights.to(torch.float64).flatten(0, -2).sum(0)


@torch.no_grad()
def depth_weight_sums(sources: list, reader, keep: torch.Tensor | None = None) -> tuple[torch.Tensor, int]:
    """(sum over the tokens of the reader's weights, (n,) float64; the number of tokens). keep None: the softmax over all n
    sources; else over the two it names, zero on the others."""
    held = [t.detach() for t in sources]
    tokens = held[0].shape[0] * held[0].shape[1]
    if keep is not None:
        two = _token_weight_sums(pair_sources(held, keep), reader)
        return torch.zeros(len(held), dtype=two.dtype, device=two.device).index_copy(0, keep, two), int(tokens)
    return _token_weight_sums(held, reader), int(tokens)


def _query_mix_of(layer):
    """The layer's arms when it has a query mix of its own under the qmix variant, else None."""
    arms = getattr(layer, "gdn_arms", None)
    return arms if arms is not None and arms.variant == "qmix" and arms.qmix_query is not None else None


def record_query_weights(rec: dict, i: int, layer, sources: list | None) -> None:
    """Before layer i of a forward whose encoder has `qmix_record` set: rec[i] = (token-sums of the layer's query-mix
    weights as it is about to use them, tokens). A layer without a query mix of its own adds nothing."""
    arms = _query_mix_of(layer)
    if arms is not None and sources is not None:
        rec[i] = depth_weight_sums(sources, arms.qmix_query, arms.qmix_keep if arms.qmix_static else None)


def read_query_weights(rec: dict) -> dict:
    """{layer: (token-mean weights as Python floats, tokens)}: the sums over the tokens, divided in float64; one host read."""
    order = sorted(rec)
    if not order:
        return {}
    host = torch.cat([rec[i][0] / rec[i][1] for i in order]).tolist()          # float64 sums / int tokens, one copy to the host
    sizes = [rec[i][0].numel() for i in order]
    starts = [sum(sizes[:k]) for k in range(len(order))]
    return {i: (host[a:a + n], rec[i][1]) for i, a, n in zip(order, starts, sizes)}


def _waiting(encoder):
    """(index, arms) of the layers that hold the buffer and have not chosen, in stack order."""
    for i, layer in enumerate(encoder.layers):
        arms = getattr(layer, "gdn_arms", None)
        if arms is not None and hasattr(arms, "qmix_keep") and not arms.qmix_static:
            yield i, arms


def sync_static(encoder) -> None:
    """After tensors were copied into the model's buffers without `load_state_dict` (a trainer's resume): every layer's
    form follows its buffer, as the post-load hook would set it."""
    from .gdn import _sync_qmix_static

    for layer in encoder.layers:
        arms = getattr(layer, "gdn_arms", None)
        if arms is not None and hasattr(arms, "qmix_keep"):
            _sync_qmix_static(arms, None)


def pending(encoder) -> bool:
    """Whether a layer has the buffer and has not chosen yet."""
    return next(_waiting(encoder), None) is not None


def top_pair(weights: list) -> list:
    """The KEEP largest entries' indices, ties to the lower index, ascending."""
    ranked = sorted(range(len(weights)), key=lambda j: (-weights[j], j))
    return sorted(ranked[:KEEP])


@torch.no_grad()
def select_pairs(encoder, rec: dict) -> dict:
    """The choice: every layer with the buffer that has not chosen takes the KEEP sources with the largest token-mean weight
    in `rec` (a record of the full softmax), ties to the lower index, written ascending into its buffer. Returns
    {layer: {"pair", "weights" (every source's token-mean), "tokens"}} for the layers chosen now, in stack order."""
    means, chosen = read_query_weights(rec), {}
    for i, arms in list(_waiting(encoder)):
        if i not in means:
            raise ValueError(f"layer {i} has no recorded query-mix weights: the choice follows a forward with encoder.qmix_record set")
        weights, tokens = means[i]
        if len(weights) != arms.n_sources:
            raise ValueError(f"layer {i}: {len(weights)} recorded weights for its {arms.n_sources} sources")
        pair = top_pair(weights)
        arms.qmix_keep.copy_(torch.as_tensor(pair, dtype=arms.qmix_keep.dtype, device=arms.qmix_keep.device))
        arms.qmix_static = True
        chosen[i] = dict(pair=pair, weights=weights, tokens=tokens)
    return chosen


def weights_metrics(encoder, rec: dict) -> dict:
    """The log of a recorded forward: layers, their source counts, every source's token-mean weight as the layer used it
    (after the choice: the pair's, zero on the others), the tokens, and each layer's pair (None before the choice)."""
    means = read_query_weights(rec)
    rows = sorted(means.items())
    pairs = [encoder.layers[i].gdn_arms.chosen_sources() if hasattr(encoder.layers[i].gdn_arms, "qmix_keep") else None for i, _ in rows]
    return dict(layers=[i for i, _ in rows], n_sources=[len(w) for _, (w, _) in rows], weights=[[round(x, 8) for x in w] for _, (w, _) in rows],
                tokens=rows[0][1][1] if rows else 0, chosen=pairs)


def choose(encoder, forward) -> dict:
    """Runs `forward()` (the training forward of the step's first micro-batch; its result is discarded) with the encoder's
    record set, then makes the choice. Returns the log record {"layers", "pair", "weights", "tokens"}."""
    encoder.qmix_record = {}
    try:
        forward()
    finally:
        rec, encoder.qmix_record = encoder.qmix_record, None
    picked = select_pairs(encoder, rec)
    order = sorted(picked)
    return dict(layers=order, pair=[picked[i]["pair"] for i in order], weights=[picked[i]["weights"] for i in order],
                tokens=picked[order[0]]["tokens"] if order else 0)
