"""Fixed-capacity decoder slots of the looped encoder-decoder and its decoder-position spans."""

import math

import pytest
import torch
from torch.utils._python_dispatch import TorchDispatchMode

from gdn_hybrid_architecture_ideas_b200 import config as C
from gdn_hybrid_architecture_ideas_b200.data.spans import sample_spans, span_lengths
from gdn_hybrid_architecture_ideas_b200.models import build_model
from gdn_hybrid_architecture_ideas_b200.models.looped_decoder import decoder_capacity, select_slots, two_head_loss


def test_capacity_rule():
    assert decoder_capacity(64, 0.25, 8) == 16 and decoder_capacity(64, 0.26, 8) == 24 and decoder_capacity(8192, 0.25, 128) == 2048
    assert decoder_capacity(10, 0.9, 128) == 10 and decoder_capacity(1, 0.25, 128) == 1


def test_the_first_decoder_positions_take_the_slots_in_order():
    g = torch.Generator().manual_seed(0)
    mask = torch.rand(5, 37, generator=g) < 0.4
    mask[3] = False
    mask[4] = True
    C_ = 9
    s = select_slots(mask, C_)
    for b in range(5):
        where = mask[b].nonzero().flatten().tolist()
        want = where[:C_] + [37] * (C_ - len(where[:C_]))
        assert s.index[b].tolist() == want and s.valid[b].tolist() == [i < len(where) for i in range(C_)]
        assert s.kept[b].nonzero().flatten().tolist() == where[:C_] and int(s.n_dropped[b]) == max(0, len(where) - C_)
        assert [int(s.inverse[b, t]) for t in where[:C_]] == list(range(len(where[:C_]))) and (s.inverse[b][~s.kept[b]] == C_).all()
    x = torch.randn(5, 37, 3, generator=g)
    taken = s.take(x, fill=7.0)
    assert torch.equal(taken[0, 0], x[0, s.index[0, 0]]) and (taken[3] == 7.0).all()
    back = s.put(torch.zeros_like(x), s.take(x))
    assert torch.equal(back, x * s.kept[..., None])


def test_selection_is_prefix_stable():
    """Whether position t runs the decoder depends on dec_mask[: t + 1] alone."""
    g = torch.Generator().manual_seed(1)
    mask = torch.rand(3, 50, generator=g) < 0.5
    full = select_slots(mask, 12).kept
    for cut in (1, 10, 25, 49):
        assert torch.equal(select_slots(mask[:, :cut], 12).kept, full[:, :cut])


class _Ops(TorchDispatchMode):
    def __init__(self):
        super().__init__()
        self.names = set()

    def __torch_dispatch__(self, func, types, args=(), kwargs=None):
        self.names.add(func.__name__)
        return func(*args, **(kwargs or {}))


def test_a_training_forward_and_backward_run_no_data_dependent_shape():
    """No nonzero, masked select or boolean-index op: every shape is a function of (B, L, C)."""
    torch.manual_seed(0)
    cfg = C.tiny_looped_config()
    cfg.encoder.gdn.kernel = cfg.decoder.gdn.kernel = "chunked"
    model = build_model(cfg)
    tok = torch.randint(0, cfg.vocab_size, (2, 32))
    doc = (torch.arange(32) >= 20).long().expand(2, 32)
    dm = torch.rand(2, 32) < 0.3
    with _Ops() as seen:
        out = model(tok, doc, dm, T=2, return_hidden=True)
        loss, _ = two_head_loss(model, out, torch.roll(tok, -1, 1), torch.ones_like(dm), 64.0, 16.0, 48.0, z_loss=1e-4)
        loss.backward()
    banned = {n for n in seen.names if any(b in n for b in ("nonzero", "masked_select", "index.Tensor", "unique", "_local_scalar_dense"))}
    assert not banned, banned
    assert math.isfinite(float(loss))


def test_spans_cover_exactly_the_capacity_and_depend_on_the_generator_alone():
    for seed in range(40):
        g = torch.Generator().manual_seed(seed)
        m = sample_spans(256, 64, g, median=20.0, span_min=4, span_max=48)
        assert m.dtype == torch.bool and int(m.sum()) == 64
        runs = (m[1:] & ~m[:-1]).sum() + int(m[0])
        lengths = span_lengths(64, torch.Generator().manual_seed(seed), "lognormal", 20.0, 1.16, 4, 48)
        assert int(runs) == len(lengths) and sum(lengths) == 64 and min(lengths) >= 4 and max(lengths) < 48 + 4
    assert torch.equal(sample_spans(64, 16, torch.Generator().manual_seed(5)), sample_spans(64, 16, torch.Generator().manual_seed(5)))
    assert int(sample_spans(32, 32, torch.Generator().manual_seed(0)).sum()) == 32 and int(sample_spans(32, 0, torch.Generator().manual_seed(0)).sum()) == 0
    with pytest.raises(ValueError, match="span_distribution"):
        sample_spans(32, 8, torch.Generator().manual_seed(0), distribution="normal")


def test_spans_equal_the_reference_draw_for_draw(reference):
    from ced.train.data import sample_spans as theirs

    for seed in range(60):
        for L, n, kw in ((64, 16, dict(median=5.0, span_min=2, span_max=12)), (200, 50, {}), (40, 39, dict(distribution="uniform", span_min=3, span_max=9))):
            assert torch.equal(sample_spans(L, n, torch.Generator().manual_seed(seed), **kw), theirs(L, n, torch.Generator().manual_seed(seed), **kw))


def test_the_probe_scorer_runs_the_looped_model_with_the_answer_at_decoder_positions():
    """Stored probes score a looped encoder-decoder: the answer's positions run the decoder, every slot kept; the numbers are
    those of the model's own forward on the same mask."""
    from gdn_hybrid_architecture_ideas_b200.eval import probes

    torch.manual_seed(0)
    cfg = C.tiny_looped_config()
    model = build_model(cfg).eval()
    items = [probes.build_probe(kind, cfg.vocab_size, 48, 0, i) for kind in ("needle", "copy") for i in range(2)]
    res = probes.score_probes(model, items, batch_size=4, passes=2)
    assert res["n"] == 4 and all(math.isfinite(it["ce"]) for it in res["items"])
    p = items[0]
    ids = torch.tensor(p.ids)[None]
    dec = torch.zeros(1, len(p.ids) - 1, dtype=torch.bool)
    dec[0, p.answer_start - 1: p.answer_start - 1 + p.answer_len] = True
    with torch.no_grad():
        logits = model(ids[:, :-1], torch.zeros_like(ids[:, :-1]), dec, T=2, capacity=dec.shape[1]).logits
    sl = slice(p.answer_start - 1, p.answer_start - 1 + p.answer_len)
    ce = torch.nn.functional.cross_entropy(logits[0, sl].float(), ids[0, 1:][sl])
    assert abs(float(ce) - res["items"][0]["ce"]) < 1e-4
    with pytest.raises(ValueError, match="arch"):
        from gdn_hybrid_architecture_ideas_b200.infer.engine import DecodeEngine

        DecodeEngine(model, 1, 64, device="cpu", use_graph=False)


def test_loopspec_emits_the_greedy_tokens_of_two_passes():
    """Speculative decoding from the first pass: exactly `generate` at T = 2 whatever the acceptance; a model whose draft head
    is its decoder head after an identity second pass accepts everything; the statistics count steps and accepts."""
    from gdn_hybrid_architecture_ideas_b200.infer.loopspec import LoopSpec

    torch.manual_seed(0)
    cfg = C.tiny_looped_config()
    model = build_model(cfg).double().eval()
    g = torch.Generator().manual_seed(2)
    with torch.no_grad():
        for p in model.parameters():
            p.add_(torch.randn(p.shape, generator=g, dtype=p.dtype) * 0.05)
    prompt = torch.randint(0, cfg.vocab_size, (1, 14), generator=g)
    doc, dec = torch.zeros_like(prompt), torch.zeros_like(prompt, dtype=torch.bool)
    dec[0, 9:] = True
    want, _ = model.generate(prompt, doc, dec, 12, T=2)
    got, stats = LoopSpec(model).generate(prompt, doc, dec, 12)
    assert got == want[0].tolist() and stats.steps == 11 and stats.accepted == sum(stats.flags) and 0 <= stats.acceptance <= 1
    assert LoopSpec(model).generate(prompt, doc, dec, 1)[0] == want[0, :1].tolist()
    with torch.no_grad():                    # the draft norm equal to the decoder norm and a second pass that changes nothing: every draft is right
        model.readout_norms[0].weight.copy_(model.decoder_norm.weight)
        for layer in model.decoder_layers:
            layer.residual_scale = 0.0
        model.injection.A_log.fill_(-30.0)               # decay 1: the injection passes the state through
        model.injection.B.zero_()
        model.loop_embedding.zero_()
    same, stats = LoopSpec(model).generate(prompt, doc, dec, 8)
    assert same == model.generate(prompt, doc, dec, 8, T=2)[0][0].tolist() and stats.acceptance == 1.0
    bad = C.tiny_looped_config()
    bad.loop.depth_attention, bad.loop.depth_attention_head_dim = "layer", 8
    with pytest.raises(ValueError, match="depth_attention"):
        LoopSpec(build_model(bad))
