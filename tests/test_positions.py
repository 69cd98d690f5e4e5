"""Span masks with an exact count, and the positions around scored spans."""

import pytest
import torch

from gdn_hybrid_architecture_ideas_b200.data.synthetic import counter_generator
from gdn_hybrid_architecture_ideas_b200.eval import span_bpb as S
from gdn_hybrid_architecture_ideas_b200.train import positions as P


def runs(mask):
    out, n = [], 0
    for x in mask.tolist() + [False]:
        if x:
            n += 1
        elif n:
            out.append(n)
            n = 0
    return out


@pytest.mark.parametrize("law", ["lognormal", "uniform"])
def test_span_mask_marks_exactly_the_count_in_spans_of_the_law(law):
    lengths = []
    for i in range(60):
        m = P.span_mask(2048, 512, counter_generator(3, i, 5), distribution=law, median=60.0, sigma=0.8, span_min=16, span_max=200)
        assert m.dtype == torch.bool and int(m.sum()) == 512
        r = runs(m)
        assert all(16 <= n < 200 + 16 for n in r[:-1]) and sum(r) == 512
        lengths += r
        assert torch.equal(m, P.span_mask(2048, 512, counter_generator(3, i, 5), distribution=law, median=60.0, sigma=0.8, span_min=16, span_max=200))
    lengths = sorted(lengths)
    if law == "lognormal":
        assert 35 <= lengths[len(lengths) // 2] <= 90                      # the median of the truncated law sits near the asked one
    assert torch.equal(P.span_mask(64, 64, counter_generator(0, 0, 5)), torch.ones(64, dtype=torch.bool)) and int(P.span_mask(64, 0, counter_generator(0, 0, 5)).sum()) == 0
    tight = P.span_mask(40, 38, counter_generator(1, 2, 5), span_min=4, span_max=10)    # no room to keep every pair of spans apart
    assert int(tight.sum()) == 38
    with pytest.raises(ValueError):
        P.span_mask(10, 11, counter_generator(0, 0, 5))
    draws = P.truncated_lognormal(counter_generator(5, 0, 0), 4000, 16, 4096, 230.0, 1.16)
    assert int(draws.min()) >= 16 and int(draws.max()) <= 4096 and 180 <= int(draws.median()) <= 290


def test_positions_around_scored_spans():
    docs = torch.tensor([[0, 0, 0, 0, 0, 1, 1, 1, 1, 1, 1, 2]])
    scored = torch.tensor([[0, 0, 0, 1, 1, 0, 0, 0, 1, 1, 0, 1]]).bool()
    within, first = P.document_positions(docs)
    assert within.tolist() == [[0, 1, 2, 3, 4, 0, 1, 2, 3, 4, 5, 0]] and first.tolist() == [[0] * 5 + [5] * 6 + [11]]
    assert P.sink_positions(docs, 2).tolist() == [[True, True, False, False, False, True, True, False, False, False, False, True]]
    assert P.span_starts(docs, scored).nonzero()[:, 1].tolist() == [3, 8, 11]
    assert P.replay_positions(docs, scored, 2).nonzero()[:, 1].tolist() == [1, 2, 6, 7]          # position 11 opens its document: nothing to replay
    assert P.replay_positions(docs, scored, 10).nonzero()[:, 1].tolist() == [0, 1, 2, 5, 6, 7]    # never outside the document


def test_span_rows_depend_on_the_seed_and_not_on_the_tokens():
    g = torch.Generator().manual_seed(0)
    mk = lambda seed: [S.TokenizedDoc(torch.randint(4, 60, (n,), generator=torch.Generator().manual_seed(seed + n)).tolist(), [1] * n) for n in (70, 90, 40)]
    a, b = S.build_span_rows(mk(0), 32, 12, seed=4, span_min=3, span_max=8, median=5.0), S.build_span_rows(mk(9), 32, 12, seed=4, span_min=3, span_max=8, median=5.0)
    plain = S.build_stream_rows(mk(0), 32)
    assert a.kind == "spans" and torch.equal(a.scored | ~plain.scored, b.scored | ~plain.scored)     # same marks wherever the target is valid
    assert all(int(a.scored[r].sum()) <= 12 for r in range(len(a))) and int(a.scored.sum()) > 0
    assert not torch.equal(a.scored, S.build_span_rows(mk(0), 32, 12, seed=5, span_min=3, span_max=8, median=5.0).scored)
