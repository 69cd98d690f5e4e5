"""Row packings, strata and standard errors of the bits-per-byte evaluator."""

import math

import pytest
import torch

from gdn_hybrid_architecture_ideas_b200 import config as C
from gdn_hybrid_architecture_ideas_b200.eval import span_bpb as S
from gdn_hybrid_architecture_ideas_b200.models import build_model


def make_docs(lengths, seed=0, vocab=60):
    g = torch.Generator().manual_seed(seed)
    return [S.TokenizedDoc(torch.randint(4, vocab, (n,), generator=g).tolist(), torch.randint(1, 5, (n,), generator=g).tolist()) for n in lengths]


@pytest.fixture(scope="module")
def model():
    torch.manual_seed(0)
    return build_model(C.tiny_full_config()).eval()


def test_stream_rows_score_every_target_of_every_document_once():
    docs = make_docs([5, 40, 3, 17, 64])
    rows = S.build_stream_rows(docs, 16)
    total = sum(len(d.ids) for d in docs)
    assert len(rows) == math.ceil((total - 1) / 16) and rows.kind == "stream" and not rows.skipped
    # a document of n tokens has n - 1 in-document targets and a row boundary loses none of them (rows overlap by one token)
    per_doc = torch.zeros(len(docs), dtype=torch.long).index_add_(0, rows.doc_index[rows.scored], torch.ones(int(rows.scored.sum()), dtype=torch.long))
    assert all(int(per_doc[i]) == len(d.ids) - 1 for i, d in enumerate(docs)), per_doc.tolist()
    flat_targets = rows.targets[rows.scored].tolist()
    want = [t for d in docs for t in d.ids[1:]]
    assert flat_targets == want
    assert int((rows.target_bytes * rows.scored).sum()) == sum(sum(d.byte_lens[1:]) for d in docs)
    # document ids restart at zero in every row and grow along it; padding is the last document
    assert bool((rows.doc_ids[:, 0] == 0).all()) and bool((rows.doc_ids[:, 1:] >= rows.doc_ids[:, :-1]).all())


def test_role_rows_score_assistant_tokens_and_whole_rows_cut_no_document():
    g = torch.Generator().manual_seed(1)
    docs = []
    for n in (12, 9, 20, 7):
        ids = torch.randint(4, 60, (n,), generator=g).tolist()
        asst = [int(i >= n // 2) for i in range(n)]
        docs.append(S.RoleDoc(ids, [1] * n, None, "", assistant=asst, token_class=[i % 3 for i in range(n)]))
    stream = S.build_role_rows(docs, 16)
    assert stream.kind == "roles" and int(stream.scored.sum()) == sum(sum(d.assistant[1:]) for d in docs)
    whole = S.build_role_rows(docs, 24, whole=True)
    for r in range(len(whole)):
        present = set(whole.doc_index[r][whole.doc_index[r] >= 0].tolist())
        for i in present:               # a document that appears in a row appears there in full
            assert int((whole.doc_index[r] == i).sum()) >= len(docs[i].ids) - 1
    assert int(whole.scored.sum()) == int(stream.scored.sum())
    assert whole.target_class is not None and int(whole.target_class[~whole.scored].sum()) == 0
    capped = S.build_role_rows(docs, 24, whole=True, max_scored=8)
    assert len(capped) > len(whole) and all(int(capped.scored[r].sum()) <= 10 for r in range(len(capped)))
    with pytest.raises(ValueError, match="more than a row"):
        S.build_role_rows(docs, 12, whole=True)
    empty = S.EvalRows(*(getattr(whole, f) for f in S.EvalRows._TENSORS), n_docs=whole.n_docs)
    empty.scored = empty.scored.clone()
    empty.scored[0] = False
    assert len(S.drop_unscored_rows(empty)) == len(whole) - 1


def test_rows_persist_with_a_fingerprint(tmp_path):
    rows = S.build_stream_rows(make_docs([30, 30, 30]), 16)
    rows.doc_group = torch.tensor([0, 0, 1])
    rows.save(tmp_path / "rows.pt")
    back = S.EvalRows.load(tmp_path / "rows.pt")
    assert back.fingerprint() == rows.fingerprint() and torch.equal(back.doc_group, rows.doc_group) and back.kind == "stream"
    assert rows[1:3].fingerprint() != rows.fingerprint() and len(rows[1:3]) == 2
    blob = torch.load(tmp_path / "rows.pt", weights_only=False)
    blob["targets"][0, 0] += 1
    torch.save(blob, tmp_path / "bad.pt")
    with pytest.raises(ValueError, match="fingerprint"):
        S.EvalRows.load(tmp_path / "bad.pt")


def test_strata_special_bytes_clusters_and_joining(model):
    g = torch.Generator().manual_seed(2)
    docs = []
    for n in (40, 25, 33, 18, 29, 41):
        ids = torch.randint(4, 60, (n,), generator=g).tolist()
        docs.append(S.RoleDoc(ids, [2] * n, None, "", assistant=[1] * n, token_class=[(i // 5) % 3 for i in range(n)]))
    rows = S.build_role_rows(docs, 16)
    rows.special_ids = torch.tensor([4, 5, 6])
    rows.doc_group = torch.tensor([0, 0, 1, 1, 2, 2])
    ev = S.evaluate(model, rows, 3)
    # strata add up to the whole
    assert torch.allclose(ev.class_nats.sum(), ev.row_nats.sum()) and float(ev.class_bytes.sum()) == float(ev.row_bytes.sum())
    strata = ev.class_bpb()
    assert set(strata) == {0, 1, 2} and sum(v["tokens"] for v in strata.values()) == int(rows.scored.sum())
    assert ev.bpb_without_special_bytes() >= ev.bpb and float(ev.row_special_bytes.sum()) == 2.0 * int((torch.isin(rows.targets, rows.special_ids) & rows.scored).sum())
    # clusters: rows of one group are one unit, so there are three units and the standard error differs from the per-row one
    assert set(ev.clusters.tolist()) == {0, 1, 2}
    se_rows, se_cl, se_doc = S.bpb_se(ev, "row"), S.bpb_se(ev, "cluster"), S.bpb_se(ev, "doc")
    assert all(x == x and x > 0 for x in (se_rows, se_cl, se_doc)) and se_cl != se_rows
    # sharded scoring joins to the same record, through its dict form too
    a = S.evaluate(model, rows, 2, row_indices=list(range(0, len(rows), 2)))
    b = S.evaluate(model, rows, 2, row_indices=list(range(1, len(rows), 2)))
    joined = S.join_batches([a, S.SpanEval.from_dict(b.to_dict())])
    for f in ("row_nats", "row_bytes", "doc_nats", "class_nats", "row_special_bytes"):
        assert torch.allclose(getattr(joined, f), getattr(ev, f)), f
    assert torch.equal(joined.clusters, ev.clusters)


def test_stream_and_document_packings_agree_where_nothing_is_cut(model):
    docs = make_docs([15, 15, 15, 15], seed=3)         # n - 1 = 14 targets each; rows of 15 hold one document's 14 targets + 1
    by_doc = S.evaluate(model, S.build_eval_rows(docs, 14), 4)
    by_stream = S.evaluate(model, S.build_stream_rows(docs, 15), 4)
    assert torch.allclose(by_doc.doc_nats, by_stream.doc_nats, atol=1e-5) and torch.equal(by_doc.doc_bytes, by_stream.doc_bytes)


def test_set_size_from_a_pilot():
    pilot = S.PairedDifference(0.01, 0.004, 100)
    assert S.eval_set_size(pilot, 0.002) == 400 and S.eval_set_size(pilot, 0.004) == 100
    with pytest.raises(ValueError):
        S.eval_set_size(S.PairedDifference(0.0, float("nan"), 1), 0.01)
