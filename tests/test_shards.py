"""Shard sets: both on-disk layouts read through one interface, unions with concatenated side arrays, the per-token
loss mask (assistant flags and loss-span classes) reaches the loss, and its invariants are checked when a set is opened."""

import json

import numpy as np
import pytest
import torch

from gdn_hybrid_architecture_ideas_b200 import config as C
from gdn_hybrid_architecture_ideas_b200.data import shard_format as SF
from gdn_hybrid_architecture_ideas_b200.data.shards import ShardPacker


def _docs(seed=0, n=12, vocab=200):
    g = np.random.default_rng(seed)
    out = []
    for i in range(n):
        L = int(g.integers(20, 60))
        ids = g.integers(0, vocab, L)
        chat = i % 2 == 0
        gen = np.zeros(L, dtype=np.uint8)
        spans = np.zeros(L, dtype=np.uint8)
        if chat:
            gen[max(L // 2, 14):] = 1
            spans[2:6] = 3
            spans[6:10] = 2
            spans[10:14] = 1
        out.append((ids, gen, spans, chat))
    return out


def _write_own(path, docs, vocab=200):
    with SF.ShardWriter(path, vocab) as w:
        for ids, gen, spans, chat in docs:
            w.add_document(ids, n_bytes=3 * len(ids), generated=gen, loss_spans=spans, chat=chat)
    return SF.open_shards([path])


def test_side_arrays_round_trip_and_union(tmp_path):
    a, b = _docs(0), _docs(1, n=5)
    sa, sb = _write_own(tmp_path / "a", a), _write_own(tmp_path / "b", b)
    assert len(sa) == 12 and sa.side("generated") is not None
    for i, (ids, gen, spans, chat) in enumerate(a):
        lo, hi = int(sa.starts[i]), int(sa.ends[i])
        assert np.array_equal(sa.doc(i), ids) and np.array_equal(sa.side("generated")[lo:hi], gen)
        assert np.array_equal(sa.side("loss_spans")[lo:hi], spans) and bool(sa.doc_chat[i]) == chat
    u = SF.open_shards([tmp_path / "a", tmp_path / "b"])
    assert len(u) == 17 and u.n_tokens == sa.n_tokens + sb.n_tokens
    whole = np.concatenate([np.asarray(sa.side("loss_spans")), np.asarray(sb.side("loss_spans"))])
    view = u.side("loss_spans")
    assert np.array_equal(view[:], whole) and view[sa.n_tokens - 3: sa.n_tokens + 4].tolist() == whole[sa.n_tokens - 3: sa.n_tokens + 4].tolist()
    assert int(view[sa.n_tokens]) == int(whole[sa.n_tokens]) and int(view[-1]) == int(whole[-1])
    lo = int(u.starts[12])
    assert np.array_equal(u.doc(12), b[0][0]) and np.array_equal(view[lo:lo + len(b[0][0])], b[0][2])


def test_writer_refuses_what_a_mask_cannot_rely_on(tmp_path):
    w = SF.ShardWriter(tmp_path / "x", 50)
    ids = np.arange(10)
    with pytest.raises(ValueError, match="chat"):
        w.add_document(ids, loss_spans=np.array([0, 1] * 5), chat=False)
    with pytest.raises(ValueError, match="generated token"):
        w.add_document(ids, generated=np.ones(10, dtype=np.uint8), loss_spans=np.full(10, 3), chat=True)


@pytest.mark.parametrize("mode", ["assistant", "spans_full", "spans_head_tail", "spans_mask"])
def test_loss_mask_reaches_rows_and_loss(tmp_path, mode):
    docs = _docs(2, n=30)
    shards = _write_own(tmp_path / "s", docs)
    dcfg = C.DataConfig(kind="shards", shard_dir=str(tmp_path / "s"), seq_len=32, batch_size=3, seed=5, loss_mask=mode)
    packer = ShardPacker(shards, dcfg)
    plain = ShardPacker(shards, C.DataConfig(kind="shards", shard_dir=str(tmp_path / "s"), seq_len=32, batch_size=3, seed=5))
    b, p = packer.batch(1), plain.batch(1)
    assert torch.equal(b.tokens, p.tokens) and p.loss_mask is None and b.loss_mask.shape == b.targets.shape
    # every target's mask value is its token's own flag: look the tokens up again by walking the packer's stream
    seq, _, keep = packer.row(3)
    assert keep.shape == seq.shape
    kept_classes = {"assistant": None, **SF.LOSS_SPAN_KEEP}[mode]
    state = packer.loss_spans_state
    assert state["mode"] == mode and (mode == "assistant" or sum(state["class_tokens"].values()) == shards.n_tokens)
    if kept_classes is not None and 1 not in kept_classes:
        assert int((~b.loss_mask).sum()) > 0
    # the trainer scores only kept targets
    from gdn_hybrid_architecture_ideas_b200.train.trainer import Trainer, _scored

    cfg = C.TrainConfig(model=C.tiny_control_config(), data=dcfg, steps=2, seed=1)
    cfg.metrics_jsonl, cfg.log_every, cfg.device, cfg.head_impl = False, 0, "cpu", "chunked"
    t = Trainer(cfg, None)
    batch = t.batch_at(0)
    n, _ = t._global_counts(batch)
    assert n == int((batch.target_valid & batch.loss_mask).sum()) < int(batch.target_valid.sum())
    m = t.train_step()
    assert m["n_targets"] == n and t.data_state()["loss_mask"] == mode
    with torch.no_grad():      # the loss is the mean over the kept targets only
        logits = t.model(batch.tokens, batch.doc_ids).logits.float()
    assert _scored(batch).dtype == torch.bool


def test_reference_layout_reads_like_the_reference(reference, tmp_path):
    """A set written by the reference's writer: same documents, flags, classes and fingerprint through this reader."""
    import ced.data.shard_format as RSF

    docs = _docs(3)
    w = RSF.ShardWriter(tmp_path / "r", token_dtype="uint16", loss_spans=True)
    for ids, gen, spans, chat in docs:
        w.add_arrays(ids.astype(np.int64), np.full(len(ids), 3, dtype=np.uint8), generated=gen, chat=chat, source="web" if not chat else "chat", spans=spans)
    w.close()
    mine, theirs = SF.open_shards([tmp_path / "r"]), RSF.ShardSet(tmp_path / "r")
    assert isinstance(mine, SF.ReferenceLayoutSet) and len(mine) == theirs.n_docs and mine.fingerprint() == theirs.fingerprint()
    for i, (ids, gen, spans, chat) in enumerate(docs):
        lo, hi = int(mine.starts[i]), int(mine.ends[i])
        assert np.array_equal(mine.doc(i), ids) and np.array_equal(mine.side("generated")[lo:hi], gen) and np.array_equal(mine.side("loss_spans")[lo:hi], spans)
    assert mine.byte_lens.tolist() == [3 * len(d[0]) for d in docs]
    got = SF.check_loss_spans(mine, "spans_head_tail")
    want = RSF.check_loss_spans(theirs, "spans_head_tail")["parts"][0]
    assert got["class_tokens"] == want["class_tokens"] and got["blake2b"] == want["blake2b"]
    packer = ShardPacker(mine, C.DataConfig(kind="shards", shard_dir=str(tmp_path / "r"), seq_len=24, batch_size=2, seed=1, loss_mask="spans_mask"))
    assert packer.batch(0).loss_mask is not None


def test_check_names_a_broken_set(tmp_path):
    shards = _write_own(tmp_path / "s", _docs(4))
    raw = np.memmap(tmp_path / "s" / "loss_spans.bin", dtype=np.uint8, mode="r+")
    raw[int(shards.starts[1]) + 3] = 2          # a tool-content class inside a document that is not chat
    raw.flush()
    with pytest.raises(ValueError, match="outside a chat document"):
        SF.check_loss_spans(SF.open_shards([tmp_path / "s"]), "spans_full")
    with pytest.raises(ValueError, match="none"):
        plain = tmp_path / "p"
        with SF.ShardWriter(plain, 50) as w:
            w.add_document(np.arange(40))
        SF.check_loss_spans(SF.open_shards([plain]), "assistant")


def test_chat_whole_keeps_chat_documents_off_the_row_boundaries(tmp_path):
    """With data.chat_whole no chat document of at most a row is cut by a row boundary, every token is still used once per
    epoch, a filler's tail follows the chat document it made room for, and without chat documents nothing changes."""
    docs = _docs(7, n=60)
    shards = _write_own(tmp_path / "s", docs)
    L = 63                                             # rows of 64 tokens; documents are 20..59 tokens
    mk = lambda whole: ShardPacker(shards, C.DataConfig(kind="shards", shard_dir=str(tmp_path / "s"), seq_len=L, batch_size=2, seed=3, chat_whole=whole))
    whole, plain = mk(True), mk(False)
    assert whole.rows_per_epoch == plain.rows_per_epoch
    whole._load_epoch(0)
    W = whole.row_tokens
    chat = np.asarray(shards.doc_chat).astype(bool)
    cuts = 0
    for d, o, n, start in zip(whole._seg_doc, whole._seg_off, whole._seg_len, whole._cum[:-1]):
        if chat[d]:
            assert o == 0 and n == len(shards.doc(int(d)))               # a chat document is one segment
            cuts += int(start // W != (start + n - 1) // W)
    assert cuts == whole.chat_cut <= 1                                   # at most the epoch's last chat document, with no filler left
    plain._load_epoch(0)
    plain_cuts = sum(int(chat[d]) and int(s // W != (s + n - 1) // W) for d, n, s in zip(plain._seg_doc, plain._seg_len, plain._cum[:-1]))
    assert plain_cuts > 3                                                # the plain stream does cut them: the option has work to do
    # every token of the set exactly once per epoch, in some order of pieces
    pieces = sorted((int(d), int(o), int(n)) for d, o, n in zip(whole._seg_doc, whole._seg_off, whole._seg_len))
    covered = {}
    for d, o, n in pieces:
        assert covered.get(d, 0) == o
        covered[d] = o + n
    assert covered == {i: len(shards.doc(i)) for i in range(len(docs))}
    # rows carry the same tokens the segments name, with document ids restarting at each piece
    seq, ids, _ = whole.row(2)
    lo = 2 * W
    k = int(np.searchsorted(whole._cum, lo, side="right") - 1)
    d, o = int(whole._seg_doc[k]), int(whole._seg_off[k]) + lo - int(whole._cum[k])
    take = min(int(whole._seg_off[k] + whole._seg_len[k]) - o, W)
    assert np.array_equal(seq[:take], shards.doc(d)[o:o + take]) and len(seq) == W and ids[0] == 0
    assert torch.equal(whole.rows(0, 3).tokens, whole.rows(0, 3).tokens)
    # no chat document in the set: chat_whole changes nothing
    nochat = [(ids_, g * 0, s * 0, False) for ids_, g, s, _ in docs]
    sh2 = _write_own(tmp_path / "n", nochat)
    a = ShardPacker(sh2, C.DataConfig(kind="shards", shard_dir=str(tmp_path / "n"), seq_len=L, batch_size=2, seed=3, chat_whole=True))
    b = ShardPacker(sh2, C.DataConfig(kind="shards", shard_dir=str(tmp_path / "n"), seq_len=L, batch_size=2, seed=3))
    assert torch.equal(a.batch(1).tokens, b.batch(1).tokens)


def test_build_shards_script_text_and_chat(tmp_path):
    """The shard builder: plain documents with byte counts and a held-out split, chat conversations with generated flags and
    loss-span classes that pass the set's invariants and train under the assistant mask."""
    import gzip
    import subprocess
    import sys
    from pathlib import Path

    root = Path(__file__).resolve().parent.parent
    docs = tmp_path / "docs.jsonl"
    docs.write_text("".join(json.dumps({"text": f"Document {i} says hello to the reader. " * (3 + i % 4)}) + "\n" for i in range(12)))
    r = subprocess.run([sys.executable, str(root / "scripts/build_shards.py"), "--out", str(tmp_path / "train"), "--tokenizer", "bytes", "--input", str(docs),
                        "--holdout-every", "4", "--holdout-out", str(tmp_path / "held")], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stderr[-2000:]
    rep = json.loads(r.stdout.strip().splitlines()[-1])
    assert rep["documents"] == {"train": 9, "held": 3, "short": 0} and rep["train"]["documents"] == 9
    train = SF.open_shards([tmp_path / "train"])
    first = "Document 0 says hello to the reader. " * 3
    assert bytes(train.doc(0).astype(np.uint8).tolist()).decode() == first and train.n_tokens == rep["train"]["tokens"]
    with gzip.open(tmp_path / "held" / "docs.jsonl.gz", "rt") as f:
        held = [json.loads(x) for x in f]
    assert len(held) == 3 and held[0]["text"].startswith("Document 3 ")
    # chat conversations
    conv = {"messages": [{"role": "system", "content": "You are terse."}, {"role": "user", "content": "List the files."},
                         {"role": "assistant", "content": "Looking.", "tool_calls": [{"name": "ls", "arguments": {"path": "."}}]},
                         {"role": "tool", "content": "a.txt\n" * 40}, {"role": "assistant", "content": "Forty copies of a.txt."}]}
    chat = tmp_path / "chat.jsonl"
    chat.write_text("".join(json.dumps(conv) + "\n" for _ in range(6)))
    r = subprocess.run([sys.executable, str(root / "scripts/build_shards.py"), "--out", str(tmp_path / "chat"), "--tokenizer", "bytes", "--input", str(chat), "--chat"],
                       capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stderr[-2000:]
    s = SF.open_shards([tmp_path / "chat"])
    assert bool(np.asarray(s.doc_chat).all()) and s.vocab_size == 256 + 11
    a, b = int(s.starts[0]), int(s.ends[0])
    gen, cls = np.asarray(s.side("generated")[a:b]), np.asarray(s.side("loss_spans")[a:b])
    toks = np.asarray(s.doc(0))
    text_of = lambda mask: bytes(int(t) for t in toks[mask] if t < 256).decode()
    assert "Looking." in text_of(gen == 1) and "Forty copies" in text_of(gen == 1) and "List the files" not in text_of(gen == 1)
    assert set(np.unique(cls)) == {0, 1, 2, 3} and not bool((cls[gen == 1] > 0).any())
    assert "a.txt" in text_of(cls == 1) and "a.txt" in text_of(cls == 2) and "You are terse" in text_of(cls == 3)
    state = SF.check_loss_spans(s, "assistant")
    assert state["mode"] == "assistant"
    packer = ShardPacker(s, C.DataConfig(kind="shards", shard_dir=str(tmp_path / "chat"), seq_len=64, batch_size=2, seed=1, loss_mask="assistant", chat_whole=True))
    b0 = packer.batch(0)
    assert b0.loss_mask is not None and 0 < int(b0.loss_mask.sum()) < b0.loss_mask.numel()
